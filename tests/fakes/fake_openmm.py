"""A stand-in for the parts of OpenMM / pdbfixer that ``relax/amber_minimize.py`` and ``relax/cleanup.py`` call, so that the
OpenMM back end's control flow (clean-up, restraint selection, retries, energies, PDB round trip) runs in tests on a
machine without OpenMM.  The "force field" is the harmonic restraint alone: minimisation moves every restrained atom
back to its reference position.  Installed into ``sys.modules`` by ``install()``; nothing outside tests imports it."""
import io
import sys
import types

import numpy as np


class _Unit:
    def __init__(self, name):
        self.name = name

    def __mul__(self, o):
        return _Quantity(o, self) if not isinstance(o, (_Unit, _Quantity)) else _Unit("%s*%s" % (self.name, getattr(o, "name", "q")))

    __rmul__ = __mul__

    def __truediv__(self, o):
        return _Unit("%s/%s" % (self.name, getattr(o, "name", o)))

    def __pow__(self, p):
        return _Unit("%s^%s" % (self.name, p))


class _Quantity:
    def __init__(self, value, unit):
        self.value, self.unit = value, unit

    def value_in_unit(self, unit):
        return self.value

    def __truediv__(self, o):
        return _Quantity(self.value, self.unit)

    def __mul__(self, o):
        return _Quantity(self.value, self.unit)

    __rmul__ = __mul__

    def __float__(self):
        return float(self.value)


class _Element:
    def __init__(self, symbol):
        self.symbol = symbol
        self.name = {"H": "hydrogen", "C": "carbon", "N": "nitrogen", "O": "oxygen", "S": "sulfur"}.get(symbol, symbol.lower())


class _Residue:
    def __init__(self, index, name, chain, number):
        self.index, self.name, self.chain, self.number = index, name, chain, number


class _Atom:
    def __init__(self, name, element, residue, line):
        self.name, self.element, self.residue, self.line = name, element, residue, line


class _Topology:
    def __init__(self, atom_list):
        self._atoms = atom_list

    def atoms(self):
        return iter(self._atoms)


def _parse(pdb_text):
    atoms, positions, residues = [], [], {}
    for line in pdb_text.splitlines():
        if not line.startswith(("ATOM", "HETATM")):
            continue
        key = (line[21], line[22:27])
        if key not in residues:
            residues[key] = _Residue(len(residues), line[17:20], line[21], line[22:27])
        symbol = line[76:78].strip() or line[12:16].strip()[0]
        atoms.append(_Atom(line[12:16].strip(), _Element(symbol), residues[key], line))
        positions.append([float(line[30:38]), float(line[38:46]), float(line[46:54])])
    return _Topology(atoms), np.array(positions, dtype=np.float64)


class PDBFile:
    def __init__(self, file):
        text = file.read() if hasattr(file, "read") else open(file).read()
        self.topology, self.positions = _parse(text)

    @staticmethod
    def writeFile(topology, positions, file, keepIds=False):
        pos = np.asarray(positions.value_in_unit(None) if isinstance(positions, _Quantity) else positions)
        for atom, xyz in zip(topology.atoms(), pos):
            file.write("%s%8.3f%8.3f%8.3f%s\n" % (atom.line[:30], xyz[0], xyz[1], xyz[2], atom.line[54:]))
        file.write("END\n")


class _System:
    def __init__(self):
        self.forces = []

    def addForce(self, f):
        self.forces.append(f)


class ForceField:
    calls = []

    def __init__(self, *files):
        self.files = files

    def createSystem(self, topology, constraints=None):
        ForceField.calls.append((self.files, constraints))
        return _System()


class CustomExternalForce:
    instances = []

    def __init__(self, expression):
        self.expression, self.globals, self.per_particle, self.particles = expression, {}, [], []
        CustomExternalForce.instances.append(self)

    def addGlobalParameter(self, name, value):
        self.globals[name] = value

    def addPerParticleParameter(self, name):
        self.per_particle.append(name)

    def addParticle(self, index, params):
        self.particles.append((index, np.asarray(params, dtype=np.float64)))


class LangevinIntegrator:
    def __init__(self, *a):
        pass


class Platform:
    requested = []

    @staticmethod
    def getPlatformByName(name):
        Platform.requested.append(name)
        return name


class _State:
    def __init__(self, energy, positions):
        self._e, self._p = energy, positions

    def getPotentialEnergy(self):
        return _Quantity(self._e, None)

    def getPositions(self, asNumpy=False):
        return _Quantity(self._p.copy(), None)


class _Context:
    def __init__(self, system):
        self.system, self.positions = system, None

    def setPositions(self, positions):
        self.positions = np.array(positions, dtype=np.float64)

    def _energy(self):
        e = 100.0          # a constant standing in for the molecular-mechanics terms
        for f in self.system.forces:
            k = float(f.globals["k"].value if isinstance(f.globals["k"], _Quantity) else f.globals["k"])
            for i, ref in f.particles:
                e += 0.5 * k * float(np.sum((self.positions[i] - ref) ** 2))
        return e

    def getState(self, getEnergy=False, getPositions=False):
        return _State(self._energy(), self.positions)


class Simulation:
    def __init__(self, topology, system, integrator, platform):
        self.topology, self.system, self.context = topology, system, _Context(system)

    def minimizeEnergy(self, maxIterations=0, tolerance=None):
        for f in self.system.forces:
            for i, ref in f.particles:
                self.context.positions[i] = ref


class PDBFixer:
    instances = []

    def __init__(self, pdbfile=None):
        self.topology, self.positions = _parse(pdbfile.read())
        self.nonstandardResidues, self.missingAtoms, self.missingTerminals, self.steps = [], {}, {}, []
        PDBFixer.instances.append(self)

    def _step(self, name):
        self.steps.append(name)

    def findNonstandardResidues(self): self._step("findNonstandardResidues")
    def replaceNonstandardResidues(self): self._step("replaceNonstandardResidues")
    def removeHeterogens(self, keepWater=False): self._step("removeHeterogens")
    def findMissingResidues(self): self._step("findMissingResidues")
    def findMissingAtoms(self): self._step("findMissingAtoms")
    def addMissingAtoms(self, seed=None): self._step("addMissingAtoms")
    def addMissingHydrogens(self, pH=7.0): self._step("addMissingHydrogens")


def install():
    """Puts ``openmm``, ``openmm.app``, ``openmm.unit`` and ``pdbfixer`` into ``sys.modules``; returns the names added."""
    openmm = types.ModuleType("openmm")
    app = types.ModuleType("openmm.app")
    unit = types.ModuleType("openmm.unit")
    unit.kilocalories_per_mole, unit.angstroms = _Unit("kcal/mol"), _Unit("A")
    app.PDBFile, app.ForceField, app.Simulation, app.HBonds = PDBFile, ForceField, Simulation, "HBonds"
    openmm.app, openmm.unit = app, unit
    openmm.CustomExternalForce, openmm.LangevinIntegrator, openmm.Platform = CustomExternalForce, LangevinIntegrator, Platform
    fixer = types.ModuleType("pdbfixer")
    fixer.PDBFixer = PDBFixer
    added = {"openmm": openmm, "openmm.app": app, "openmm.unit": unit, "pdbfixer": fixer}
    sys.modules.update(added)
    for cls in (ForceField, CustomExternalForce, Platform, PDBFixer):
        for attr in ("calls", "instances", "requested"):
            if hasattr(cls, attr):
                getattr(cls, attr).clear()
    return list(added)


def uninstall(names):
    for n in names:
        sys.modules.pop(n, None)
