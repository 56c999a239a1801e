"""Stand-in for ``Bio.PDB.Structure``: the small part of BioPython's structure hierarchy (structure > model > chain >
residue > atom) that the reference package's mmCIF code walks."""


class Atom:
    def __init__(self, name, coord, occupancy, element):
        self.name, self.coord, self.occupancy, self.element = name, coord, occupancy, element

    def get_name(self):
        return self.name

    def get_coord(self):
        return self.coord


class Residue:
    def __init__(self, residue_id, resname):
        self.id, self.resname, self._atoms = residue_id, resname, {}

    def add(self, atom):
        old = self._atoms.get(atom.name)
        if old is None or atom.occupancy > old.occupancy:          # alternative locations: the most occupied one wins
            self._atoms[atom.name] = atom

    def get_atoms(self):
        return iter(self._atoms.values())

    def get_resname(self):
        return self.resname

    def get_id(self):
        return self.id


class Chain:
    def __init__(self, chain_id):
        self.id, self._residues = chain_id, {}

    def residue(self, residue_id, resname):
        if residue_id not in self._residues:
            self._residues[residue_id] = Residue(residue_id, resname)
        return self._residues[residue_id]

    def __getitem__(self, residue_id):
        return self._residues[residue_id]

    def __contains__(self, residue_id):
        return residue_id in self._residues

    def get_residues(self):
        return iter(self._residues.values())

    def __iter__(self):
        return self.get_residues()


class Model:
    def __init__(self, model_id):
        self.id, self._chains = model_id, {}

    def chain(self, chain_id):
        if chain_id not in self._chains:
            self._chains[chain_id] = Chain(chain_id)
        return self._chains[chain_id]

    def __getitem__(self, chain_id):
        return self._chains[chain_id]

    def get_chains(self):
        return iter(self._chains.values())

    def __iter__(self):
        return self.get_chains()


class Structure:
    def __init__(self, structure_id):
        self.id, self._models = structure_id, {}

    def model(self, model_id):
        if model_id not in self._models:
            self._models[model_id] = Model(model_id)
        return self._models[model_id]

    def get_models(self):
        return iter(self._models.values())

    def get_chains(self):
        for m in self._models.values():
            yield from m.get_chains()

    def __iter__(self):
        return self.get_models()
