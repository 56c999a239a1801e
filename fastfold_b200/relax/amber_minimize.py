"""Restrained energy minimisation of a predicted structure.

Two back ends produce the same result dictionary:

* ``openmm``: Amber99sb force field, hydrogens added, heavy atoms restrained to their predicted positions by a harmonic
  potential, L-BFGS minimisation, repeated while structural violations remain (at most ``max_outer_iterations``
  rounds, the offending residues losing their restraints) - the procedure of fastfold/relax/amber_minimize.py:417-550.
  Used when OpenMM (and pdbfixer, for clean-up) can be imported.
* ``violation``: a self-contained minimiser on the framework's own differentiable structural-violation terms (peptide
  bond lengths and angles, inter-residue clashes, within-residue bounds; models/hub/loss.py) plus the same harmonic
  restraint, optimised with L-BFGS in PyTorch on whatever device the caller picks.  It removes the violations the
  model's loss measures without a molecular-mechanics package, which makes ``--relaxation`` usable on a bare install.
"""
import io
import time
from typing import Any, Dict, Optional, Sequence

import numpy as np
import torch

from ..common import protein, residue_constants as rc
from ..models.hub import loss as L
from . import utils


def openmm_available() -> bool:
    try:
        import openmm  # noqa: F401
        return True
    except ImportError:
        try:
            from simtk import openmm  # noqa: F401
            return True
        except ImportError:
            return False


# ---------------------------------------------------------------------------
# violation features shared by both back ends
# ---------------------------------------------------------------------------
def _atom14_batch(prot: protein.Protein, device):
    from ..data import data_transforms as dt
    feats = {"aatype": torch.tensor(prot.aatype, dtype=torch.long), "all_atom_positions": torch.tensor(prot.atom_positions, dtype=torch.float32),
             "all_atom_mask": torch.tensor(prot.atom_mask, dtype=torch.float32)}
    feats = dt.make_atom14_masks(feats)
    feats = dt.make_atom14_positions(feats)
    feats["residue_index"] = torch.tensor(prot.residue_index, dtype=torch.long)
    feats["seq_mask"] = torch.ones(len(prot.aatype))
    return {k: (v.to(device) if isinstance(v, torch.Tensor) else v) for k, v in feats.items()}


def find_violations(prot: protein.Protein, device="cpu"):
    """Structural violations of a protein: per-residue mask + summary counts (amber_minimize.py:346-414)."""
    batch = _atom14_batch(prot, device)
    v = L.find_structural_violations(batch, batch["atom14_gt_positions"], violation_tolerance_factor=12.0, clash_overlap_tolerance=1.5)
    per_res = v["total_per_residue_violations_mask"].cpu().numpy()
    return {"per_residue_mask": per_res, "num_violations": float(per_res.sum()),
            "bonds_c_n_loss_mean": float(v["between_residues"]["bonds_c_n_loss_mean"]),
            "angles_ca_c_n_loss_mean": float(v["between_residues"]["angles_ca_c_n_loss_mean"]),
            "angles_c_n_ca_loss_mean": float(v["between_residues"]["angles_c_n_ca_loss_mean"]),
            "clashes_mean_loss": float(v["between_residues"]["clashes_mean_loss"])}


# ---------------------------------------------------------------------------
# violation back end
# ---------------------------------------------------------------------------
def _violation_minimize(prot: protein.Protein, stiffness: float, max_iterations: int, tolerance: float, exclude_residues: Sequence[int],
                        device="cpu"):
    batch = _atom14_batch(prot, device)
    ref = batch["atom14_gt_positions"].clone()
    exists = batch["atom14_atom_exists"]
    restrain = exists.clone()
    if len(exclude_residues):
        restrain[list(exclude_residues)] = 0
    x = ref.clone().requires_grad_(True)
    opt = torch.optim.LBFGS([x], max_iter=max_iterations if max_iterations > 0 else 200, tolerance_change=tolerance * 1e-3, history_size=20,
                            line_search_fn="strong_wolfe")
    state = {"e0": None, "e": None}

    def energy():
        v = L.find_structural_violations(batch, x, violation_tolerance_factor=12.0, clash_overlap_tolerance=1.5)
        e_v = L.violation_loss(v, exists)
        e_r = 0.5 * stiffness * ((x - ref) ** 2 * restrain[..., None]).sum() / restrain.sum().clamp(min=1.0)
        return e_v * 100.0 + e_r, e_v

    def closure():
        opt.zero_grad()
        e, e_v = energy()
        e.backward()
        if state["e0"] is None:
            state["e0"] = float(e_v.detach())
        state["e"] = float(e_v.detach())
        return e

    opt.step(closure)
    with torch.no_grad():
        pos14 = x.detach()
        idx = batch["residx_atom37_to_atom14"]
        pos37 = torch.gather(pos14, 1, idx[..., None].expand(-1, -1, 3)) * batch["atom37_atom_exists"][..., None]
    return pos37.cpu().numpy(), state["e0"], state["e"]


# ---------------------------------------------------------------------------
# OpenMM back end
# ---------------------------------------------------------------------------
def _openmm_minimize(pdb_str: str, max_iterations: int, tolerance: float, stiffness: float, restraint_set: str,
                     exclude_residues: Sequence[int], use_gpu: bool):
    try:
        import openmm
        from openmm import app as openmm_app, unit
    except ImportError:
        from simtk import openmm, unit
        from simtk.openmm import app as openmm_app
    ENERGY = unit.kilocalories_per_mole
    LENGTH = unit.angstroms
    pdb = openmm_app.PDBFile(io.StringIO(pdb_str))
    ff = openmm_app.ForceField("amber99sb.xml")
    system = ff.createSystem(pdb.topology, constraints=openmm_app.HBonds)
    if stiffness > 0:
        force = openmm.CustomExternalForce("0.5 * k * ((x-x0)^2 + (y-y0)^2 + (z-z0)^2)")
        force.addGlobalParameter("k", stiffness * ENERGY / (LENGTH ** 2))
        for p in ("x0", "y0", "z0"):
            force.addPerParticleParameter(p)
        skip = set(exclude_residues)
        for i, atom in enumerate(pdb.topology.atoms()):
            if atom.residue.index in skip:
                continue
            heavy = atom.element.name != "hydrogen"
            if (restraint_set == "non_hydrogen" and heavy) or (restraint_set == "c_alpha" and atom.name == "CA"):
                force.addParticle(i, pdb.positions[i])
        system.addForce(force)
    integrator = openmm.LangevinIntegrator(0, 0.01, 0.0)
    platform = openmm.Platform.getPlatformByName("CUDA" if use_gpu else "CPU")
    sim = openmm_app.Simulation(pdb.topology, system, integrator, platform)
    sim.context.setPositions(pdb.positions)
    ret = {}
    st = sim.context.getState(getEnergy=True, getPositions=True)
    ret["einit"] = st.getPotentialEnergy().value_in_unit(ENERGY)
    ret["posinit"] = st.getPositions(asNumpy=True).value_in_unit(LENGTH)
    sim.minimizeEnergy(maxIterations=max_iterations, tolerance=tolerance * ENERGY / LENGTH if hasattr(tolerance, "__float__") else tolerance)
    st = sim.context.getState(getEnergy=True, getPositions=True)
    ret["efinal"] = st.getPotentialEnergy().value_in_unit(ENERGY)
    ret["pos"] = st.getPositions(asNumpy=True).value_in_unit(LENGTH)
    out = io.StringIO()
    openmm_app.PDBFile.writeFile(sim.topology, st.getPositions(), out)
    ret["min_pdb"] = out.getvalue()
    return ret


def _clean_for_openmm(prot: protein.Protein) -> str:
    from . import cleanup
    pdb_str = protein.to_pdb(prot)
    return cleanup.fix_pdb_string(pdb_str)


def will_restrain(atom, rset: str) -> bool:
    """Whether the harmonic position restraint of set ``rset`` (``non_hydrogen`` / ``c_alpha``) applies to an OpenMM atom."""
    if rset == "non_hydrogen":
        return atom.element.name != "hydrogen"
    if rset == "c_alpha":
        return atom.name == "CA"
    raise ValueError("unknown restraint set %r" % rset)


def clean_protein(prot: protein.Protein, checks: bool = True) -> str:
    """PDB text of ``prot`` ready for the force field: the atom mask must be the ideal one for the sequence (every heavy
    atom present), then pdbfixer adds hydrogens / fixes residues (OpenMM back end only)."""
    if checks:
        ideal = protein.ideal_atom_mask(prot)
        utils.assert_equal_nonterminal_atom_types(np.asarray(prot.atom_mask), ideal)
    return _clean_for_openmm(prot)


def get_violation_metrics(prot: protein.Protein, device="cpu") -> Dict[str, Any]:
    """Violations of ``prot`` with the indices of the violating residues (what the outer relaxation loop frees next)."""
    v = find_violations(prot, device)
    idx = np.flatnonzero(v["per_residue_mask"])
    metrics = dict(v)
    metrics.update({"residue_violations": idx, "num_residue_violations": len(idx), "structural_violations": v})
    return metrics


def get_initial_energies(pdb_strs: Sequence[str], stiffness: float = 0.0, restraint_set: str = "non_hydrogen",
                         exclude_residues: Optional[Sequence[int]] = None):
    """Potential energy (kcal/mol) of each ready-to-minimise PDB string before any minimisation step (OpenMM back end)."""
    return [_openmm_minimize(s_, max_iterations=1, tolerance=2.39, stiffness=stiffness, restraint_set=restraint_set,
                             exclude_residues=list(exclude_residues or []), use_gpu=False)["einit"] for s_ in pdb_strs]


# ---------------------------------------------------------------------------
# pipeline
# ---------------------------------------------------------------------------
def run_pipeline(prot: protein.Protein, stiffness: float, use_gpu: bool = False, max_outer_iterations: int = 1, place_hydrogens_every_iteration: bool = True,
                 max_iterations: int = 0, tolerance: float = 2.39, restraint_set: str = "non_hydrogen", max_attempts: int = 100,
                 checks: bool = True, exclude_residues: Optional[Sequence[int]] = None, backend: Optional[str] = None) -> Dict[str, Any]:
    """Minimise, look for violations, free the violating residues, repeat.  Returns ``min_pdb``, energies, the
    per-iteration violation counts and ``opt_time``."""
    backend = backend or ("openmm" if openmm_available() else "violation")
    exclude = set(exclude_residues or [])
    device = "cuda" if (use_gpu and torch.cuda.is_available()) else "cpu"
    t0 = time.time()
    cur = prot
    out: Dict[str, Any] = {"backend": backend}
    violations, iteration = np.inf, 0
    einit = None
    while violations > 0 and iteration < max_outer_iterations:
        if backend == "openmm":
            pdb_str = _clean_for_openmm(cur)
            ret = None
            for attempt in range(max_attempts):
                try:
                    ret = _openmm_minimize(pdb_str, max_iterations, tolerance, stiffness, restraint_set, sorted(exclude), use_gpu)
                    break
                except Exception as e:  # noqa: BLE001 - OpenMM raises plain Exceptions on NaN energies
                    last = e
            if ret is None:
                raise ValueError("Minimization failed after %d attempts: %s" % (max_attempts, last))
            cur = protein.from_pdb_string(ret["min_pdb"])
            e0, e1 = ret["einit"], ret["efinal"]
        else:
            pos37, e0, e1 = _violation_minimize(cur, stiffness, max_iterations, tolerance, sorted(exclude), device)
            cur = protein.Protein(atom_positions=pos37, aatype=cur.aatype, atom_mask=cur.atom_mask, residue_index=cur.residue_index,
                                  b_factors=cur.b_factors, **({"chain_index": cur.chain_index} if hasattr(cur, "chain_index") else {}))
        if einit is None:
            einit = e0
        v = find_violations(cur, device)
        violations = v["num_violations"]
        exclude |= set(np.nonzero(v["per_residue_mask"])[0].tolist())
        out.update({"einit": einit, "efinal": e1, "num_residue_violations": violations, "violations": v, "num_exclusions": len(exclude),
                    "iteration": iteration})
        iteration += 1
    if checks:
        utils.assert_equal_nonterminal_atom_types(cur.atom_mask, prot.atom_mask)
    out["min_pdb"] = protein.to_pdb(cur)
    out["final_protein"] = cur
    out["opt_time"] = time.time() - t0
    out["min_attempts"] = iteration
    return out


def make_atom14_positions(prot):
    """Adds the 14-slot (per-residue-type) view of a structure given as numpy arrays ``aatype [N]``, ``all_atom_positions
    [N, 37, 3]``, ``all_atom_mask [N, 37]``: index maps both ways, existence masks, positions, and the alternative naming
    of the 180-degree-symmetric side chains (fastfold/relax/amber_minimize.py:185-312).  Same code as the training
    transforms, run on tensors and handed back as numpy."""
    from ..data import data_transforms as dt
    t = {k: torch.as_tensor(np.asarray(v)) for k, v in prot.items() if isinstance(v, (np.ndarray, list, tuple)) or torch.is_tensor(v)}
    t["aatype"] = t["aatype"].long()
    t["all_atom_positions"] = t["all_atom_positions"].float()
    t["all_atom_mask"] = t["all_atom_mask"].float()
    t = dt.make_atom14_positions(dt.make_atom14_masks(t))
    for k, v in t.items():
        prot[k] = v.numpy()
    return prot
