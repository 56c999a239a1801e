"""Relaxation stage: PDB helpers and the self-contained violation minimiser (OpenMM is not required)."""
import numpy as np
import pytest
import torch

from fastfold_b200.common import protein, residue_constants as rc
from fastfold_b200.relax import AmberRelaxation, amber_minimize, utils


def _helix(n=12, seed=0):
    """An ideal-ish poly-alanine backbone (+CB) built from literature coordinates along a helix axis."""
    rng = np.random.default_rng(seed)
    aatype = np.full(n, rc.restype_order["A"])
    pos = np.zeros((n, 37, 3), np.float32)
    mask = np.zeros((n, 37), np.float32)
    lit = {a[0]: np.array(a[2]) for a in rc.rigid_group_atom_positions["ALA"]}
    for i in range(n):
        ang = np.deg2rad(100.0 * i)
        rot = np.array([[np.cos(ang), -np.sin(ang), 0], [np.sin(ang), np.cos(ang), 0], [0, 0, 1]], np.float32)
        origin = np.array([2.3 * np.cos(ang), 2.3 * np.sin(ang), 1.5 * i], np.float32)
        for name in ("N", "CA", "C", "O", "CB"):
            pos[i, rc.atom_order[name]] = rot @ lit[name] + origin
            mask[i, rc.atom_order[name]] = 1
    return protein.Protein(atom_positions=pos, aatype=aatype, atom_mask=mask, residue_index=np.arange(1, n + 1), b_factors=np.ones((n, 37), np.float32) * 50)


def test_pdb_helpers_round_trip():
    prot = _helix()
    pdb = protein.to_pdb(prot)
    shifted = utils.overwrite_pdb_coordinates(pdb, prot.atom_positions + 1.0)
    back = protein.from_pdb_string(shifted)
    assert np.allclose(back.atom_positions[prot.atom_mask > 0], prot.atom_positions[prot.atom_mask > 0] + 1.0, atol=2e-3)
    b = utils.overwrite_b_factors(pdb, np.full((len(prot.aatype), 37), 12.5))
    assert " 12.50" in b.splitlines()[1]
    with pytest.raises(ValueError):
        utils.overwrite_b_factors(pdb, np.zeros((len(prot.aatype), 3)))


def test_violation_minimiser_reduces_violation_energy():
    prot = _helix()
    res = amber_minimize.run_pipeline(prot, stiffness=1.0, max_iterations=30, max_outer_iterations=2, backend="violation")
    assert res["backend"] == "violation"
    assert res["efinal"] <= res["einit"] + 1e-6
    assert "ATOM" in res["min_pdb"]
    # atoms stay near their start (restraint) and the set of atoms is unchanged
    moved = np.abs(res["final_protein"].atom_positions - prot.atom_positions)[prot.atom_mask > 0].max()
    assert moved < 5.0


def test_amber_relaxation_api():
    prot = _helix(8)
    relaxer = AmberRelaxation(max_iterations=10, tolerance=2.39, stiffness=10.0, exclude_residues=[], max_outer_iterations=1, use_gpu=False,
                              backend="violation")
    pdb, debug, viol = relaxer.process(prot=prot)
    assert pdb.startswith(("ATOM", "MODEL", "PARENT", "REMARK")) and viol.shape == (8,)
    assert {"initial_energy", "final_energy", "rmsd", "backend"} <= set(debug)


def test_openmm_back_end_control_flow_against_a_fake():
    """OpenMM is not installed on the test machines: a stand-in with the same call surface checks that the back end
    cleans the structure, restrains exactly the heavy atoms of the non-excluded residues, reports energies in order and
    returns a structure with the same atoms."""
    from fakes import fake_openmm
    names = fake_openmm.install()
    try:
        assert amber_minimize.openmm_available()
        prot = _helix(6)
        moved = protein.Protein(atom_positions=prot.atom_positions + 0.0, aatype=prot.aatype, atom_mask=prot.atom_mask,
                                residue_index=prot.residue_index, b_factors=prot.b_factors)
        res = amber_minimize.run_pipeline(moved, stiffness=10.0, max_iterations=5, max_outer_iterations=1, backend="openmm",
                                          exclude_residues=[2], checks=True)
        assert res["backend"] == "openmm" and res["efinal"] <= res["einit"] and "ATOM" in res["min_pdb"]
        fixer = fake_openmm.PDBFixer.instances[-1]
        assert fixer.steps == ["findNonstandardResidues", "replaceNonstandardResidues", "removeHeterogens", "findMissingResidues",
                               "findMissingAtoms", "addMissingAtoms", "addMissingHydrogens"]
        force = fake_openmm.CustomExternalForce.instances[-1]
        n_heavy_per_res = int(prot.atom_mask[0].sum())
        assert len(force.particles) == n_heavy_per_res * 5                      # residue 2 is free
        assert force.per_particle == ["x0", "y0", "z0"] and "k" in force.globals
        assert fake_openmm.Platform.requested[-1] == "CPU"
        back = res["final_protein"]
        assert np.allclose(back.atom_mask, prot.atom_mask)
        assert amber_minimize.get_initial_energies([protein.to_pdb(prot)], stiffness=10.0)[0] == pytest.approx(100.0)
        relaxer = AmberRelaxation(max_iterations=5, tolerance=2.39, stiffness=10.0, exclude_residues=[], max_outer_iterations=1,
                                  use_gpu=False, backend="openmm")
        pdb, debug, viol = relaxer.process(prot=prot)
        assert debug["backend"] == "openmm" and viol.shape == (6,)
    finally:
        fake_openmm.uninstall(names)
