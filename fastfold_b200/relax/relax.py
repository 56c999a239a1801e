"""``AmberRelaxation``: the relaxation stage of the inference script (fastfold/relax/relax.py:24-92)."""
from typing import Any, Dict, Sequence, Tuple

import numpy as np

from ..common import protein
from . import amber_minimize, utils


class AmberRelaxation:
    def __init__(self, *, max_iterations: int, tolerance: float, stiffness: float, exclude_residues: Sequence[int], max_outer_iterations: int,
                 use_gpu: bool, backend=None):
        """``max_iterations``: L-BFGS iteration cap (0: none); ``tolerance``: energy tolerance (kcal/mol); ``stiffness``:
        restraint spring constant (kcal/mol/A^2); ``exclude_residues``: residues without restraints;
        ``max_outer_iterations``: violation-informed repetitions (1 = the non-iterative CASP14 procedure);
        ``backend``: ``"openmm"``, ``"violation"`` or None (OpenMM when importable)."""
        self._max_iterations = max_iterations
        self._tolerance = tolerance
        self._stiffness = stiffness
        self._exclude_residues = exclude_residues
        self._max_outer_iterations = max_outer_iterations
        self._use_gpu = use_gpu
        self._backend = backend

    def process(self, *, prot: protein.Protein) -> Tuple[str, Dict[str, Any], np.ndarray]:
        """Returns the relaxed PDB string, debug data and the per-residue violation mask."""
        out = amber_minimize.run_pipeline(prot=prot, max_iterations=self._max_iterations, tolerance=self._tolerance, stiffness=self._stiffness,
                                          exclude_residues=self._exclude_residues, max_outer_iterations=self._max_outer_iterations,
                                          use_gpu=self._use_gpu, backend=self._backend)
        final = out["final_protein"]
        rmsd = float(np.sqrt(np.sum((prot.atom_positions - final.atom_positions) ** 2 * prot.atom_mask[..., None]) / max(prot.atom_mask.sum(), 1)))
        debug = {"initial_energy": out["einit"], "final_energy": out["efinal"], "attempts": out["min_attempts"], "rmsd": rmsd,
                 "backend": out["backend"], "opt_time": out["opt_time"]}
        min_pdb = utils.overwrite_b_factors(out["min_pdb"], prot.b_factors)
        violations = out["violations"]["per_residue_mask"]
        return min_pdb, debug, violations
