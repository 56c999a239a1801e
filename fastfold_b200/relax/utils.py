"""PDB text helpers of the relaxation stage (fastfold/relax/utils.py:1-111)."""
import io

import numpy as np

from ..common import residue_constants as rc


def _atom_lines(pdb_str):
    for i, line in enumerate(pdb_str.splitlines()):
        if line.startswith(("ATOM", "HETATM")):
            yield i, line


def overwrite_pdb_coordinates(pdb_str: str, pos) -> str:
    """Replaces the coordinates of a PDB string by ``pos`` ([num_res, 37, 3] in atom37 order, or [num_atoms, 3] in file order)."""
    pos = np.asarray(pos)
    lines = pdb_str.splitlines()
    flat = pos.reshape(-1, 3) if pos.ndim == 2 else None
    res_keys, k = {}, 0
    for i, line in _atom_lines(pdb_str):
        if flat is not None:
            xyz = flat[k]
            k += 1
        else:
            key = (line[21], line[22:27])
            if key not in res_keys:
                res_keys[key] = len(res_keys)
            xyz = pos[res_keys[key], rc.atom_order[line[12:16].strip()]]
        lines[i] = "%s%8.3f%8.3f%8.3f%s" % (line[:30], xyz[0], xyz[1], xyz[2], line[54:])
    return "\n".join(lines) + "\n"


def overwrite_b_factors(pdb_str: str, bfactors: np.ndarray) -> str:
    """Per-residue B-factors ([num_res, 37], column of CA is used) written over every atom line."""
    bfactors = np.asarray(bfactors)
    if bfactors.shape[-1] != rc.atom_type_num:
        raise ValueError("Invalid final dimension size for bfactors: %d." % bfactors.shape[-1])
    lines = pdb_str.splitlines()
    res_keys = {}
    for i, line in _atom_lines(pdb_str):
        key = (line[21], line[22:27])
        if key not in res_keys:
            res_keys[key] = len(res_keys)
        b = bfactors[res_keys[key], rc.atom_order["CA"]]
        lines[i] = "%s%6.2f%s" % (line[:60], b, line[66:])
    return "\n".join(lines) + "\n"


def assert_equal_nonterminal_atom_types(atom_mask: np.ndarray, ref_atom_mask: np.ndarray):
    """Checks that pre- and post-minimisation proteins have the same atoms, except the terminal oxygen OXT."""
    oxt = rc.atom_order["OXT"]
    keep = np.ones_like(atom_mask, dtype=bool)
    keep[..., oxt] = False
    np.testing.assert_almost_equal(ref_atom_mask[keep], atom_mask[keep])


def mask_mean_np(mask, value, axis=None, drop_mask_channel=False, eps=1e-10):
    """Mean of ``value`` over ``axis`` (all axes when None) counting only entries where ``mask`` is set; mask axes of
    extent 1 broadcast."""
    mask, value = np.asarray(mask), np.asarray(value)
    if drop_mask_channel:
        mask = mask[..., 0]
    assert mask.ndim == value.ndim
    axes = list(range(mask.ndim)) if axis is None else ([axis] if np.isscalar(axis) else list(axis))
    broadcast = 1.0
    for a in axes:
        if mask.shape[a] == 1:
            broadcast *= value.shape[a]
        else:
            assert mask.shape[a] == value.shape[a]
    axes = tuple(axes)
    return np.sum(mask * value, axis=axes) / (np.sum(mask, axis=axes) * broadcast + eps)

