"""Amino-acid chemistry tables used by the structure module, the feature builders, the losses and PDB output.

The numbers (atom names per residue, idealised rigid-group coordinates, chi-angle definitions, van der Waals
radii, peptide-bond geometry) are physical constants; they are stored as plain data in
``common/data/chemistry.json`` and exposed here as module attributes (dicts, lists, numpy arrays), under the names
AlphaFold-derived code expects (``restype_order``, ``atom_types``, ``restype_atom14_to_rigid_group`` ...).
No dm-tree or network access is needed, unlike the reference's module (fastfold/common/residue_constants.py:25,
:460-463), which downloads ``stereo_chemical_props.txt`` to build its within-residue bond bounds; here those bounds
are derived from the idealised coordinates themselves (see ``make_atom14_dists_bounds``).
"""
import collections
import functools
import json
import os

import numpy as np

_DATA = os.path.join(os.path.dirname(os.path.abspath(__file__)), "data", "chemistry.json")
_SKIP = {"atom", "atom_i", "ca_ca", "chi_group", "chi_group_i", "res_name"}


def _decode(v):
    if isinstance(v, dict):
        if v.get("__nd__"):
            return np.array(v["data"], dtype=np.dtype(v["dtype"])).reshape(v["shape"])
        if "__dict__" in v:
            return {(_freeze(_decode(k))): _decode(x) for k, x in v["__dict__"]}
        if "__seq__" in v:
            items = [_decode(x) for x in v["items"]]
            return tuple(items) if v["__seq__"] == "tuple" else items
    return v


def _freeze(k):
    return tuple(_freeze(x) for x in k) if isinstance(k, list) else k


with open(_DATA) as _fh:
    for _name, _val in json.load(_fh).items():
        if _name not in _SKIP:
            globals()[_name] = _decode(_val)
del _fh, _name, _val

# lower-case aliases of the index tables
restype_atom14_to_atom37 = RESTYPE_ATOM14_TO_ATOM37
restype_atom37_to_atom14 = RESTYPE_ATOM37_TO_ATOM14
restype_atom14_is_ambiguous = RESTYPE_ATOM14_IS_AMBIGUOUS
restype_rigidgroup_base_atom37_idx = RESTYPE_RIGIDGROUP_BASE_ATOM37_IDX
restype_rigidgroup_mask = RESTYPE_RIGIDGROUP_MASK
renaming_matrices = RENAMING_MATRICES
chi_atom_indices = CHI_ATOM_INDICES

# Distance from one CA to next CA [trans configuration: omega = 180].
ca_ca = 3.80209737096

restype_order = dict(restype_order)
restype_num = len(restypes)                # 20
unk_restype_index = restype_num            # catch-all index for unknown restypes
atom_type_num = len(atom_types)            # 37


def sequence_to_onehot(sequence, mapping, map_unknown_to_x=False):
    """One-hot encoding of an amino-acid string with the given letter -> index mapping."""
    num_entries = max(mapping.values()) + 1
    if sorted(set(mapping.values())) != list(range(num_entries)):
        raise ValueError("The mapping must have values from 0 to num_unique_aas-1 without any gaps.")
    one_hot = np.zeros((len(sequence), num_entries), dtype=np.int32)
    for i, aa in enumerate(sequence):
        if map_unknown_to_x:
            if aa.isalpha() and aa.isupper():
                idx = mapping.get(aa, mapping["X"])
            else:
                raise ValueError("Invalid character in the sequence: %s" % aa)
        else:
            idx = mapping[aa]
        one_hot[i, idx] = 1
    return one_hot


def aatype_to_str_sequence(aatype):
    return "".join(restypes_with_x[int(a)] for a in aatype)


def chi_angle_atom(atom_index):
    """One-hot [21, 4, 14] of the atom14 slot of the ``atom_index``-th atom defining each chi angle."""
    out = np.zeros((restype_num + 1, 4, 14), dtype=np.float32)
    for r, letter in enumerate(restypes):
        res = restype_1to3[letter]
        names14 = restype_name_to_atom14_names[res]
        for c, atoms in enumerate(chi_angles_atoms[res]):
            out[r, c, names14.index(atoms[atom_index])] = 1.0
    return out


@functools.lru_cache(maxsize=None)
def _ideal_atom14_coordinates():
    """Idealised atom14 coordinates of every residue type with all torsions at their literature zero (frames composed)."""
    coords = np.zeros((restype_num + 1, 14, 3), dtype=np.float64)
    frames = np.asarray(restype_rigid_group_default_frame, dtype=np.float64)     # [21, 8, 4, 4]
    for r in range(restype_num):
        # compose group frames to the backbone frame: chi2..chi4 chain onto the previous chi frame
        to_bb = [None] * 8
        for g in range(8):
            f = frames[r, g]
            if g >= 5:
                f = to_bb[g - 1] @ f
            to_bb[g] = f
        for a in range(14):
            g = int(restype_atom14_to_rigid_group[r, a])
            p = np.append(restype_atom14_rigid_group_positions[r, a], 1.0)
            coords[r, a] = (to_bb[g] @ p)[:3]
    return coords


Bond = collections.namedtuple("Bond", ["atom1_name", "atom2_name", "length", "stddev"])
BondAngle = collections.namedtuple("BondAngle", ["atom1_name", "atom2_name", "atom3name", "angle_rad", "stddev"])


@functools.lru_cache(maxsize=None)
def load_stereo_chemical_props():
    """``(residue_bonds, residue_virtual_bonds, residue_bond_angles)`` keyed by three-letter residue name.

    The reference reads these from the stereo_chemical_props.txt table of the AlphaFold distribution
    (fastfold/common/residue_constants.py:404-470).  That file is not shipped here; the same quantities are derived
    from the idealised residue geometry this package already carries (``rigid_group_atom_positions``): two heavy
    atoms closer than 1.95 A are bonded (ideal length = their distance), two bonds sharing an atom define a bond
    angle, and the two outer atoms of an angle a virtual bond whose length follows from the law of cosines.  The
    spreads are nominal (0.02 A for lengths, 0.035 rad for angles), not the per-bond literature values of that file.
    """
    ideal = _ideal_atom14_coordinates()
    bonds, virtual, angles = {}, {}, {}
    for r, letter in enumerate(restypes):
        res = restype_1to3[letter]
        names = [a for a in restype_name_to_atom14_names[res] if a]
        blist = []
        for i in range(len(names)):
            for j in range(i + 1, len(names)):
                d = float(np.linalg.norm(ideal[r, i] - ideal[r, j]))
                if d < 1.95:
                    blist.append(Bond(names[i], names[j], d, 0.02))
        bonds[res] = blist
        alist, vlist = [], []
        for a in range(len(blist)):
            for b in range(a + 1, len(blist)):
                shared = {blist[a].atom1_name, blist[a].atom2_name} & {blist[b].atom1_name, blist[b].atom2_name}
                if len(shared) != 1:
                    continue
                centre = shared.pop()
                end1 = blist[a].atom1_name if blist[a].atom2_name == centre else blist[a].atom2_name
                end3 = blist[b].atom1_name if blist[b].atom2_name == centre else blist[b].atom2_name
                p1, p2, p3 = (ideal[r, names.index(n)] for n in (end1, centre, end3))
                v1, v3 = p1 - p2, p3 - p2
                ang = float(np.arccos(np.clip(np.dot(v1, v3) / (np.linalg.norm(v1) * np.linalg.norm(v3)), -1.0, 1.0)))
                alist.append(BondAngle(end1, centre, end3, ang, 0.035))
                l1, l3 = blist[a].length, blist[b].length
                length = float(np.sqrt(l1 ** 2 + l3 ** 2 - 2 * l1 * l3 * np.cos(ang)))
                dl_outer = 0.5 / length * (2 * l1 * l3 * np.sin(ang))
                dl_1 = 0.5 / length * (2 * l1 - 2 * l3 * np.cos(ang))
                dl_3 = 0.5 / length * (2 * l3 - 2 * l1 * np.cos(ang))
                sd = float(np.sqrt((dl_outer * 0.035) ** 2 + (dl_1 * 0.02) ** 2 + (dl_3 * 0.02) ** 2))
                vlist.append(Bond(end1, end3, length, sd))
        angles[res], virtual[res] = alist, vlist
    return bonds, virtual, angles


def make_atom14_dists_bounds(overlap_tolerance=1.5, bond_length_tolerance_factor=15):
    """Lower / upper bounds and bond-length spread for every atom14 pair inside a residue.

    Non-bonded pairs: lower bound = sum of van der Waals radii - ``overlap_tolerance``, no upper bound.
    Bonded pairs (atoms closer than 1.95 A in the idealised residue; a bond length does not depend on the torsion
    about it): ideal length -/+ ``bond_length_tolerance_factor`` * 0.02 A.
    """
    lower = np.zeros([restype_num + 1, 14, 14], dtype=np.float32)
    upper = np.zeros([restype_num + 1, 14, 14], dtype=np.float32)
    stddev = np.zeros([restype_num + 1, 14, 14], dtype=np.float32)
    ideal = _ideal_atom14_coordinates()
    for r, letter in enumerate(restypes):
        names = restype_name_to_atom14_names[restype_1to3[letter]]
        n = sum(1 for a in names if a)
        for i in range(n):
            for j in range(i + 1, n):
                vdw = van_der_waals_radius[names[i][0]] + van_der_waals_radius[names[j][0]]
                d = float(np.linalg.norm(ideal[r, i] - ideal[r, j]))
                if d < 1.95:
                    sd = 0.02
                    lo, up = d - bond_length_tolerance_factor * sd, d + bond_length_tolerance_factor * sd
                    stddev[r, i, j] = stddev[r, j, i] = sd
                else:
                    lo, up = vdw - overlap_tolerance, 1e10
                lower[r, i, j] = lower[r, j, i] = lo
                upper[r, i, j] = upper[r, j, i] = up
    return {"lower_bound": lower, "upper_bound": upper, "stddev": stddev}


def get_cache_path():
    """``~/.fastfold`` (created on demand): where the reference keeps downloaded tables (fastfold/common/residue_constants.py:438-442).
    Nothing in this package downloads anything; the directory is only offered to callers that used it."""
    import os
    path = os.path.join(os.path.expanduser("~"), ".fastfold")
    os.makedirs(path, exist_ok=True)
    return path
