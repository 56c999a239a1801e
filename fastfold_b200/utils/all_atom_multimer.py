"""All-atom helpers of the multimer code paths on the struct-of-arrays geometry (role of
fastfold/utils/all_atom_multimer.py): atom14 <-> atom37 conversion, backbone frames from N / CA / C, chi angles."""
import torch

from ..common import residue_constants as rc
from .geometry import Rigid3Array, Rot3Array, Vec3Array, dihedral_angle


def _table(arr, aatype, dtype=None):
    t = torch.tensor(arr, device=aatype.device)
    if dtype is not None:
        t = t.to(dtype)
    return t[aatype]


def get_atom37_mask(aatype):
    return _table(rc.restype_atom37_mask, aatype, torch.float32)


def get_atom14_mask(aatype):
    return _table(rc.restype_atom14_mask, aatype, torch.float32)


def atom14_to_atom37(atom14_data, aatype):
    """``atom14_data [*, N, 14, ...]`` -> ``[*, N, 37, ...]`` (zeros where an atom type does not exist)."""
    idx = _table(rc.restype_atom37_to_atom14, aatype).long()
    mask = get_atom37_mask(aatype)
    extra = atom14_data.dim() - idx.dim()
    idx_e = idx.reshape(idx.shape + (1,) * extra).expand(idx.shape + atom14_data.shape[idx.dim():])
    out = torch.gather(atom14_data, idx.dim() - 1, idx_e)
    return out * mask.reshape(mask.shape + (1,) * extra).to(out.dtype)


def atom37_to_atom14(atom37_data, aatype, all_atom_mask=None):
    """``atom37_to_atom14(data [*, N, 37, ...], aatype)`` gathers any per-atom quantity into the 14-slot layout (slots a
    residue type does not have are zeroed).  The reference's call, ``atom37_to_atom14(aatype, all_atom_pos, all_atom_mask)
    -> (positions14, mask14)`` (fastfold/utils/all_atom_multimer.py:57-79), is recognised by its third argument."""
    if all_atom_mask is not None:
        aatype, positions = atom37_data, aatype
        mask14 = atom37_to_atom14(all_atom_mask.to(torch.float32), aatype)
        if isinstance(positions, Vec3Array):                  # struct-of-arrays in, struct-of-arrays out
            return Vec3Array.from_array(atom37_to_atom14(positions.to_tensor(), aatype) * mask14[..., None]), mask14
        return atom37_to_atom14(positions, aatype) * mask14[..., None].to(positions.dtype), mask14
    idx = _table(rc.restype_atom14_to_atom37, aatype).long()
    mask = get_atom14_mask(aatype)
    extra = atom37_data.dim() - idx.dim()
    idx_e = idx.reshape(idx.shape + (1,) * extra).expand(idx.shape + atom37_data.shape[idx.dim():])
    out = torch.gather(atom37_data, idx.dim() - 1, idx_e)
    return out * mask.reshape(mask.shape + (1,) * extra).to(out.dtype)


def make_backbone_affine(positions: Vec3Array, mask, aatype):
    """Backbone frames (origin CA, x axis towards C, xy plane through N) and their mask from atom37 positions."""
    n, ca, c = (rc.atom_order[a] for a in ("N", "CA", "C"))
    rigid_mask = mask[..., n] * mask[..., ca] * mask[..., c]
    e0 = positions[..., c] - positions[..., ca]
    e1 = positions[..., n] - positions[..., ca]
    rot = Rot3Array.from_two_vectors(e0, e1)
    return Rigid3Array(rot, positions[..., ca]), rigid_mask


def compute_chi_angles(positions: Vec3Array, mask, aatype):
    """The four side-chain dihedrals and their mask: ``[*, N, 4]`` each."""
    chi_idx = torch.tensor(rc.chi_atom_indices() if callable(getattr(rc, "chi_atom_indices", None)) else _chi_atom_indices(),
                           device=aatype.device)[aatype]                    # [*, N, 4, 4]
    chi_mask_tab = torch.tensor(list(rc.chi_angles_mask) + [[0.0] * 4], device=aatype.device, dtype=torch.float32)[aatype]
    pts = []
    for k in range(4):
        ix = chi_idx[..., k].long()
        pts.append(Vec3Array(torch.gather(positions.x, -1, ix), torch.gather(positions.y, -1, ix), torch.gather(positions.z, -1, ix)))
    angles = dihedral_angle(*pts)
    atoms_ok = torch.stack([torch.gather(mask, -1, chi_idx[..., k].long()) for k in range(4)], dim=-1).prod(dim=-1)
    return angles, chi_mask_tab * atoms_ok


def _chi_atom_indices():
    out = []
    for res in rc.restypes:
        res3 = rc.restype_1to3[res]
        rows = [[rc.atom_order[a] for a in chi] for chi in rc.chi_angles_atoms[res3]]
        rows += [[0, 0, 0, 0]] * (4 - len(rows))
        out.append(rows)
    out.append([[0, 0, 0, 0]] * 4)
    return out


# ---------------------------------------------------------------------------
# Frames, torsions and idealised coordinates on the struct-of-arrays geometry
# (roles of fastfold/utils/all_atom_multimer.py:26-32, 82-98, 100-209, 211-319, 321-340, 342-366, 447-474)
# ---------------------------------------------------------------------------
def squared_difference(x, y):
    return (x - y) ** 2


def get_rc_tensor(rc_np, aatype):
    """Row ``aatype`` of a per-residue-type constant table, on the device of ``aatype``."""
    return _table(rc_np, aatype)


def get_chi_atom_indices(device=None):
    """``[21, 4, 4]`` atom37 indices of the four atoms of every chi angle (zeros where a residue has fewer)."""
    return torch.tensor(_chi_atom_indices(), device=device)


def get_alt_atom14(aatype, positions: Vec3Array, mask):
    """Atom14 positions / mask with the names of the 180-degree-symmetric groups swapped (ASP OD1/OD2, GLU OE1/OE2,
    PHE / TYR ring atoms): the alternative ground truth the FAPE and chi losses choose from."""
    renaming = _table(rc.renaming_matrices, aatype, torch.float32)                 # [*, N, 14, 14]
    def mix(t):
        return torch.sum(t[..., None].to(renaming.dtype) * renaming, dim=-2)
    alt_pos = Vec3Array(mix(positions.x), mix(positions.y), mix(positions.z))
    return alt_pos, mix(mask.to(renaming.dtype))


def make_transform_from_reference(a_xyz: Vec3Array, b_xyz: Vec3Array, c_xyz: Vec3Array) -> Rigid3Array:
    """Frame with origin ``b``, x axis towards ``c`` and ``a`` in the xy plane (Gram-Schmidt on ``c - b`` and ``a - b``)."""
    rot = Rot3Array.from_two_vectors(c_xyz - b_xyz, a_xyz - b_xyz)
    return Rigid3Array(rot, b_xyz)


def atom37_to_frames(aatype, all_atom_positions: Vec3Array, all_atom_mask):
    """The eight rigid-group frames of every residue from atom37 coordinates (Algorithm 21 inputs): ground-truth
    frames, their existence mask, which groups are ambiguous under atom renaming and the alternative frames."""
    base = _table(rc.restype_rigidgroup_base_atom37_idx, aatype).long()           # [*, N, 8, 3]
    def pick(k):
        ix = base[..., k]
        return Vec3Array(torch.gather(all_atom_positions.x, -1, ix), torch.gather(all_atom_positions.y, -1, ix),
                         torch.gather(all_atom_positions.z, -1, ix))
    # group frames (Algorithm 21): origin at the second base atom, x axis from the first to the second, third in the xy plane
    a, b, c = pick(0), pick(1), pick(2)
    gt_frames = Rigid3Array(Rot3Array.from_two_vectors(b - a, c - b), b)
    group_exists = _table(rc.restype_rigidgroup_mask, aatype, torch.float32)
    atoms_exist = torch.stack([torch.gather(all_atom_mask.to(torch.float32), -1, base[..., k]) for k in range(3)], dim=-1).min(dim=-1)[0]
    gt_exists = atoms_exist * group_exists
    # the backbone group's x axis and z axis point the other way in AlphaFold's convention
    flip = torch.ones(8, 3, device=aatype.device)
    flip[0, 0] = -1.0
    flip[0, 2] = -1.0
    def flipped(rot, sgn):
        return Rot3Array(rot.xx * sgn[..., 0], rot.xy * sgn[..., 1], rot.xz * sgn[..., 2],
                         rot.yx * sgn[..., 0], rot.yy * sgn[..., 1], rot.yz * sgn[..., 2],
                         rot.zx * sgn[..., 0], rot.zy * sgn[..., 1], rot.zz * sgn[..., 2])
    gt_frames = Rigid3Array(flipped(gt_frames.rotation, flip), gt_frames.translation)
    # ambiguity: a 180-degree rotation about the x axis maps the frame onto its renamed twin
    amb_tab = torch.zeros(21, 8)
    rot_tab = torch.ones(21, 8, 3)
    for res in rc.residue_atom_renaming_swaps:          # residues with a 180-degree-symmetric terminal group
        r = rc.restype_order[rc.restype_3to1[res]]
        g = int(sum(rc.chi_angles_mask[r]) - 1) + 4
        amb_tab[r, g] = 1.0
        rot_tab[r, g, 1] = -1.0
        rot_tab[r, g, 2] = -1.0
    is_ambiguous = amb_tab.to(aatype.device)[aatype]
    alt_sgn = rot_tab.to(aatype.device)[aatype]
    alt_frames = Rigid3Array(flipped(gt_frames.rotation, alt_sgn), gt_frames.translation)
    return {"rigidgroups_gt_frames": gt_frames, "rigidgroups_gt_exists": gt_exists, "rigidgroups_group_exists": group_exists,
            "rigidgroups_group_is_ambiguous": is_ambiguous, "rigidgroups_alt_gt_frames": alt_frames}


def torsion_angles_to_frames(aatype, backb_to_global: Rigid3Array, torsion_angles_sin_cos):
    """Backbone frames ``[*, N]`` and the seven torsions ``[*, N, 7, 2]`` (sin, cos) -> the eight group frames ``[*, N, 8]``
    in the global frame (Algorithm 24, first half)."""
    default = _table(rc.restype_rigid_group_default_frame, aatype, torch.float32)  # [*, N, 8, 4, 4]
    default_frames = Rigid3Array.from_tensor_4x4(default)
    sin = torch.cat([torch.zeros_like(torsion_angles_sin_cos[..., :1, 0]), torsion_angles_sin_cos[..., 0]], dim=-1)
    cos = torch.cat([torch.ones_like(torsion_angles_sin_cos[..., :1, 1]), torsion_angles_sin_cos[..., 1]], dim=-1)
    one, zero = torch.ones_like(sin), torch.zeros_like(sin)
    # rotation about the x axis by each torsion angle
    rot_x = Rot3Array(one, zero, zero, zero, cos, -sin, zero, sin, cos)
    all_frames = default_frames @ Rigid3Array(rot_x, Vec3Array(zero, zero, zero))
    # chi2..chi4 frames are defined relative to the previous chi frame
    chain = [all_frames[..., i] for i in range(8)]
    chi2 = chain[4] @ chain[5]
    chi3 = chi2 @ chain[6]
    chi4 = chi3 @ chain[7]
    parts = chain[:5] + [chi2, chi3, chi4]
    def stack(get):
        return torch.stack([get(p) for p in parts], dim=-1)
    rot = Rot3Array(*[stack(lambda p, n=n: getattr(p.rotation, n)) for n in ("xx", "xy", "xz", "yx", "yy", "yz", "zx", "zy", "zz")])
    trans = Vec3Array(*[stack(lambda p, n=n: getattr(p.translation, n)) for n in ("x", "y", "z")])
    to_backbone = Rigid3Array(rot, trans)
    return backb_to_global[..., None] @ to_backbone


def frames_and_literature_positions_to_atom14_pos(aatype, all_frames_to_global: Rigid3Array) -> Vec3Array:
    """Idealised local coordinates of every atom14 slot placed with the frame of its rigid group (Algorithm 24, second half)."""
    group = _table(rc.restype_atom14_to_rigid_group, aatype).long()                # [*, N, 14]
    def pick(t):
        return torch.gather(t, -1, group)
    r = all_frames_to_global.rotation
    rot = Rot3Array(*[pick(getattr(r, n)) for n in ("xx", "xy", "xz", "yx", "yy", "yz", "zx", "zy", "zz")])
    tr = all_frames_to_global.translation
    frames = Rigid3Array(rot, Vec3Array(pick(tr.x), pick(tr.y), pick(tr.z)))
    lit = _table(rc.restype_atom14_rigid_group_positions, aatype, torch.float32)   # [*, N, 14, 3]
    pos = frames.apply_to_point(Vec3Array(lit[..., 0], lit[..., 1], lit[..., 2]))
    mask = get_atom14_mask(aatype)
    return pos * mask


def extreme_ca_ca_distance_violations(positions: Vec3Array, mask, residue_index, max_angstrom_tolerance=1.5, eps=1e-6):
    """Fraction of consecutive residues whose CA-CA distance exceeds the ideal 3.8 A by more than the tolerance."""
    from .geometry import euclidean_distance
    this_ca, next_ca = positions[..., :-1, 1], positions[..., 1:, 1]
    this_m, next_m = mask[..., :-1, 1], mask[..., 1:, 1]
    no_gap = ((residue_index[..., 1:] - residue_index[..., :-1]) == 1).to(mask.dtype)
    d = euclidean_distance(this_ca, next_ca, eps)
    viol = ((d - rc.ca_ca) > max_angstrom_tolerance).to(mask.dtype)
    m = this_m * next_m * no_gap
    return (viol * m).sum(dim=-1) / (m.sum(dim=-1) + eps)
