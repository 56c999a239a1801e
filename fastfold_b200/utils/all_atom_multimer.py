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


def atom37_to_atom14(atom37_data, aatype):
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
