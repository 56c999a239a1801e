"""Tensor-level feature transforms (CPU): ground-truth structure features and MSA features.

Part 1 (this section): atom14 / atom37 index maps, alternative ("renamed") ground truth for symmetric side
chains, rigid-group frames and torsion angles from atom37 coordinates.  Part 2: MSA sampling, clustering, BERT-style
masking, ``msa_feat`` / ``target_feat`` assembly, cropping and padding to fixed size.  Each transform maps a feature
dict to a feature dict; ``curry1`` turns ``f(x, a, b)`` into ``f(a, b)(x)`` for use in transform lists.
Same roles as fastfold/data/data_transforms.py.
"""
import itertools
from functools import reduce, wraps
from operator import add

import numpy as np
import torch

from ..common import residue_constants as rc
from ..utils.rigid_utils import Rigid, Rotation
from ..utils.tensor_utils import batched_gather, tensor_tree_map, tree_map

MSA_FEATURE_NAMES = ["msa", "deletion_matrix", "msa_mask", "msa_row_mask", "bert_mask", "true_msa"]


def curry1(f):
    @wraps(f)
    def fc(*args, **kwargs):
        return lambda x: f(x, *args, **kwargs)
    return fc


# ---------------------------------------------------------------------------
# Part 1: structure features
# ---------------------------------------------------------------------------
def make_atom14_masks(protein):
    """Index maps between the 14-slot per-residue-type atom layout and the fixed 37-atom layout."""
    aatype = protein["aatype"]
    dev = aatype.device
    protein["atom14_atom_exists"] = torch.tensor(rc.restype_atom14_mask, dtype=torch.float32, device=dev)[aatype]
    protein["residx_atom14_to_atom37"] = torch.tensor(rc.restype_atom14_to_atom37, dtype=torch.long, device=dev)[aatype]
    protein["residx_atom37_to_atom14"] = torch.tensor(rc.restype_atom37_to_atom14, dtype=torch.long, device=dev)[aatype]
    protein["atom37_atom_exists"] = torch.tensor(rc.restype_atom37_mask, dtype=torch.float32, device=dev)[aatype]
    return protein


def make_atom14_positions(protein):
    """Ground-truth positions in atom14 layout plus the alternative naming of 180-degree-symmetric side chains."""
    residx_atom14_mask = protein["atom14_atom_exists"]
    residx_atom14_to_atom37 = protein["residx_atom14_to_atom37"]
    nb = len(protein["all_atom_mask"].shape[:-1])
    gt_mask = residx_atom14_mask * batched_gather(protein["all_atom_mask"], residx_atom14_to_atom37, dim=-1, no_batch_dims=nb)
    gt_pos = gt_mask[..., None] * batched_gather(protein["all_atom_positions"], residx_atom14_to_atom37, dim=-2, no_batch_dims=nb)
    protein["atom14_atom_exists"] = residx_atom14_mask
    protein["atom14_gt_exists"] = gt_mask
    protein["atom14_gt_positions"] = gt_pos
    renaming = protein["all_atom_mask"].new_tensor(rc.renaming_matrices)[protein["aatype"]]
    protein["atom14_alt_gt_positions"] = torch.einsum("...rac,...rab->...rbc", gt_pos, renaming)
    protein["atom14_alt_gt_exists"] = torch.einsum("...ra,...rab->...rb", gt_mask, renaming)
    protein["atom14_atom_is_ambiguous"] = protein["all_atom_mask"].new_tensor(rc.restype_atom14_is_ambiguous)[protein["aatype"]]
    return protein


def atom37_to_frames(protein, eps=1e-8):
    """The 8 rigid-group frames of every residue from atom37 coordinates (and the alternative frames of ambiguous groups)."""
    aatype = protein["aatype"]
    all_atom_positions = protein["all_atom_positions"]
    all_atom_mask = protein["all_atom_mask"]
    batch_dims = len(aatype.shape[:-1])
    base_idx = aatype.new_tensor(rc.restype_rigidgroup_base_atom37_idx)          # [21, 8, 3]
    group_exists = all_atom_mask.new_tensor(rc.restype_rigidgroup_mask)          # [21, 8]
    residx_base = base_idx[aatype]
    base_atom_pos = batched_gather(all_atom_positions, residx_base, dim=-2, no_batch_dims=len(all_atom_positions.shape[:-2]))
    gt_frames = Rigid.from_3_points(p_neg_x_axis=base_atom_pos[..., 0, :], origin=base_atom_pos[..., 1, :], p_xy_plane=base_atom_pos[..., 2, :], eps=eps)
    gt_exists_table = group_exists[aatype]
    gt_atoms_exist = batched_gather(all_atom_mask, residx_base, dim=-1, no_batch_dims=len(all_atom_mask.shape[:-1]))
    gt_exists = torch.min(gt_atoms_exist, dim=-1)[0] * gt_exists_table
    rots = torch.eye(3, dtype=all_atom_mask.dtype, device=aatype.device)
    rots = torch.tile(rots, (*((1,) * batch_dims), 8, 1, 1)).clone()
    rots[..., 0, 0, 0] = -1
    rots[..., 0, 2, 2] = -1
    gt_frames = gt_frames.compose(Rigid(Rotation(rot_mats=rots), None))
    # ambiguity: a 180-degree flip about the x axis of the last chi group of D, E, F, Y (and similar)
    is_ambiguous = all_atom_mask.new_zeros(*((1,) * batch_dims), 21, 8)
    ambiguity_rot = torch.eye(3, dtype=all_atom_mask.dtype, device=aatype.device)
    ambiguity_rot = torch.tile(ambiguity_rot, (*((1,) * batch_dims), 21, 8, 1, 1)).clone()
    for resname in rc.residue_atom_renaming_swaps:
        restype = rc.restype_order[rc.restype_3to1[resname]]
        chi_idx = int(sum(rc.chi_angles_mask[restype]) - 1)
        is_ambiguous[..., restype, chi_idx + 4] = 1
        ambiguity_rot[..., restype, chi_idx + 4, 1, 1] = -1
        ambiguity_rot[..., restype, chi_idx + 4, 2, 2] = -1
    residx_is_ambiguous = batched_gather(is_ambiguous, aatype, dim=-2, no_batch_dims=batch_dims)
    residx_ambiguity_rot = batched_gather(ambiguity_rot, aatype, dim=-4, no_batch_dims=batch_dims)
    alt_gt_frames = gt_frames.compose(Rigid(Rotation(rot_mats=residx_ambiguity_rot), None))
    protein["rigidgroups_gt_frames"] = gt_frames.to_tensor_4x4()
    protein["rigidgroups_gt_exists"] = gt_exists
    protein["rigidgroups_group_exists"] = gt_exists_table
    protein["rigidgroups_group_is_ambiguous"] = residx_is_ambiguous
    protein["rigidgroups_alt_gt_frames"] = alt_gt_frames.to_tensor_4x4()
    return protein


def _chi_atom_indices():
    """[21, 4, 4] atom37 indices of the four atoms defining each chi angle (zeros where undefined)."""
    out = []
    for letter in rc.restypes:
        rows = [[rc.atom_order[a] for a in atoms] for atoms in rc.chi_angles_atoms[rc.restype_1to3[letter]]]
        rows += [[0, 0, 0, 0]] * (4 - len(rows))
        out.append(rows)
    out.append([[0, 0, 0, 0]] * 4)
    return out


@curry1
def atom37_to_torsion_angles(protein, prefix=""):
    """Seven torsions per residue (pre-omega, phi, psi, chi1-4) as (sin, cos), their mask, and the pi-shifted alternative."""
    aatype = protein[prefix + "aatype"]
    all_atom_positions = protein[prefix + "all_atom_positions"]
    all_atom_mask = protein[prefix + "all_atom_mask"]
    aatype = torch.clamp(aatype, max=20)
    pad = all_atom_positions.new_zeros([*all_atom_positions.shape[:-3], 1, 37, 3])
    prev_pos = torch.cat([pad, all_atom_positions[..., :-1, :, :]], dim=-3)
    pad = all_atom_mask.new_zeros([*all_atom_mask.shape[:-2], 1, 37])
    prev_mask = torch.cat([pad, all_atom_mask[..., :-1, :]], dim=-2)
    pre_omega_pos = torch.cat([prev_pos[..., 1:3, :], all_atom_positions[..., :2, :]], dim=-2)
    phi_pos = torch.cat([prev_pos[..., 2:3, :], all_atom_positions[..., :3, :]], dim=-2)
    psi_pos = torch.cat([all_atom_positions[..., :3, :], all_atom_positions[..., 4:5, :]], dim=-2)
    pre_omega_mask = torch.prod(prev_mask[..., 1:3], dim=-1) * torch.prod(all_atom_mask[..., :2], dim=-1)
    phi_mask = prev_mask[..., 2] * torch.prod(all_atom_mask[..., :3], dim=-1, dtype=all_atom_mask.dtype)
    psi_mask = torch.prod(all_atom_mask[..., :3], dim=-1, dtype=all_atom_mask.dtype) * all_atom_mask[..., 4]
    chi_idx = torch.as_tensor(_chi_atom_indices(), device=aatype.device)
    atom_indices = chi_idx[..., aatype, :, :]
    chis_pos = batched_gather(all_atom_positions, atom_indices, -2, len(atom_indices.shape[:-2]))
    chi_angles_mask = list(rc.chi_angles_mask)
    chi_angles_mask.append([0.0, 0.0, 0.0, 0.0])
    chi_angles_mask = all_atom_mask.new_tensor(chi_angles_mask)
    chis_mask = chi_angles_mask[aatype, :]
    chi_atoms_mask = batched_gather(all_atom_mask, atom_indices, dim=-1, no_batch_dims=len(atom_indices.shape[:-2]))
    chis_mask = chis_mask * torch.prod(chi_atoms_mask, dim=-1, dtype=chi_atoms_mask.dtype)
    torsions_pos = torch.cat([pre_omega_pos[..., None, :, :], phi_pos[..., None, :, :], psi_pos[..., None, :, :], chis_pos], dim=-3)
    torsion_mask = torch.cat([pre_omega_mask[..., None], phi_mask[..., None], psi_mask[..., None], chis_mask], dim=-1)
    frames = Rigid.from_3_points(torsions_pos[..., 1, :], torsions_pos[..., 2, :], torsions_pos[..., 0, :], eps=1e-8)
    fourth = frames.invert().apply(torsions_pos[..., 3, :])
    sin_cos = torch.stack([fourth[..., 2], fourth[..., 1]], dim=-1)
    sin_cos = sin_cos / torch.sqrt(torch.sum(torch.square(sin_cos), dim=-1, dtype=sin_cos.dtype, keepdims=True) + 1e-8)
    sin_cos = sin_cos * all_atom_mask.new_tensor([1.0, 1.0, -1.0, 1.0, 1.0, 1.0, 1.0])[((None,) * len(sin_cos.shape[:-2])) + (slice(None), None)]
    chi_is_ambiguous = sin_cos.new_tensor(rc.chi_pi_periodic)[aatype, ...]
    mirror = torch.cat([all_atom_mask.new_ones(*aatype.shape, 3), 1.0 - 2.0 * chi_is_ambiguous], dim=-1)
    protein[prefix + "torsion_angles_sin_cos"] = sin_cos
    protein[prefix + "alt_torsion_angles_sin_cos"] = sin_cos * mirror[..., None]
    protein[prefix + "torsion_angles_mask"] = torsion_mask
    return protein


@curry1
def make_pseudo_beta(protein, prefix=""):
    from ..utils.feats import pseudo_beta_fn
    assert prefix in ["", "template_"]
    protein[prefix + "pseudo_beta"], protein[prefix + "pseudo_beta_mask"] = pseudo_beta_fn(
        protein["template_aatype" if prefix else "aatype"], protein[prefix + "all_atom_positions"],
        protein["template_all_atom_mask" if prefix else "all_atom_mask"])
    return protein


def get_backbone_frames(protein):
    protein["backbone_rigid_tensor"] = protein["rigidgroups_gt_frames"][..., 0, :, :]
    protein["backbone_rigid_mask"] = protein["rigidgroups_gt_exists"][..., 0]
    return protein


def get_chi_angles(protein):
    dtype = protein["all_atom_mask"].dtype
    protein["chi_angles_sin_cos"] = protein["torsion_angles_sin_cos"][..., 3:, :].to(dtype)
    protein["chi_mask"] = protein["torsion_angles_mask"][..., 3:].to(dtype)
    return protein
