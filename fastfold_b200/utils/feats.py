"""Feature builders and frame / atom-position geometry shared by the model (role of fastfold/utils/feats.py).

``pseudo_beta_fn``, ``atom14_to_atom37``, the template angle (57 ch) / pair (88 ch) features, the extra-MSA feature
(25 ch), and the two structure-module geometry steps: torsion angles -> the 8 rigid-group frames of every residue,
and frames + idealised local coordinates -> atom14 positions.
"""
import torch
import torch.nn as nn

from ..common import residue_constants as rc
from .rigid_utils import Rigid, Rotation
from .tensor_utils import batched_gather, const_like, one_hot


def dgram_from_positions(pos, min_bin=3.25, max_bin=50.75, no_bins=39, inf=1e8):
    """One-hot distance histogram ``[*, N, N, no_bins]`` of the pairwise distances of ``pos [*, N, 3]``."""
    dgram = torch.sum((pos[..., None, :] - pos[..., None, :, :]) ** 2, dim=-1, keepdim=True)
    lower = torch.linspace(min_bin, max_bin, no_bins, device=pos.device) ** 2
    upper = torch.cat([lower[1:], const_like(lower, [inf], "inf_%r" % (inf,))], dim=-1)
    return ((dgram > lower) * (dgram < upper)).type(dgram.dtype)


def pseudo_beta_fn(aatype, all_atom_positions, all_atom_masks):
    """``(pseudo_beta, mask)``: CB position (CA for glycine) of every residue and its mask; the mask is ``None`` when
    ``all_atom_masks`` is (fastfold/utils/feats.py:51-71)."""
    is_gly = aatype == rc.restype_order["G"]
    ca_idx, cb_idx = rc.atom_order["CA"], rc.atom_order["CB"]
    pseudo_beta = torch.where(is_gly[..., None].expand(*((-1,) * len(is_gly.shape)), 3),
                              all_atom_positions[..., ca_idx, :], all_atom_positions[..., cb_idx, :])
    if all_atom_masks is not None:
        mask = torch.where(is_gly, all_atom_masks[..., ca_idx], all_atom_masks[..., cb_idx])
        return pseudo_beta, mask
    return pseudo_beta, None


def atom14_to_atom37(atom14, batch):
    atom37 = batched_gather(atom14, batch["residx_atom37_to_atom14"], dim=-2, no_batch_dims=len(atom14.shape[:-2]))
    return atom37 * batch["atom37_atom_exists"][..., None]


def build_template_angle_feat(template_feats):
    """[*, N_templ, N_res, 57]: aatype one-hot (22) + torsion sin/cos (14) + alternative torsions (14) + mask (7)."""
    aatype = template_feats["template_aatype"]
    tors = template_feats["template_torsion_angles_sin_cos"]
    alt = template_feats["template_alt_torsion_angles_sin_cos"]
    mask = template_feats["template_torsion_angles_mask"]
    return torch.cat([nn.functional.one_hot(aatype, 22), tors.reshape(*tors.shape[:-2], 14), alt.reshape(*alt.shape[:-2], 14), mask], dim=-1)


def build_template_pair_feat(batch, min_bin, max_bin, no_bins, use_unit_vector=False, eps=1e-20, inf=1e8, chunk=None):
    """[*, N_res, N_res, 88]: distogram (39) + pair mask (1) + aatype of both residues (2 x 22) + unit vector (3) + mask (1)."""
    template_mask = batch["template_pseudo_beta_mask"]
    template_mask_2d = template_mask[..., None] * template_mask[..., None, :]
    tpb = batch["template_pseudo_beta"]
    dgram = dgram_from_positions(tpb, min_bin, max_bin, no_bins, inf)
    to_concat = [dgram, template_mask_2d[..., None]]
    aatype_one_hot = nn.functional.one_hot(batch["template_aatype"], rc.restype_num + 2)
    n_res = batch["template_aatype"].shape[-1]
    to_concat.append(aatype_one_hot[..., None, :, :].expand(*aatype_one_hot.shape[:-2], n_res, -1, -1))
    to_concat.append(aatype_one_hot[..., None, :].expand(*aatype_one_hot.shape[:-2], -1, n_res, -1))
    n, ca, c = [rc.atom_order[a] for a in ["N", "CA", "C"]]
    rigids = Rigid.make_transform_from_reference(n_xyz=batch["template_all_atom_positions"][..., n, :],
                                                 ca_xyz=batch["template_all_atom_positions"][..., ca, :],
                                                 c_xyz=batch["template_all_atom_positions"][..., c, :], eps=eps)
    points = rigids.get_trans()[..., None, :, :]
    rigid_vec = rigids[..., None].invert_apply(points)
    inv_distance_scalar = torch.rsqrt(eps + torch.sum(rigid_vec ** 2, dim=-1))
    t_aa_masks = batch["template_all_atom_mask"]
    template_mask = t_aa_masks[..., n] * t_aa_masks[..., ca] * t_aa_masks[..., c]
    template_mask_2d = template_mask[..., None] * template_mask[..., None, :]
    inv_distance_scalar = inv_distance_scalar * template_mask_2d
    unit_vector = rigid_vec * inv_distance_scalar[..., None]
    if not use_unit_vector:
        unit_vector = unit_vector * 0.0
    to_concat.extend(torch.unbind(unit_vector[..., None, :], dim=-1))
    to_concat.append(template_mask_2d[..., None])
    act = torch.cat(to_concat, dim=-1)
    return act * template_mask_2d[..., None]


def build_extra_msa_feat(batch):
    """[*, N_extra, N_res, 25]: residue one-hot (23) + has_deletion + deletion_value."""
    msa_1hot = nn.functional.one_hot(batch["extra_msa"], 23)
    return torch.cat([msa_1hot, batch["extra_has_deletion"].unsqueeze(-1), batch["extra_deletion_value"].unsqueeze(-1)], dim=-1)


def torsion_angles_to_frames(r, alpha, aatype, rrgdf):
    """Backbone frames ``r [*, N]`` + torsions ``alpha [*, N, 7, 2]`` (sin, cos) -> the 8 rigid-group frames ``[*, N, 8]``
    in the global frame.  ``rrgdf [21, 8, 4, 4]``: default frame of every group of every residue type."""
    default_4x4 = rrgdf[aatype, ...]
    default_r = r.from_tensor_4x4(default_4x4)
    bb_rot = alpha.new_zeros((*((1,) * len(alpha.shape[:-1])), 2))
    bb_rot[..., 1] = 1
    alpha = torch.cat([bb_rot.expand(*alpha.shape[:-2], -1, -1), alpha], dim=-2)
    # rotation about the x axis by the torsion angle: [[1, 0, 0], [0, cos, -sin], [0, sin, cos]]
    all_rots = alpha.new_zeros(default_r.get_rots().get_rot_mats().shape)
    all_rots[..., 0, 0] = 1
    all_rots[..., 1, 1] = alpha[..., 1]
    all_rots[..., 1, 2] = -alpha[..., 0]
    all_rots[..., 2, 1:] = alpha
    all_frames = default_r.compose(Rigid(Rotation(rot_mats=all_rots), None))
    chi2_to_bb = all_frames[..., 4].compose(all_frames[..., 5])
    chi3_to_bb = chi2_to_bb.compose(all_frames[..., 6])
    chi4_to_bb = chi3_to_bb.compose(all_frames[..., 7])
    all_to_bb = Rigid.cat([all_frames[..., :5], chi2_to_bb.unsqueeze(-1), chi3_to_bb.unsqueeze(-1), chi4_to_bb.unsqueeze(-1)], dim=-1)
    return r[..., None].compose(all_to_bb)


def frames_and_literature_positions_to_atom14_pos(r, aatype, default_frames, group_idx, atom_mask, lit_positions):
    """Places the idealised local coordinates of every atom14 slot with the frame of the group it belongs to."""
    group_mask = nn.functional.one_hot(group_idx[aatype, ...], num_classes=default_frames.shape[-3])
    t_atoms_to_global = r[..., None, :] * group_mask
    t_atoms_to_global = t_atoms_to_global.map_tensor_fn(lambda x: torch.sum(x, dim=-1))
    atom_mask = atom_mask[aatype, ...].unsqueeze(-1)
    lit_positions = lit_positions[aatype, ...]
    return t_atoms_to_global.apply(lit_positions) * atom_mask
