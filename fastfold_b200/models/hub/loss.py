"""AlphaFold training loss (supplement 1.9): FAPE, torsion, distogram, masked-MSA, pLDDT, experimentally-resolved,
structural violations and (for pTM models) the TM head loss, combined by ``AlphaFoldLoss``.

Terms that evaluate to NaN / Inf are skipped with a warning; the total is scaled by sqrt(min(N_res, crop_size)).
Same contract as fastfold/model/hub/loss.py:1565-1655 (``AlphaFoldLoss(config)(out, batch, _return_breakdown)``).
"""
import logging
from typing import Dict, Optional

import torch
import torch.nn as nn

from ...common import residue_constants as rc
from ...utils import feats
from ...utils.rigid_utils import Rigid, Rotation
from ...utils.tensor_utils import batched_gather, const_like, masked_mean, permute_final_dims, tensor_tree_map, tree_map


def softmax_cross_entropy(logits, labels):
    return -1 * torch.sum(labels * torch.nn.functional.log_softmax(logits.float(), dim=-1), dim=-1)


def sigmoid_cross_entropy(logits, labels):
    logits = logits.float()
    log_p = torch.nn.functional.logsigmoid(logits)
    log_not_p = torch.nn.functional.logsigmoid(-logits)
    return -labels * log_p - (1 - labels) * log_not_p


# ---------------------------------------------------------------------------
# FAPE
# ---------------------------------------------------------------------------
def compute_fape(pred_frames: Rigid, target_frames: Rigid, frames_mask, pred_positions, target_positions, positions_mask, length_scale,
                 l1_clamp_distance: Optional[float] = None, eps=1e-8):
    """Frame-aligned point error (Algorithm 28): every atom seen from every frame, clamped L2 error, masked mean."""
    local_pred = pred_frames.invert()[..., None].apply(pred_positions[..., None, :, :])
    local_target = target_frames.invert()[..., None].apply(target_positions[..., None, :, :])
    error = torch.sqrt(torch.sum((local_pred - local_target) ** 2, dim=-1) + eps)
    if l1_clamp_distance is not None:
        error = torch.clamp(error, min=0, max=l1_clamp_distance)
    normed = error / length_scale
    normed = normed * frames_mask[..., None] * positions_mask[..., None, :]
    normed = torch.sum(normed, dim=-1) / (eps + torch.sum(frames_mask, dim=-1))[..., None]
    return torch.sum(normed, dim=-1) / (eps + torch.sum(positions_mask, dim=-1))


def backbone_loss(backbone_rigid_tensor, backbone_rigid_mask, traj, use_clamped_fape=None, clamp_distance=10.0, loss_unit_distance=10.0,
                  eps=1e-4, **kwargs):
    pred_aff = Rigid.from_tensor_7(traj)
    pred_aff = Rigid(Rotation(rot_mats=pred_aff.get_rots().get_rot_mats(), quats=None), pred_aff.get_trans())
    gt_aff = Rigid.from_tensor_4x4(backbone_rigid_tensor)
    args = (pred_aff, gt_aff[None], backbone_rigid_mask[None], pred_aff.get_trans(), gt_aff[None].get_trans(), backbone_rigid_mask[None])
    fape = compute_fape(*args, l1_clamp_distance=clamp_distance, length_scale=loss_unit_distance, eps=eps)
    if use_clamped_fape is not None:
        unclamped = compute_fape(*args, l1_clamp_distance=None, length_scale=loss_unit_distance, eps=eps)
        fape = fape * use_clamped_fape + unclamped * (1 - use_clamped_fape)
    return torch.mean(fape)


def sidechain_loss(sidechain_frames, sidechain_atom_pos, rigidgroups_gt_frames, rigidgroups_alt_gt_frames, rigidgroups_gt_exists,
                   renamed_atom14_gt_positions, renamed_atom14_gt_exists, alt_naming_is_better, clamp_distance=10.0, length_scale=10.0,
                   eps=1e-4, **kwargs):
    renamed_gt_frames = (1.0 - alt_naming_is_better[..., None, None, None]) * rigidgroups_gt_frames + \
        alt_naming_is_better[..., None, None, None] * rigidgroups_alt_gt_frames
    sidechain_frames = sidechain_frames[-1]
    batch_dims = sidechain_frames.shape[:-4]
    sidechain_frames = Rigid.from_tensor_4x4(sidechain_frames.reshape(*batch_dims, -1, 4, 4))
    renamed_gt_frames = Rigid.from_tensor_4x4(renamed_gt_frames.view(*batch_dims, -1, 4, 4))
    rigidgroups_gt_exists = rigidgroups_gt_exists.reshape(*batch_dims, -1)
    sidechain_atom_pos = sidechain_atom_pos[-1].view(*batch_dims, -1, 3)
    renamed_atom14_gt_positions = renamed_atom14_gt_positions.view(*batch_dims, -1, 3)
    renamed_atom14_gt_exists = renamed_atom14_gt_exists.view(*batch_dims, -1)
    return compute_fape(sidechain_frames, renamed_gt_frames, rigidgroups_gt_exists, sidechain_atom_pos, renamed_atom14_gt_positions,
                        renamed_atom14_gt_exists, l1_clamp_distance=clamp_distance, length_scale=length_scale, eps=eps)


def fape_loss(out, batch, config):
    bb = backbone_loss(traj=out["sm"]["frames"], **{**batch, **config.backbone})
    sc = sidechain_loss(out["sm"]["sidechain_frames"], out["sm"]["positions"], **{**batch, **config.sidechain})
    return torch.mean(config.backbone.weight * bb + config.sidechain.weight * sc)


def supervised_chi_loss(angles_sin_cos, unnormalized_angles_sin_cos, aatype, seq_mask, chi_mask, chi_angles_sin_cos, chi_weight,
                        angle_norm_weight, eps=1e-6, **kwargs):
    """Torsion loss (Algorithm 27) with the pi-periodic alternative for symmetric side chains."""
    pred_angles = angles_sin_cos[..., 3:, :]
    residue_type_one_hot = torch.nn.functional.one_hot(aatype, rc.restype_num + 1)
    chi_pi_periodic = torch.einsum("...ij,jk->ik", residue_type_one_hot.type(angles_sin_cos.dtype),
                                   const_like(angles_sin_cos, rc.chi_pi_periodic, "chi_pi_periodic"))
    true_chi = chi_angles_sin_cos[None]
    shifted_mask = (1 - 2 * chi_pi_periodic).unsqueeze(-1)
    true_chi_shifted = shifted_mask * true_chi
    sq_chi_error = torch.sum((true_chi - pred_angles) ** 2, dim=-1)
    sq_chi_error_shifted = torch.sum((true_chi_shifted - pred_angles) ** 2, dim=-1)
    sq_chi_error = torch.minimum(sq_chi_error, sq_chi_error_shifted)
    sq_chi_error = sq_chi_error.permute(*range(len(sq_chi_error.shape))[1:-2], 0, -2, -1)
    sq_chi_loss = masked_mean(chi_mask[..., None, :, :], sq_chi_error, dim=(-1, -2, -3))
    loss = chi_weight * sq_chi_loss
    angle_norm = torch.sqrt(torch.sum(unnormalized_angles_sin_cos ** 2, dim=-1) + eps)
    norm_error = torch.abs(angle_norm - 1.0)
    norm_error = norm_error.permute(*range(len(norm_error.shape))[1:-2], 0, -2, -1)
    angle_norm_loss = masked_mean(seq_mask[..., None, :, None], norm_error, dim=(-1, -2, -3))
    loss = loss + angle_norm_weight * angle_norm_loss
    return torch.mean(loss)


# ---------------------------------------------------------------------------
# confidence / distogram / MSA heads
# ---------------------------------------------------------------------------
def lddt(all_atom_pred_pos, all_atom_positions, all_atom_mask, cutoff=15.0, eps=1e-10, per_residue=True):
    n = all_atom_mask.shape[-2]
    dmat_true = torch.sqrt(eps + torch.sum((all_atom_positions[..., None, :] - all_atom_positions[..., None, :, :]) ** 2, dim=-1))
    dmat_pred = torch.sqrt(eps + torch.sum((all_atom_pred_pos[..., None, :] - all_atom_pred_pos[..., None, :, :]) ** 2, dim=-1))
    dists_to_score = (dmat_true < cutoff) * all_atom_mask * permute_final_dims(all_atom_mask, (1, 0)) * \
        (1.0 - torch.eye(n, device=all_atom_mask.device))
    dist_l1 = torch.abs(dmat_true - dmat_pred)
    score = ((dist_l1 < 0.5).type(dist_l1.dtype) + (dist_l1 < 1.0).type(dist_l1.dtype) + (dist_l1 < 2.0).type(dist_l1.dtype) +
             (dist_l1 < 4.0).type(dist_l1.dtype)) * 0.25
    dims = (-1,) if per_residue else (-2, -1)
    norm = 1.0 / (eps + torch.sum(dists_to_score, dim=dims))
    return norm * (eps + torch.sum(dists_to_score * score, dim=dims))


def lddt_ca(all_atom_pred_pos, all_atom_positions, all_atom_mask, cutoff=15.0, eps=1e-10, per_residue=True):
    ca = rc.atom_order["CA"]
    return lddt(all_atom_pred_pos[..., ca, :], all_atom_positions[..., ca, :], all_atom_mask[..., ca:(ca + 1)], cutoff=cutoff, eps=eps,
                per_residue=per_residue)


def lddt_loss(logits, all_atom_pred_pos, all_atom_positions, all_atom_mask, resolution, cutoff=15.0, no_bins=50, min_resolution=0.1,
              max_resolution=3.0, eps=1e-10, **kwargs):
    ca = rc.atom_order["CA"]
    score = lddt(all_atom_pred_pos[..., ca, :], all_atom_positions[..., ca, :], all_atom_mask[..., ca:(ca + 1)], cutoff=cutoff, eps=eps).detach()
    bin_index = torch.clamp(torch.floor(score * no_bins).long(), max=(no_bins - 1))
    lddt_ca_one_hot = torch.nn.functional.one_hot(bin_index, num_classes=no_bins)
    errors = softmax_cross_entropy(logits, lddt_ca_one_hot)
    mask = all_atom_mask[..., ca:(ca + 1)].squeeze(-1)
    loss = torch.sum(errors * mask, dim=-1) / (eps + torch.sum(mask, dim=-1))
    loss = loss * ((resolution >= min_resolution) & (resolution <= max_resolution))
    return torch.mean(loss)


def distogram_loss(logits, pseudo_beta, pseudo_beta_mask, min_bin=2.3125, max_bin=21.6875, no_bins=64, eps=1e-6, **kwargs):
    boundaries = torch.linspace(min_bin, max_bin, no_bins - 1, device=logits.device) ** 2
    dists = torch.sum((pseudo_beta[..., None, :] - pseudo_beta[..., None, :, :]) ** 2, dim=-1, keepdims=True)
    true_bins = torch.sum(dists > boundaries, dim=-1)
    errors = softmax_cross_entropy(logits, torch.nn.functional.one_hot(true_bins, no_bins))
    square_mask = pseudo_beta_mask[..., None] * pseudo_beta_mask[..., None, :]
    denom = eps + torch.sum(square_mask, dim=(-1, -2))
    mean = torch.sum(errors * square_mask, dim=-1) / denom[..., None]
    return torch.mean(torch.sum(mean, dim=-1))


def masked_msa_loss(logits, true_msa, bert_mask, eps=1e-8, **kwargs):
    errors = softmax_cross_entropy(logits, torch.nn.functional.one_hot(true_msa, num_classes=logits.shape[-1]))
    loss = errors * bert_mask
    loss = torch.sum(loss, dim=-1)
    scale = 0.5
    denom = eps + torch.sum(scale * bert_mask, dim=(-1, -2))
    loss = torch.sum(loss, dim=-1) * scale / denom
    return torch.mean(loss)


def experimentally_resolved_loss(logits, atom37_atom_exists, all_atom_mask, resolution, min_resolution, max_resolution, eps=1e-8, **kwargs):
    errors = sigmoid_cross_entropy(logits, all_atom_mask)
    loss = torch.sum(errors * atom37_atom_exists, dim=-1)
    loss = loss / (eps + torch.sum(atom37_atom_exists, dim=(-1, -2)))
    loss = torch.sum(loss, dim=-1)
    loss = loss * ((resolution >= min_resolution) & (resolution <= max_resolution))
    return torch.mean(loss)


def tm_loss(logits, final_affine_tensor, backbone_rigid_tensor, backbone_rigid_mask, resolution, max_bin=31, no_bins=64, min_resolution=0.1,
            max_resolution=3.0, eps=1e-8, **kwargs):
    pred_affine = Rigid.from_tensor_7(final_affine_tensor)
    backbone_rigid = Rigid.from_tensor_4x4(backbone_rigid_tensor)

    def points(affine):
        pts = affine.get_trans()[..., None, :, :]
        return affine.invert()[..., None].apply(pts)

    sq_diff = torch.sum((points(pred_affine) - points(backbone_rigid)) ** 2, dim=-1).detach()
    boundaries = torch.linspace(0, max_bin, steps=(no_bins - 1), device=logits.device) ** 2
    true_bins = torch.sum(sq_diff[..., None] > boundaries, dim=-1)
    errors = softmax_cross_entropy(logits, torch.nn.functional.one_hot(true_bins, no_bins))
    square_mask = backbone_rigid_mask[..., None] * backbone_rigid_mask[..., None, :]
    loss = torch.sum(errors * square_mask, dim=-1)
    scale = 0.5
    denom = eps + torch.sum(scale * square_mask, dim=(-1, -2))
    loss = torch.sum(loss / denom[..., None], dim=-1) * scale
    loss = loss * ((resolution >= min_resolution) & (resolution <= max_resolution))
    return torch.mean(loss)


# ---------------------------------------------------------------------------
# structural violations (supplement 1.9.11)
# ---------------------------------------------------------------------------
def between_residue_bond_loss(pred_atom_positions, pred_atom_mask, residue_index, aatype, tolerance_factor_soft=12.0,
                              tolerance_factor_hard=12.0, eps=1e-6):
    """Peptide-bond geometry between consecutive residues: C-N length, CA-C-N and C-N-CA angles (flat-bottom L1)."""
    this_ca_pos, this_ca_mask = pred_atom_positions[..., :-1, 1, :], pred_atom_mask[..., :-1, 1]
    this_c_pos, this_c_mask = pred_atom_positions[..., :-1, 2, :], pred_atom_mask[..., :-1, 2]
    next_n_pos, next_n_mask = pred_atom_positions[..., 1:, 0, :], pred_atom_mask[..., 1:, 0]
    next_ca_pos, next_ca_mask = pred_atom_positions[..., 1:, 1, :], pred_atom_mask[..., 1:, 1]
    has_no_gap_mask = (residue_index[..., 1:] - residue_index[..., :-1]) == 1.0
    c_n_bond_length = torch.sqrt(eps + torch.sum((this_c_pos - next_n_pos) ** 2, dim=-1))
    next_is_proline = aatype[..., 1:] == rc.resname_to_idx["PRO"]
    gt_length = (~next_is_proline) * rc.between_res_bond_length_c_n[0] + next_is_proline * rc.between_res_bond_length_c_n[1]
    gt_stddev = (~next_is_proline) * rc.between_res_bond_length_stddev_c_n[0] + next_is_proline * rc.between_res_bond_length_stddev_c_n[1]
    c_n_error = torch.sqrt(eps + (c_n_bond_length - gt_length) ** 2)
    c_n_loss_per_residue = torch.nn.functional.relu(c_n_error - tolerance_factor_soft * gt_stddev)
    mask = this_c_mask * next_n_mask * has_no_gap_mask
    c_n_loss = torch.sum(mask * c_n_loss_per_residue, dim=-1) / (torch.sum(mask, dim=-1) + eps)
    c_n_violation_mask = mask * (c_n_error > (tolerance_factor_hard * gt_stddev))
    ca_c_bond_length = torch.sqrt(eps + torch.sum((this_ca_pos - this_c_pos) ** 2, dim=-1))
    n_ca_bond_length = torch.sqrt(eps + torch.sum((next_n_pos - next_ca_pos) ** 2, dim=-1))
    c_ca_unit = (this_ca_pos - this_c_pos) / ca_c_bond_length[..., None]
    c_n_unit = (next_n_pos - this_c_pos) / c_n_bond_length[..., None]
    n_ca_unit = (next_ca_pos - next_n_pos) / n_ca_bond_length[..., None]

    def angle_term(cos_angle, gt, m):
        err = torch.sqrt(eps + (cos_angle - gt[0]) ** 2)
        per_res = torch.nn.functional.relu(err - tolerance_factor_soft * gt[1])
        loss = torch.sum(m * per_res, dim=-1) / (torch.sum(m, dim=-1) + eps)
        return loss, per_res, m * (err > (tolerance_factor_hard * gt[1]))

    m1 = this_ca_mask * this_c_mask * next_n_mask * has_no_gap_mask
    # AlphaFold (and the reference, fastfold/model/hub/loss.py:808-811) scale this angle's tolerance by the C-N BOND LENGTH
    # deviation (0.014) instead of the angle's own cosine deviation (0.031); kept, since published models were trained with it
    ca_c_n_target = (rc.between_res_cos_angles_ca_c_n[0], rc.between_res_bond_length_stddev_c_n[0])
    ca_c_n_loss, ca_c_n_per, ca_c_n_viol = angle_term(torch.sum(c_ca_unit * c_n_unit, dim=-1), ca_c_n_target, m1)
    m2 = this_c_mask * next_n_mask * next_ca_mask * has_no_gap_mask
    c_n_ca_loss, c_n_ca_per, c_n_ca_viol = angle_term(torch.sum((-c_n_unit) * n_ca_unit, dim=-1), rc.between_res_cos_angles_c_n_ca, m2)
    per_residue_loss_sum = c_n_loss_per_residue + ca_c_n_per + c_n_ca_per
    per_residue_loss_sum = 0.5 * (torch.nn.functional.pad(per_residue_loss_sum, (0, 1)) + torch.nn.functional.pad(per_residue_loss_sum, (1, 0)))
    violation_mask = torch.max(torch.stack([c_n_violation_mask, ca_c_n_viol, c_n_ca_viol], dim=-2), dim=-2)[0]
    violation_mask = torch.maximum(torch.nn.functional.pad(violation_mask, (0, 1)), torch.nn.functional.pad(violation_mask, (1, 0)))
    return {"c_n_loss_mean": c_n_loss, "ca_c_n_loss_mean": ca_c_n_loss, "c_n_ca_loss_mean": c_n_ca_loss,
            "per_residue_loss_sum": per_residue_loss_sum, "per_residue_violation_mask": violation_mask}


def between_residue_clash_loss(atom14_pred_positions, atom14_atom_exists, atom14_atom_radius, residue_index, overlap_tolerance_soft=1.5,
                               overlap_tolerance_hard=1.5, eps=1e-10):
    """Steric clashes between atoms of different residues (peptide and disulfide bonds excluded)."""
    fp_type = atom14_pred_positions.dtype
    dists = torch.sqrt(eps + torch.sum((atom14_pred_positions[..., :, None, :, None, :] - atom14_pred_positions[..., None, :, None, :, :]) ** 2, dim=-1))
    dists_mask = (atom14_atom_exists[..., :, None, :, None] * atom14_atom_exists[..., None, :, None, :]).type(fp_type)
    dists_mask = dists_mask * (residue_index[..., :, None, None, None] < residue_index[..., None, :, None, None])
    c_one_hot = torch.nn.functional.one_hot(const_like(residue_index, 2, "idx2"), num_classes=14)
    c_one_hot = c_one_hot.reshape(*((1,) * len(residue_index.shape[:-1])), *c_one_hot.shape).type(fp_type)
    n_one_hot = torch.nn.functional.one_hot(const_like(residue_index, 0, "idx0"), num_classes=14)
    n_one_hot = n_one_hot.reshape(*((1,) * len(residue_index.shape[:-1])), *n_one_hot.shape).type(fp_type)
    neighbour_mask = (residue_index[..., :, None, None, None] + 1) == residue_index[..., None, :, None, None]
    c_n_bonds = neighbour_mask * c_one_hot[..., None, None, :, None] * n_one_hot[..., None, None, None, :]
    dists_mask = dists_mask * (1.0 - c_n_bonds)
    cys_sg_idx = rc.restype_name_to_atom14_names["CYS"].index("SG")
    cys_sg_one_hot = torch.nn.functional.one_hot(const_like(residue_index, cys_sg_idx, "cys_sg_idx"), num_classes=14)
    cys_sg_one_hot = cys_sg_one_hot.reshape(*((1,) * len(residue_index.shape[:-1])), *cys_sg_one_hot.shape)
    disulfide_bonds = cys_sg_one_hot[..., None, None, :, None] * cys_sg_one_hot[..., None, None, None, :]
    dists_mask = dists_mask * (1.0 - disulfide_bonds)
    dists_lower_bound = dists_mask * (atom14_atom_radius[..., :, None, :, None] + atom14_atom_radius[..., None, :, None, :])
    dists_to_low_error = dists_mask * torch.nn.functional.relu(dists_lower_bound - overlap_tolerance_soft - dists)
    mean_loss = torch.sum(dists_to_low_error) / (1e-6 + torch.sum(dists_mask))
    per_atom_loss_sum = torch.sum(dists_to_low_error, dim=(-4, -2)) + torch.sum(dists_to_low_error, dim=(-3, -1))
    clash_mask = dists_mask * (dists < (dists_lower_bound - overlap_tolerance_hard))
    per_atom_clash_mask = torch.maximum(torch.amax(clash_mask, dim=(-4, -2)), torch.amax(clash_mask, dim=(-3, -1)))
    return {"mean_loss": mean_loss, "per_atom_loss_sum": per_atom_loss_sum, "per_atom_clash_mask": per_atom_clash_mask}


def within_residue_violations(atom14_pred_positions, atom14_atom_exists, atom14_dists_lower_bound, atom14_dists_upper_bound,
                              tighten_bounds_for_loss=0.0, eps=1e-10):
    dists_masks = 1.0 - torch.eye(14, device=atom14_atom_exists.device)[None]
    dists_masks = dists_masks.reshape(*((1,) * len(atom14_atom_exists.shape[:-2])), *dists_masks.shape)
    dists_masks = atom14_atom_exists[..., :, :, None] * atom14_atom_exists[..., :, None, :] * dists_masks
    dists = torch.sqrt(eps + torch.sum((atom14_pred_positions[..., :, :, None, :] - atom14_pred_positions[..., :, None, :, :]) ** 2, dim=-1))
    dists_to_low_error = torch.nn.functional.relu(atom14_dists_lower_bound + tighten_bounds_for_loss - dists)
    dists_to_high_error = torch.nn.functional.relu(dists - (atom14_dists_upper_bound - tighten_bounds_for_loss))
    loss = dists_masks * (dists_to_low_error + dists_to_high_error)
    per_atom_loss_sum = torch.sum(loss, dim=-2) + torch.sum(loss, dim=-1)
    violations = dists_masks * ((dists < atom14_dists_lower_bound) | (dists > atom14_dists_upper_bound))
    per_atom_violations = torch.maximum(torch.max(violations, dim=-2)[0], torch.max(violations, axis=-1)[0])
    return {"per_atom_loss_sum": per_atom_loss_sum, "per_atom_violations": per_atom_violations}


def find_structural_violations(batch, atom14_pred_positions, violation_tolerance_factor, clash_overlap_tolerance, **kwargs):
    connection = between_residue_bond_loss(atom14_pred_positions, batch["atom14_atom_exists"], batch["residue_index"], batch["aatype"],
                                           tolerance_factor_soft=violation_tolerance_factor, tolerance_factor_hard=violation_tolerance_factor)
    atomtype_radius = const_like(atom14_pred_positions, [rc.van_der_waals_radius[name[0]] for name in rc.atom_types], "vdw_radius")
    atom14_atom_radius = batch["atom14_atom_exists"] * atomtype_radius[batch["residx_atom14_to_atom37"]]
    clashes = between_residue_clash_loss(atom14_pred_positions, batch["atom14_atom_exists"], atom14_atom_radius, batch["residue_index"],
                                         overlap_tolerance_soft=clash_overlap_tolerance, overlap_tolerance_hard=clash_overlap_tolerance)
    bounds = rc.make_atom14_dists_bounds(overlap_tolerance=clash_overlap_tolerance, bond_length_tolerance_factor=violation_tolerance_factor)
    bkey = "%r_%r" % (clash_overlap_tolerance, violation_tolerance_factor)
    lower = const_like(atom14_pred_positions, bounds["lower_bound"], "atom14_lower_" + bkey)[batch["aatype"]]
    upper = const_like(atom14_pred_positions, bounds["upper_bound"], "atom14_upper_" + bkey)[batch["aatype"]]
    within = within_residue_violations(atom14_pred_positions, batch["atom14_atom_exists"], lower, upper, tighten_bounds_for_loss=0.0)
    per_residue = torch.max(torch.stack([connection["per_residue_violation_mask"], torch.max(clashes["per_atom_clash_mask"], dim=-1)[0],
                                         torch.max(within["per_atom_violations"], dim=-1)[0]], dim=-1), dim=-1)[0]
    return {
        "between_residues": {"bonds_c_n_loss_mean": connection["c_n_loss_mean"], "angles_ca_c_n_loss_mean": connection["ca_c_n_loss_mean"],
                             "angles_c_n_ca_loss_mean": connection["c_n_ca_loss_mean"],
                             "connections_per_residue_loss_sum": connection["per_residue_loss_sum"],
                             "connections_per_residue_violation_mask": connection["per_residue_violation_mask"],
                             "clashes_mean_loss": clashes["mean_loss"], "clashes_per_atom_loss_sum": clashes["per_atom_loss_sum"],
                             "clashes_per_atom_clash_mask": clashes["per_atom_clash_mask"]},
        "within_residues": {"per_atom_loss_sum": within["per_atom_loss_sum"], "per_atom_violations": within["per_atom_violations"]},
        "total_per_residue_violations_mask": per_residue,
    }


def find_structural_violations_np(batch, atom14_pred_positions, config):
    """``find_structural_violations`` on numpy inputs, numpy out (the relaxation loop works in numpy)."""
    import numpy as np
    as_t = lambda x: torch.as_tensor(x)
    out = find_structural_violations(tree_map(as_t, dict(batch), np.ndarray), as_t(atom14_pred_positions), **config)
    return tensor_tree_map(lambda t: t.detach().cpu().numpy(), out)


def extreme_ca_ca_distance_violations(pred_atom_positions, pred_atom_mask, residue_index, max_angstrom_tolerance=1.5, eps=1e-6):
    """Fraction of consecutive residue pairs (no chain break between them, both CA present) whose CA-CA distance is more
    than ``max_angstrom_tolerance`` above the ideal 3.80 A; positions are atom14 / atom37 (CA is slot 1 in both)."""
    this_ca, next_ca = pred_atom_positions[..., :-1, 1, :], pred_atom_positions[..., 1:, 1, :]
    pair_mask = pred_atom_mask[..., :-1, 1] * pred_atom_mask[..., 1:, 1]
    pair_mask = pair_mask * ((residue_index[..., 1:] - residue_index[..., :-1]) == 1.0).to(pair_mask.dtype)
    dist = torch.sqrt(eps + torch.sum((this_ca - next_ca) ** 2, dim=-1))
    return masked_mean(pair_mask, ((dist - rc.ca_ca) > max_angstrom_tolerance).to(pair_mask.dtype), -1)


def compute_violation_metrics(batch, atom14_pred_positions, violations):
    """Per-structure summaries of ``find_structural_violations``: fractions of residues with a broken peptide bond, a
    clash, a within-residue violation or any of them, and the fraction of stretched CA-CA steps."""
    between, within = violations["between_residues"], violations["within_residues"]
    seq_mask = batch["seq_mask"]
    return {
        "violations_extreme_ca_ca_distance": extreme_ca_ca_distance_violations(atom14_pred_positions, batch["atom14_atom_exists"],
                                                                                batch["residue_index"]),
        "violations_between_residue_bond": masked_mean(seq_mask, between["connections_per_residue_violation_mask"], dim=-1),
        "violations_between_residue_clash": masked_mean(seq_mask, torch.max(between["clashes_per_atom_clash_mask"], dim=-1)[0], dim=-1),
        "violations_within_residue": masked_mean(seq_mask, torch.max(within["per_atom_violations"], dim=-1)[0], dim=-1),
        "violations_per_residue": masked_mean(seq_mask, violations["total_per_residue_violations_mask"], dim=-1),
    }


def compute_violation_metrics_np(batch, atom14_pred_positions, violations):
    import numpy as np
    as_t = lambda x: torch.as_tensor(x)
    out = compute_violation_metrics(tree_map(as_t, dict(batch), np.ndarray), as_t(atom14_pred_positions),
                                    tree_map(as_t, violations, np.ndarray))
    return {k: v.detach().cpu().numpy() for k, v in out.items()}


def torsion_angle_loss(a, a_gt, a_alt_gt):
    """Algorithm 27 on raw angle predictions ``a [*, N, 7, 2]``: squared chord distance of the normalised prediction to
    the nearer of the true and the pi-shifted ("alt") angle, plus 0.02 x the deviation of the raw norm from 1."""
    norm = torch.norm(a, dim=-1)
    unit = a / norm.unsqueeze(-1)
    d_gt = torch.sum((unit - a_gt) ** 2, dim=-1)
    d_alt = torch.sum((unit - a_alt_gt) ** 2, dim=-1)
    return torch.mean(torch.minimum(d_gt, d_alt), dim=(-1, -2)) + 0.02 * torch.mean(torch.abs(norm - 1), dim=(-1, -2))


def compute_drmsd(structure_1, structure_2, mask=None):
    """Distance-matrix RMSD of two point sets ``[*, N, 3]``: root mean square difference of all pairwise distances."""
    if mask is not None:
        structure_1 = structure_1 * mask[..., None]
        structure_2 = structure_2 * mask[..., None]
    d1 = torch.cdist(structure_1, structure_1)
    d2 = torch.cdist(structure_2, structure_2)
    sq = torch.sum((d1 - d2) ** 2, dim=(-1, -2))
    n = d1.shape[-1] if mask is None else torch.sum(mask, dim=-1)
    n = torch.as_tensor(n, dtype=sq.dtype, device=sq.device)
    return torch.sqrt(torch.where(n > 1, sq / (n * (n - 1)).clamp(min=1), torch.zeros_like(sq)))


def compute_drmsd_np(structure_1, structure_2, mask=None):
    return compute_drmsd(torch.as_tensor(structure_1), torch.as_tensor(structure_2), None if mask is None else torch.as_tensor(mask))


def violation_loss(violations, atom14_atom_exists, eps=1e-6, **kwargs):
    num_atoms = torch.sum(atom14_atom_exists)
    l_clash = torch.sum(violations["between_residues"]["clashes_per_atom_loss_sum"] + violations["within_residues"]["per_atom_loss_sum"])
    l_clash = l_clash / (eps + num_atoms)
    return (violations["between_residues"]["bonds_c_n_loss_mean"] + violations["between_residues"]["angles_ca_c_n_loss_mean"] +
            violations["between_residues"]["angles_c_n_ca_loss_mean"] + l_clash)


def compute_renamed_ground_truth(batch, atom14_pred_positions, eps=1e-10):
    """Chooses, per residue, the naming of symmetric side-chain atoms that is closer to the prediction (Algorithm 26)."""
    def dmat(x):
        return torch.sqrt(eps + torch.sum((x[..., None, :, None, :] - x[..., None, :, None, :, :]) ** 2, dim=-1))

    pred_dists = dmat(atom14_pred_positions)
    gt_dists = dmat(batch["atom14_gt_positions"])
    alt_gt_dists = dmat(batch["atom14_alt_gt_positions"])
    lddt_ = torch.sqrt(eps + (pred_dists - gt_dists) ** 2)
    alt_lddt = torch.sqrt(eps + (pred_dists - alt_gt_dists) ** 2)
    atom14_gt_exists = batch["atom14_gt_exists"]
    ambiguous = batch["atom14_atom_is_ambiguous"]
    mask = atom14_gt_exists[..., None, :, None] * ambiguous[..., None, :, None] * atom14_gt_exists[..., None, :, None, :] * \
        (1.0 - ambiguous[..., None, :, None, :])
    per_res_lddt = torch.sum(mask * lddt_, dim=(-1, -2, -3))
    alt_per_res_lddt = torch.sum(mask * alt_lddt, dim=(-1, -2, -3))
    alt_naming_is_better = (alt_per_res_lddt < per_res_lddt).type(atom14_pred_positions.dtype)
    renamed_positions = (1.0 - alt_naming_is_better[..., None, None]) * batch["atom14_gt_positions"] + \
        alt_naming_is_better[..., None, None] * batch["atom14_alt_gt_positions"]
    renamed_mask = (1.0 - alt_naming_is_better[..., None]) * batch["atom14_gt_exists"] + alt_naming_is_better[..., None] * batch["atom14_alt_gt_exists"]
    return {"alt_naming_is_better": alt_naming_is_better, "renamed_atom14_gt_positions": renamed_positions,
            "renamed_atom14_gt_exists": renamed_mask}


class AlphaFoldLoss(nn.Module):
    """Weighted sum of the loss terms configured in ``config`` (``config.loss`` of ``model_config``)."""

    def __init__(self, config):
        super().__init__()
        self.config = config

    def forward(self, out, batch, _return_breakdown=False):
        if "violation" not in out.keys():
            out["violation"] = find_structural_violations(batch, out["sm"]["positions"][-1], **self.config.violation)
        if "renamed_atom14_gt_positions" not in out.keys():
            batch.update(compute_renamed_ground_truth(batch, out["sm"]["positions"][-1]))
        loss_fns = {
            "distogram": lambda: distogram_loss(logits=out["distogram_logits"], **{**batch, **self.config.distogram}),
            "experimentally_resolved": lambda: experimentally_resolved_loss(logits=out["experimentally_resolved_logits"],
                                                                            **{**batch, **self.config.experimentally_resolved}),
            "fape": lambda: fape_loss(out, batch, self.config.fape),
            "lddt": lambda: lddt_loss(logits=out["lddt_logits"], all_atom_pred_pos=out["final_atom_positions"], **{**batch, **self.config.lddt}),
            "masked_msa": lambda: masked_msa_loss(logits=out["masked_msa_logits"], **{**batch, **self.config.masked_msa}),
            "supervised_chi": lambda: supervised_chi_loss(out["sm"]["angles"], out["sm"]["unnormalized_angles"],
                                                          **{**batch, **self.config.supervised_chi}),
            "violation": lambda: violation_loss(out["violation"], **batch),
        }
        if self.config.tm.enabled:
            loss_fns["tm"] = lambda: tm_loss(logits=out["tm_logits"], **{**batch, **out, **self.config.tm})
        cum_loss = 0.0
        losses = {}
        for name, fn in loss_fns.items():
            weight = self.config[name].weight
            loss = fn()
            if loss.is_cuda and torch.cuda.is_current_stream_capturing():
                # no host read inside a CUDA-graph capture: a non-finite term is replaced on the device
                loss = torch.where(torch.isfinite(loss), loss, torch.zeros_like(loss))
            elif torch.isnan(loss) or torch.isinf(loss):
                logging.warning("%s loss is NaN. Skipping...", name)
                loss = loss.new_tensor(0.0, requires_grad=True)
            cum_loss = cum_loss + weight * loss
            losses[name] = loss.detach().clone()
        losses["unscaled_loss"] = cum_loss.detach().clone()
        seq_len = torch.mean(batch["seq_length"].float())
        crop_len = batch["aatype"].shape[-1]
        cum_loss = cum_loss * torch.sqrt(torch.clamp(seq_len, max=float(crop_len)))      # min(seq_len, crop) without a host read
        losses["loss"] = cum_loss.detach().clone()
        if not _return_breakdown:
            return cum_loss
        return cum_loss, losses


# confidence summaries live with the heads that produce their logits; fastfold/model/hub/loss.py:1437-1532 defines them here too
from ..nn.heads import compute_plddt, compute_predicted_aligned_error, compute_tm  # noqa: E402,F401
