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


# ---------------------------------------------------------------------------
# Part 2: sequence / MSA features
# ---------------------------------------------------------------------------
def cast_to_64bit_ints(protein):
    for k, v in protein.items():
        if v.dtype == torch.int32:
            protein[k] = v.type(torch.int64)
    return protein


def make_one_hot(x, num_classes):
    return torch.nn.functional.one_hot(x.long(), num_classes).float()


def make_seq_mask(protein):
    protein["seq_mask"] = torch.ones(protein["aatype"].shape, dtype=torch.float32)
    return protein


def make_template_mask(protein):
    protein["template_mask"] = torch.ones(protein["template_aatype"].shape[0], dtype=torch.float32)
    return protein


def correct_msa_restypes(protein):
    """HHblits residue ids (alphabetical with gap) -> this package's residue order."""
    perm = torch.tensor(list(rc.MAP_HHBLITS_AATYPE_TO_OUR_AATYPE), dtype=torch.long)
    protein["msa"] = perm[protein["msa"].long()]
    return protein


def squeeze_features(protein):
    """One-hot aatype -> indices; drops the singleton dims the raw numpy features carry."""
    if protein["aatype"].dim() == 2:
        protein["aatype"] = torch.argmax(protein["aatype"], dim=-1)
    for k in ["domain_name", "msa", "num_alignments", "seq_length", "sequence", "superfamily", "deletion_matrix", "resolution",
              "between_segment_residues", "residue_index", "template_all_atom_mask"]:
        if k in protein and isinstance(protein[k], torch.Tensor) and protein[k].dim() > 0 and protein[k].shape[-1] == 1 and k not in ("msa", "deletion_matrix"):
            protein[k] = protein[k].squeeze(-1)
    for k in ["seq_length", "num_alignments"]:
        if k in protein and protein[k].dim() > 0:
            protein[k] = protein[k][0]
    return protein


@curry1
def randomly_replace_msa_with_unknown(protein, replace_proportion):
    msa_mask = torch.rand(protein["msa"].shape) < replace_proportion
    x_idx, gap_idx = 20, 21
    msa_mask = torch.logical_and(msa_mask, protein["msa"] != gap_idx)
    protein["msa"] = torch.where(msa_mask, torch.ones_like(protein["msa"]) * x_idx, protein["msa"])
    aatype_mask = torch.rand(protein["aatype"].shape) < replace_proportion
    protein["aatype"] = torch.where(aatype_mask, torch.ones_like(protein["aatype"]) * x_idx, protein["aatype"])
    return protein


@curry1
def sample_msa(protein, max_seq, keep_extra, seed=None):
    """Keeps the query plus a random subset of ``max_seq - 1`` other rows; the rest becomes the extra MSA."""
    num_seq = protein["msa"].shape[0]
    g = torch.Generator()
    if seed is not None:
        g.manual_seed(seed)
    else:
        g.seed()
    shuffled = torch.randperm(num_seq - 1, generator=g) + 1
    index_order = torch.cat((torch.tensor([0]), shuffled), dim=0)
    num_sel = min(max_seq, num_seq)
    sel_seq, not_sel_seq = torch.split(index_order, [num_sel, num_seq - num_sel])
    for k in MSA_FEATURE_NAMES:
        if k in protein:
            if keep_extra:
                protein["extra_" + k] = torch.index_select(protein[k], 0, not_sel_seq)
            protein[k] = torch.index_select(protein[k], 0, sel_seq)
    return protein


def make_all_atom_aatype(protein):
    """``all_atom_aatype`` is the residue type the all-atom ground truth is indexed by (same tensor as ``aatype``)."""
    protein["all_atom_aatype"] = protein["aatype"]
    return protein


def fix_templates_aatype(protein):
    """Template residue types arrive one-hot in the HHblits alphabet: to indices, then to this package's residue order."""
    t = protein["template_aatype"]
    if t.dim() == 3:                 # also with zero templates, so that the transforms after this one see [T, N]
        idx = t.argmax(dim=-1)
        table = torch.tensor(rc.MAP_HHBLITS_AATYPE_TO_OUR_AATYPE, dtype=torch.int64, device=idx.device)
        protein["template_aatype"] = table[idx]
    return protein


@curry1
def add_distillation_flag(protein, distillation):
    protein["is_distillation"] = distillation
    return protein


@curry1
def sample_msa_distillation(protein, max_seq):
    """Self-distillation examples are subsampled to ``max_seq`` rows before anything else sees the MSA."""
    if int(protein["is_distillation"]) == 1:
        protein = sample_msa(max_seq, keep_extra=False)(protein)
    return protein


@curry1
def block_delete_msa(protein, config, seed=None):
    """Training-time augmentation: removes ``num_blocks`` contiguous runs of MSA rows, each ``msa_fraction_per_block`` of
    the alignment long, never the query row.  ``config.randomize_num_blocks`` draws the number of runs uniformly from
    ``0 .. num_blocks``.  (Same augmentation as fastfold/data/data_transforms.py:245-276, stated with index sets.)"""
    num_seq = protein["msa"].shape[0]
    g = torch.Generator()
    if seed is not None:
        g.manual_seed(seed)
    else:
        g.seed()
    block_len = int(num_seq * float(config.msa_fraction_per_block))
    n_blocks = int(config.num_blocks)
    if getattr(config, "randomize_num_blocks", False):
        n_blocks = int(torch.randint(0, n_blocks + 1, (1,), generator=g))
    keep = torch.ones(num_seq, dtype=torch.bool)
    if block_len > 0 and n_blocks > 0:
        starts = torch.randint(0, num_seq, (n_blocks,), generator=g)
        rows = (starts[:, None] + torch.arange(block_len)[None, :]).clamp_(max=num_seq - 1).reshape(-1)
        keep[rows] = False
    keep[0] = True
    keep_indices = torch.nonzero(keep).reshape(-1)
    for k in MSA_FEATURE_NAMES:
        if k in protein:
            protein[k] = torch.index_select(protein[k], 0, keep_indices)
    return protein


@curry1
def add_constant_field(protein, key, value):
    protein[key] = torch.tensor(value, device=protein["msa"].device)
    return protein


def shaped_categorical(probs, epsilon=1e-10):
    """One categorical draw per leading index of ``probs [..., classes]``; returns the class indices ``[...]``."""
    flat = (probs + epsilon).reshape(-1, probs.shape[-1])
    return torch.multinomial(flat, 1).reshape(probs.shape[:-1])


def make_atom14_masks_np(batch):
    """``make_atom14_masks`` on a dict of numpy arrays (used by the relaxation code, which works in numpy)."""
    as_t = {k: torch.as_tensor(v) if isinstance(v, np.ndarray) else v for k, v in batch.items()}
    out = make_atom14_masks(as_t)
    return {k: v.numpy() if torch.is_tensor(v) else v for k, v in out.items()}


@curry1
def crop_extra_msa(protein, max_extra_msa):
    num_seq = protein["extra_msa"].shape[0]
    num_sel = min(max_extra_msa, num_seq)
    select_indices = torch.randperm(num_seq)[:num_sel]
    for k in MSA_FEATURE_NAMES:
        if "extra_" + k in protein:
            protein["extra_" + k] = torch.index_select(protein["extra_" + k], 0, select_indices)
    return protein


def delete_extra_msa(protein):
    for k in MSA_FEATURE_NAMES:
        protein.pop("extra_" + k, None)
    return protein


def make_msa_mask(protein):
    protein["msa_mask"] = torch.ones(protein["msa"].shape, dtype=torch.float32)
    protein["msa_row_mask"] = torch.ones(protein["msa"].shape[0], dtype=torch.float32)
    return protein


def make_hhblits_profile(protein):
    if "hhblits_profile" not in protein:
        protein["hhblits_profile"] = torch.mean(make_one_hot(protein["msa"], 22), dim=0)
    return protein


@curry1
def make_masked_msa(protein, config, replace_fraction):
    """BERT-style corruption: a fraction of positions is replaced by a draw from uniform / profile / same / mask token."""
    random_aa = torch.tensor([0.05] * 20 + [0.0, 0.0], dtype=torch.float32)
    categorical_probs = (config.uniform_prob * random_aa + config.profile_prob * protein["hhblits_profile"] +
                         config.same_prob * make_one_hot(protein["msa"], 22))
    pad_shapes = list(reduce(add, [(0, 0) for _ in range(len(categorical_probs.shape))]))
    pad_shapes[1] = 1
    mask_prob = 1.0 - config.profile_prob - config.same_prob - config.uniform_prob
    assert mask_prob >= 0.0
    categorical_probs = torch.nn.functional.pad(categorical_probs, pad_shapes, value=mask_prob)
    sh = protein["msa"].shape
    mask_position = torch.rand(sh) < replace_fraction
    counts = categorical_probs.reshape(-1, categorical_probs.shape[-1])
    bert_msa = torch.multinomial(counts + 1e-9, 1).reshape(sh)
    bert_msa = torch.where(mask_position, bert_msa, protein["msa"])
    protein["bert_mask"] = mask_position.to(torch.float32)
    protein["true_msa"] = protein["msa"]
    protein["msa"] = bert_msa
    return protein


@curry1
def nearest_neighbor_clusters(protein, gap_agreement_weight=0.0):
    """Assigns every extra sequence to the closest kept (cluster-centre) sequence by residue agreement."""
    weights = torch.cat([torch.ones(21), gap_agreement_weight * torch.ones(1), torch.zeros(1)], 0)
    msa_one_hot = make_one_hot(protein["msa"], 23)
    sample_one_hot = protein["msa_mask"][:, :, None] * msa_one_hot
    extra_msa_one_hot = make_one_hot(protein["extra_msa"], 23)
    extra_one_hot = protein["extra_msa_mask"][:, :, None] * extra_msa_one_hot
    num_seq, num_res, _ = sample_one_hot.shape
    extra_num_seq = extra_one_hot.shape[0]
    agreement = torch.matmul(torch.reshape(extra_one_hot, [extra_num_seq, num_res * 23]),
                             torch.reshape(sample_one_hot * weights, [num_seq, num_res * 23]).transpose(0, 1))
    protein["extra_cluster_assignment"] = torch.argmax(agreement, dim=1).to(torch.int64)
    return protein


def unsorted_segment_sum(data, segment_ids, num_segments):
    assert len(segment_ids.shape) == 1 and segment_ids.shape[0] == data.shape[0]
    segment_ids = segment_ids.view(segment_ids.shape[0], *((1,) * len(data.shape[1:]))).expand(data.shape)
    out = torch.zeros(num_segments, *data.shape[1:], dtype=data.dtype).scatter_add_(0, segment_ids, data.float() if data.dtype != torch.float32 else data)
    return out.type(data.dtype)


def summarize_clusters(protein):
    num_seq = protein["msa"].shape[0]

    def csum(x):
        return unsorted_segment_sum(x, protein["extra_cluster_assignment"], num_seq)

    mask = protein["extra_msa_mask"]
    mask_counts = 1e-6 + protein["msa_mask"] + csum(mask)
    msa_sum = csum(mask[:, :, None] * make_one_hot(protein["extra_msa"], 23)) + make_one_hot(protein["msa"], 23)
    protein["cluster_profile"] = msa_sum / mask_counts[:, :, None]
    del_sum = csum(mask * protein["extra_deletion_matrix"]) + protein["deletion_matrix"]
    protein["cluster_deletion_mean"] = del_sum / mask_counts
    return protein


def make_msa_feat(protein):
    """``msa_feat`` (49), ``target_feat`` (22) and the extra-MSA deletion features."""
    has_break = torch.clip(protein["between_segment_residues"].to(torch.float32), 0, 1)
    aatype_1hot = make_one_hot(protein["aatype"], 21)
    protein["target_feat"] = torch.cat([has_break.unsqueeze(-1), aatype_1hot], dim=-1)
    msa_1hot = make_one_hot(protein["msa"], 23)
    has_deletion = torch.clip(protein["deletion_matrix"], 0.0, 1.0)
    deletion_value = torch.atan(protein["deletion_matrix"] / 3.0) * (2.0 / np.pi)
    msa_feat = [msa_1hot, has_deletion.unsqueeze(-1), deletion_value.unsqueeze(-1)]
    if "cluster_profile" in protein:
        deletion_mean_value = torch.atan(protein["cluster_deletion_mean"] / 3.0) * (2.0 / np.pi)
        msa_feat.extend([protein["cluster_profile"], deletion_mean_value.unsqueeze(-1)])
    if "extra_deletion_matrix" in protein:
        protein["extra_has_deletion"] = torch.clip(protein["extra_deletion_matrix"], 0.0, 1.0)
        protein["extra_deletion_value"] = torch.atan(protein["extra_deletion_matrix"] / 3.0) * (2.0 / np.pi)
    protein["msa_feat"] = torch.cat(msa_feat, dim=-1)
    return protein


@curry1
def select_feat(protein, feature_list):
    return {k: v for k, v in protein.items() if k in feature_list}


@curry1
def crop_templates(protein, max_templates):
    for k, v in protein.items():
        if k.startswith("template_"):
            protein[k] = v[:max_templates]
    return protein


@curry1
def make_fixed_size(protein, shape_schema, msa_cluster_size, extra_msa_size, num_res=0, num_templates=0):
    """Pads every feature to the static shape given by the schema (placeholders replaced by the sizes passed in)."""
    from ..config import NUM_EXTRA_SEQ, NUM_MSA_SEQ, NUM_RES, NUM_TEMPLATES
    pad_size_map = {NUM_RES: num_res, NUM_MSA_SEQ: msa_cluster_size, NUM_EXTRA_SEQ: extra_msa_size, NUM_TEMPLATES: num_templates}
    for k, v in protein.items():
        if k == "extra_cluster_assignment":
            continue
        shape = list(v.shape)
        schema = shape_schema[k]
        assert len(shape) == len(schema), "Rank mismatch between shape and shape schema for %s: %s vs %s" % (k, shape, schema)
        pad_size = [pad_size_map.get(s2, None) or s1 for (s1, s2) in zip(shape, schema)]
        padding = [(0, p - v.shape[i]) for i, p in enumerate(pad_size)]
        padding.reverse()
        padding = list(itertools.chain(*padding))
        if padding:
            protein[k] = torch.nn.functional.pad(v, padding)
            protein[k] = torch.reshape(protein[k], pad_size)
    return protein


@curry1
def random_crop_to_size(protein, crop_size, max_templates, shape_schema, subsample_templates=False, seed=None):
    """Crops the residue axis (and the template axis) of every feature to ``crop_size`` at a random offset."""
    from ..config import NUM_RES, NUM_TEMPLATES
    g = torch.Generator()
    if seed is not None:
        g.manual_seed(seed)
    else:
        g.seed()
    seq_length = int(protein["seq_length"])
    num_templates = protein["template_mask"].shape[-1] if "template_mask" in protein else 0
    num_res_crop_size = min(seq_length, crop_size)

    def draw(upper):                                   # uniform on 0 .. upper inclusive
        return int(torch.randint(0, upper + 1, (1,), generator=g)[0])

    # Draw order and distributions of fastfold/data/data_transforms.py:1165-1184 (so that equal seeds give equal crops):
    # template window and permutation first; then the residue window - uniform over all positions for samples trained with
    # the clamped FAPE, otherwise uniform below a bound that is itself drawn uniformly, which favours early windows.
    templ_start, templates_select = 0, None
    if subsample_templates and num_templates:
        templ_start = draw(num_templates)
        templates_select = torch.randperm(num_templates, generator=g)
    num_templates_crop = min(num_templates - templ_start, max_templates)
    n = seq_length - num_res_crop_size
    if "use_clamped_fape" in protein and float(protein["use_clamped_fape"]) == 1.0:
        bound = n
    else:
        bound = n - draw(n)
    num_res_crop_start = draw(bound)
    for k, v in protein.items():
        if k not in shape_schema or ("template" not in k and NUM_RES not in shape_schema[k]):
            continue
        if k.startswith("template") and subsample_templates and templates_select is not None:
            v = v[templates_select]
        slices = []
        for dim_size, dim in zip(shape_schema[k], v.shape):
            is_res = dim_size == NUM_RES
            if dim_size == NUM_TEMPLATES and k.startswith("template"):
                start, size = templ_start, num_templates_crop
            else:
                start = num_res_crop_start if is_res else 0
                size = num_res_crop_size if is_res else dim
            slices.append(slice(start, start + size))
        protein[k] = v[tuple(slices)]
    protein["seq_length"] = protein["seq_length"].new_tensor(num_res_crop_size)
    return protein


def pseudo_beta_fn(aatype, all_atom_positions, all_atom_mask):
    """CB position (CA for glycine) and its mask (fastfold/data/data_transforms.py:353-376); one definition, in utils.feats."""
    from ..utils.feats import pseudo_beta_fn as fn
    return fn(aatype, all_atom_positions, all_atom_mask)


def get_chi_atom_indices():
    """``[21][4][4]`` nested list of atom37 indices of the atoms that define each chi angle; zeros where the residue type
    has no such angle, last row = unknown residue (fastfold/data/data_transforms.py:914-942)."""
    return _chi_atom_indices()
