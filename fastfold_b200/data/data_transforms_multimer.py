"""Tensor-level feature transforms of the multimer pipeline and the transform list that applies them
(roles of fastfold/data/data_transforms_multimer.py and input_pipeline_multimer.py).

Differences from the monomer pipeline: cluster centres are drawn by Gumbel-max sampling biased by ``cluster_bias_mask``
(the query row always wins), the BERT-style corruption draws from the MSA profile of the whole (merged) alignment,
``target_feat`` is a plain 21-class one-hot, and MSA rows of the paired block count like any other row.
"""
import numpy as np
import torch

from . import data_transforms as dt

MSA_KEYS = ("msa", "deletion_matrix", "msa_mask", "bert_mask", "cluster_bias_mask")


def make_msa_profile(batch):
    """Profile over the 22 HH-suite classes of the whole alignment (masked mean)."""
    oh = dt.make_one_hot(batch["msa"], 22)
    mask = batch["msa_mask"][..., None]
    batch["msa_profile"] = (oh * mask).sum(0) / (mask.sum(0) + 1e-4)       # same smoothing as the reference's masked_mean
    return batch


def gumbel_noise(shape, device=None, eps=1e-6, generator=None):
    """Samples of the standard Gumbel distribution: ``-log(-log(U))`` with ``U`` uniform on (0, 1)."""
    u = torch.rand(tuple(shape), dtype=torch.float32, device=device, generator=generator)
    return -torch.log(-torch.log(u + eps) + eps)


def gumbel_max_sample(logits, generator=None):
    """One draw from ``softmax(logits)`` along the last axis, one-hot (argmax of the logits plus Gumbel noise)."""
    z = gumbel_noise(logits.shape, device=logits.device, generator=generator)
    return torch.nn.functional.one_hot(torch.argmax(logits + z, dim=-1), logits.shape[-1])


def gumbel_argsort_sample_idx(logits, generator=None):
    """A random permutation of the indices: sampling without replacement with probabilities ``softmax(logits)`` -
    the order of the logits after Gumbel noise was added, largest first."""
    z = gumbel_noise(logits.shape, device=logits.device, generator=generator)
    return torch.argsort(logits + z, dim=-1, descending=True)


def sample_msa(batch, max_seq, max_extra_msa_seq, seed=None, inf=1e6):
    """Gumbel-max sampling of ``max_seq`` cluster centres; the next ``max_extra_msa_seq`` rows become the extra MSA.
    Rows without any residue (padding) score ``-inf`` and come last; rows flagged in ``cluster_bias_mask`` (default: the
    first row) score ``+inf`` and are always among the centres (fastfold/data/data_transforms_multimer.py:253-289)."""
    g = torch.Generator()
    g.manual_seed(seed) if seed is not None else g.seed()
    logits = (torch.clamp(batch["msa_mask"].sum(-1), 0.0, 1.0) - 1.0) * inf
    if "cluster_bias_mask" in batch:
        bias = batch["cluster_bias_mask"].to(logits.dtype)
    else:
        bias = torch.nn.functional.pad(torch.zeros(batch["msa"].shape[0] - 1), (1, 0), value=1.0)
    order = gumbel_argsort_sample_idx(logits + bias * inf, generator=g)
    sel, extra = order[:max_seq], order[max_seq:max_seq + max_extra_msa_seq]
    for k in ("msa", "deletion_matrix", "msa_mask", "bert_mask"):
        if k in batch:
            batch["extra_" + k] = batch[k][extra]
            batch[k] = batch[k][sel]
    if "cluster_bias_mask" in batch:
        batch["cluster_bias_mask"] = batch["cluster_bias_mask"][sel]
    return batch


def make_masked_msa(batch, config, replace_fraction, seed=None, eps=1e-6):
    """BERT-style corruption of the cluster centres (fastfold/data/data_transforms_multimer.py:70-120): a fraction of the
    positions is redrawn from a mixture of the uniform amino-acid distribution, the alignment profile, the residue itself
    and a mask token; the replacement is a Gumbel-max draw from the seeded generator.  Positions outside ``msa_mask`` are
    never corrupted and end up as class 0.  Which positions are redrawn comes from the same generator here (the reference
    takes them from the global random state)."""
    g = torch.Generator()
    g.manual_seed(seed) if seed is not None else g.seed()
    random_aa = torch.tensor([0.05] * 20 + [0.0, 0.0], dtype=torch.float32)
    probs = config.uniform_prob * random_aa + config.profile_prob * batch["msa_profile"] + config.same_prob * dt.make_one_hot(batch["msa"], 22)
    mask_prob = 1.0 - config.profile_prob - config.same_prob - config.uniform_prob
    probs = torch.nn.functional.pad(probs, (0, 1), value=mask_prob)
    drawn = torch.argmax(gumbel_max_sample(torch.log(probs + eps), generator=g), dim=-1)
    mask_position = (torch.rand(batch["msa"].shape, generator=g) < replace_fraction) & (batch["msa_mask"] > 0)
    # a ``bert_mask`` that comes with the features marks the positions that may be scored at all (a row's own chain)
    scored = mask_position.to(torch.float32)
    batch["bert_mask"] = batch["bert_mask"].to(torch.float32) * scored if "bert_mask" in batch else scored
    batch["true_msa"] = batch["msa"]
    batch["msa"] = torch.where(mask_position, drawn, batch["msa"]) * batch["msa_mask"].to(batch["msa"].dtype)
    return batch


def nearest_neighbor_clusters(batch, gap_agreement_weight=0.0):
    """Profile and mean deletion count of every cluster: each extra row is softly assigned to the centre it agrees with
    most (gap agreement down-weighted, the mask token never counted), weighted by the number of positions both rows cover,
    and a centre's summary is normalised by its total weight plus one for the centre itself - AlphaFold-Multimer's
    definition, per centre rather than per position as in the monomer pipeline
    (fastfold/data/data_transforms_multimer.py:124-180)."""
    weights = torch.tensor([1.0] * 21 + [gap_agreement_weight] + [0.0])
    msa_mask, extra_mask = batch["msa_mask"].float(), batch["extra_msa_mask"].float()
    centre = dt.make_one_hot(batch["msa"], 23) * msa_mask[..., None]                 # [n, r, 23]
    extra = dt.make_one_hot(batch["extra_msa"], 23) * extra_mask[..., None]          # [m, r, 23]
    agreement = torch.einsum("nrc,mrc->nm", weights * centre, extra)
    assign = torch.softmax(1e3 * agreement, dim=0) * (msa_mask @ extra_mask.t())     # [n, m]
    total = assign.sum(-1) + 1.0
    batch["cluster_profile"] = (torch.einsum("nm,mrc->nrc", assign, extra) + centre) / total[:, None, None]
    batch["cluster_deletion_mean"] = (assign @ (extra_mask * batch["extra_deletion_matrix"].float()) + batch["deletion_matrix"]) / total[:, None]
    return batch


def create_msa_feat(batch):
    """``msa_feat`` (49 channels) from the sampled rows and their cluster summaries."""
    msa_1hot = dt.make_one_hot(batch["msa"], 23)
    has_deletion = torch.clamp(batch["deletion_matrix"], 0.0, 1.0)[..., None]
    deletion_value = (torch.atan(batch["deletion_matrix"] / 3.0) * (2.0 / np.pi))[..., None]
    deletion_mean_value = (torch.atan(batch["cluster_deletion_mean"] / 3.0) * (2.0 / np.pi))[..., None]
    batch["msa_feat"] = torch.cat([msa_1hot, has_deletion, deletion_value, batch["cluster_profile"], deletion_mean_value], dim=-1)
    return batch


def create_target_feat(batch):
    batch["target_feat"] = dt.make_one_hot(batch["aatype"], 21)
    return batch


def create_extra_msa_feature(batch, num_extra_msa):
    """Trims the extra MSA and derives ``extra_has_deletion`` / ``extra_deletion_value`` (the 25-channel feature itself is
    assembled inside the model)."""
    for k in ("extra_msa", "extra_deletion_matrix", "extra_msa_mask"):
        batch[k] = batch[k][:num_extra_msa]
    batch["extra_has_deletion"] = torch.clamp(batch["extra_deletion_matrix"], 0.0, 1.0)
    batch["extra_deletion_value"] = torch.atan(batch["extra_deletion_matrix"] / 3.0) * (2.0 / np.pi)
    return batch


def process_tensors(batch, common_cfg, mode_cfg, seed=0):
    """One recycling iteration's worth of model features from the merged multimer example (tensors, no batch dim)."""
    batch = dict(batch)
    for k in ("msa", "aatype", "asym_id", "entity_id", "sym_id", "residue_index"):
        if k in batch:
            batch[k] = batch[k].long()
    for k in ("deletion_matrix", "msa_mask", "seq_mask"):
        batch[k] = batch[k].float()
    batch = make_msa_profile(batch)
    batch = sample_msa(batch, mode_cfg.max_msa_clusters, mode_cfg.max_extra_msa, seed=seed)
    if "masked_msa" in common_cfg:
        # a different stream from the one that ordered the rows (fastfold/data/input_pipeline_multimer.py:68-74)
        batch = make_masked_msa(batch, common_cfg.masked_msa, mode_cfg.masked_msa_replace_fraction,
                                seed=None if seed is None else seed + 1)
    batch["extra_msa_mask"] = batch["extra_msa_mask"].float()
    batch["extra_deletion_matrix"] = batch["extra_deletion_matrix"].float()
    batch = nearest_neighbor_clusters(batch)
    batch = create_msa_feat(batch)
    batch = create_target_feat(batch)
    batch = create_extra_msa_feature(batch, mode_cfg.max_extra_msa)
    batch = dt.make_atom14_masks(batch)
    batch["msa_row_mask"] = batch["msa_mask"].sum(-1).clamp(0, 1)
    batch["extra_msa_row_mask"] = batch["extra_msa_mask"].sum(-1).clamp(0, 1)
    if "template_aatype" in batch:
        batch["template_mask"] = (batch["template_all_atom_mask"].sum((-1, -2)) > 0).float()
    return batch


def build_extra_msa_feat(batch):
    """``[N_extra, N_res, 25]``: one-hot of the un-clustered rows (23 classes), has-deletion flag, squashed deletion count
    ``atan(d / 3) * 2 / pi``, computed late because the one-hot is large (fastfold/data/data_transforms_multimer.py:222-249)."""
    dels = batch["extra_deletion_matrix"].float()
    one_hot = torch.nn.functional.one_hot(batch["extra_msa"].long(), 23).to(dels.dtype)
    has_del = dels.clamp(0.0, 1.0)[..., None]
    value = (torch.atan(dels / 3.0) * (2.0 / np.pi))[..., None]
    return torch.cat([one_hot, has_del, value], dim=-1)
