"""Multimer tensor pipeline: the merged multi-chain example -> model features, one pass of the multimer transforms per
recycling iteration (fresh Gumbel draw of the cluster centres each), stacked on a trailing axis.

The transforms themselves are in ``data_transforms_multimer`` (``process_tensors`` applies one iteration's list in
order); this module gives them the entry points of fastfold/data/input_pipeline_multimer.py:26-136.
"""
import torch

from . import data_transforms as dt
from . import data_transforms_multimer as dtm
from .input_pipeline import compose, map_fn          # noqa: F401


def nonensembled_transform_fns(common_cfg, mode_cfg):
    """Once per example: integer / float casts, the profile of the whole alignment, atom14 <-> atom37 index maps."""
    def casts(batch):
        for k in ("msa", "aatype", "asym_id", "entity_id", "sym_id", "residue_index"):
            if k in batch:
                batch[k] = batch[k].long()
        for k in ("deletion_matrix", "msa_mask", "seq_mask"):
            if k in batch:
                batch[k] = batch[k].float()
        return batch
    return [casts, dtm.make_msa_profile, dt.make_atom14_masks]


def ensembled_transform_fns(common_cfg, mode_cfg, ensemble_seed):
    """Once per recycling iteration: cluster-centre draw, BERT-style masking, cluster summaries, ``msa_feat`` /
    ``target_feat``, extra-MSA trim."""
    fns = [lambda b: dtm.sample_msa(b, mode_cfg.max_msa_clusters, mode_cfg.max_extra_msa, seed=ensemble_seed)]
    if "masked_msa" in common_cfg:
        fns.append(lambda b: dtm.make_masked_msa(b, common_cfg.masked_msa, mode_cfg.masked_msa_replace_fraction, seed=ensemble_seed))

    def floats(batch):
        batch["extra_msa_mask"] = batch["extra_msa_mask"].float()
        batch["extra_deletion_matrix"] = batch["extra_deletion_matrix"].float()
        return batch

    def row_masks(batch):
        batch["msa_row_mask"] = batch["msa_mask"].sum(-1).clamp(0, 1)
        batch["extra_msa_row_mask"] = batch["extra_msa_mask"].sum(-1).clamp(0, 1)
        if "template_aatype" in batch:
            batch["template_mask"] = (batch["template_all_atom_mask"].sum((-1, -2)) > 0).float()
        return batch

    fns += [floats, dtm.nearest_neighbor_clusters, dtm.create_msa_feat, dtm.create_target_feat,
            lambda b: dtm.create_extra_msa_feature(b, mode_cfg.max_extra_msa), row_masks]
    return fns


def process_tensors_from_config(tensors, common_cfg, mode_cfg, seed=None):
    base_seed = torch.Generator().seed() % (2 ** 31) if seed is None else int(seed)
    tensors = compose(nonensembled_transform_fns(common_cfg, mode_cfg))(dict(tensors))
    n_recycle = int(tensors["no_recycling_iters"]) if "no_recycling_iters" in tensors else common_cfg.max_recycling_iters

    def one_iteration(i):
        d = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in tensors.items()}
        d = compose(ensembled_transform_fns(common_cfg, mode_cfg, base_seed + int(i)))(d)
        return {k: v for k, v in d.items() if torch.is_tensor(v) and v.numel() > 0}

    per_iter = [one_iteration(i) for i in range(n_recycle + 1)]
    keys = [k for k in per_iter[0] if all(k in d and d[k].shape == per_iter[0][k].shape for d in per_iter)]
    return {k: torch.stack([d[k] for d in per_iter], dim=-1) for k in keys}
