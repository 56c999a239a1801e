"""Monomer tensor pipeline: which feature transforms run, in which order, once per example and once per recycling
iteration.

``process_tensors_from_config(tensors, common_cfg, mode_cfg)`` takes the raw feature tensors of one example and
returns the model's feature dict with the recycling iterations stacked on a trailing axis:

* once per example (``nonensembled_transform_fns``): integer casts, HHblits -> own residue order, squeeze, sequence /
  MSA masks, the full-alignment profile, template fixes (residue order, mask, pseudo-beta, optionally torsion angles),
  atom14 <-> atom37 index maps and - for supervised modes - the ground-truth frames, torsions and chi angles;
* once per recycling iteration (``ensembled_transform_fns``): distillation subsampling, cluster-centre sampling,
  BERT-style masking, cluster profiles, extra-MSA crop, ``msa_feat`` / ``target_feat``, then either crop + pad to the
  static shapes of the schema or a plain cut of the template axis.

The number of iterations is ``no_recycling_iters`` of the example when present (the training loader samples it),
else ``common_cfg.max_recycling_iters``.  Same contract as fastfold/data/input_pipeline.py:23-208.
"""
import torch

from . import data_transforms as dt


def nonensembled_transform_fns(common_cfg, mode_cfg):
    fns = [dt.cast_to_64bit_ints, dt.correct_msa_restypes, dt.squeeze_features, dt.randomly_replace_msa_with_unknown(0.0),
           dt.make_seq_mask, dt.make_msa_mask, dt.make_hhblits_profile]
    if common_cfg.use_templates:
        fns += [dt.fix_templates_aatype, dt.make_template_mask, dt.make_pseudo_beta("template_")]
        if common_cfg.use_template_torsion_angles:
            fns.append(dt.atom37_to_torsion_angles("template_"))
    fns.append(dt.make_atom14_masks)
    if mode_cfg.supervised:
        fns += [dt.make_atom14_positions, dt.atom37_to_frames, dt.atom37_to_torsion_angles(""), dt.make_pseudo_beta(""),
                dt.get_backbone_frames, dt.get_chi_angles]
    return fns


def _max_extra_msa(common_cfg, mode_cfg):
    if "max_extra_msa" in mode_cfg:
        return mode_cfg.max_extra_msa
    return common_cfg.max_extra_msa if "max_extra_msa" in common_cfg else 0


def ensembled_transform_fns(common_cfg, mode_cfg, ensemble_seed, iteration_seed=None):
    """``iteration_seed``: seed of this iteration's cluster draw when the MSA is resampled per iteration (None: a fresh
    random draw, as in the reference); without resampling every iteration uses ``ensemble_seed``."""
    fns = []
    if "max_distillation_msa_clusters" in mode_cfg:
        fns.append(dt.sample_msa_distillation(mode_cfg.max_distillation_msa_clusters))
    n_clusters = mode_cfg.max_msa_clusters
    if common_cfg.reduce_msa_clusters_by_max_templates:
        n_clusters -= mode_cfg.max_templates
    # the same clusters in every iteration unless the configuration asks for a fresh draw per iteration
    fns.append(dt.sample_msa(n_clusters, keep_extra=True, seed=iteration_seed if common_cfg.resample_msa_in_recycling else ensemble_seed))
    if "masked_msa" in common_cfg:
        # before clustering, so that the cluster profiles carry nothing about the positions that were corrupted
        fns.append(dt.make_masked_msa(common_cfg.masked_msa, mode_cfg.masked_msa_replace_fraction))
    if common_cfg.msa_cluster_features:
        fns += [dt.nearest_neighbor_clusters(), dt.summarize_clusters]
    n_extra = _max_extra_msa(common_cfg, mode_cfg)
    fns.append(dt.crop_extra_msa(n_extra) if n_extra else dt.delete_extra_msa)
    fns.append(dt.make_msa_feat)
    schema = dict(common_cfg.feat)
    if mode_cfg.fixed_size:
        fns.append(dt.select_feat(list(schema)))
        if mode_cfg.crop_size:
            fns.append(dt.random_crop_to_size(mode_cfg.crop_size, mode_cfg.max_templates, schema, mode_cfg.subsample_templates,
                                              seed=ensemble_seed + 1))
            fns.append(dt.make_fixed_size(schema, n_clusters, n_extra, mode_cfg.crop_size, mode_cfg.max_templates))
        else:
            fns.append(dt.crop_templates(mode_cfg.max_templates))
            fns.append(_pad_to_example_length(schema, n_clusters, n_extra, mode_cfg.max_templates))
    else:
        fns.append(dt.crop_templates(mode_cfg.max_templates))
    return fns


def _pad_to_example_length(schema, n_clusters, n_extra, n_templates):
    """``fixed_size`` without a crop size (prediction): MSA / extra-MSA / template axes are padded to their static
    sizes, the residue axis keeps the length of the example."""
    def fn(protein):
        n_res = int(protein["aatype"].shape[0])
        has_templates = any(k.startswith("template_") for k in protein)
        return dt.make_fixed_size(schema, n_clusters, n_extra, n_res, n_templates if has_templates else 0)(protein)
    return fn


@dt.curry1
def compose(x, fs):
    for f in fs:
        x = f(x)
    return x


def map_fn(fun, x):
    """Applies ``fun`` to every element of ``x`` and stacks the resulting dicts on a new LAST axis."""
    per_item = [fun(elem) for elem in x]
    return {k: torch.stack([d[k] for d in per_item], dim=-1) for k in per_item[0]}


def process_tensors_from_config(tensors, common_cfg, mode_cfg, seed=None):
    ensemble_seed = torch.Generator().seed() % (2 ** 31) if seed is None else int(seed)
    tensors = compose(nonensembled_transform_fns(common_cfg, mode_cfg))(tensors)
    if "no_recycling_iters" in tensors:
        n_recycle = int(tensors["no_recycling_iters"])
    else:
        n_recycle = common_cfg.max_recycling_iters

    def one_iteration(i):
        d = {k: (v.clone() if torch.is_tensor(v) else v) for k, v in tensors.items()}
        d["ensemble_index"] = i
        it_seed = None
        if seed is not None:                                  # reproducible examples: every draw derives from ``seed``
            it_seed = ensemble_seed + int(i)
            torch.manual_seed(it_seed)                        # the transforms without a generator of their own
        return compose(ensembled_transform_fns(common_cfg, mode_cfg, ensemble_seed, it_seed))(d)

    return map_fn(one_iteration, torch.arange(n_recycle + 1))
