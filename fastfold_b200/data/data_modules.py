"""Datasets for ``train.py``: synthetic samples, and PDB-file structures with optional alignments.

Data parallelism: sample ``i`` of epoch ``e`` is drawn for DP rank ``r`` as global index ``i * dp_size + r`` (what the
reference gets from ``DistributedSampler``, data/data_modules.py:607-627); ranks of one DAP group share the sample.
Batch size is one sample per DP replica, features carry no batch dimension.
"""
import os

import numpy as np
import torch

from ..common import protein, residue_constants as rc
from ..utils.synthetic import random_features
from .data_pipeline import DataPipeline, FeaturePipeline


class SyntheticDataset:
    def __init__(self, n_res, n_seq, n_extra, n_recycle=3, length=64, seed=0, dp_rank=0, dp_size=1, uniform_recycling=True, n_templ=0):
        self.n_templ = n_templ
        self.n_res, self.n_seq, self.n_extra, self.n_recycle, self.length = n_res, n_seq, n_extra, n_recycle, length
        self.seed, self.dp_rank, self.dp_size, self.uniform_recycling = seed, dp_rank, dp_size, uniform_recycling

    def __len__(self):
        return self.length

    def get(self, epoch, i):
        s = self.seed + (epoch * self.length + i) * self.dp_size + self.dp_rank
        batch = random_features(self.n_res, self.n_seq, self.n_extra, n_templ=self.n_templ, n_recycle=self.n_recycle, seed=s, supervised=True)
        # the number of recycling iterations of a step is sampled uniformly and shared by all ranks of the step
        g = torch.Generator().manual_seed(self.seed + epoch * self.length + i)
        n = int(torch.randint(0, self.n_recycle + 1, (1,), generator=g)) if self.uniform_recycling else self.n_recycle
        batch["no_recycling_iters"] = torch.tensor([n])
        return batch


class StructureDataset:
    """``data_dir/<tag>.pdb`` ground-truth structures; alignments (``*.a3m`` / ``*.sto``) under ``alignment_dir/<tag>/``."""

    def __init__(self, data_dir, alignment_dir, data_config, mode="train", seed=0, dp_rank=0, dp_size=1):
        self.data_dir, self.alignment_dir, self.mode = data_dir, alignment_dir, mode
        self.tags = sorted(f[:-4] for f in os.listdir(data_dir) if f.endswith(".pdb"))
        if not self.tags:
            raise ValueError("no .pdb files in %s" % data_dir)
        self.pipeline = DataPipeline()
        self.features = FeaturePipeline(data_config)
        self.n_recycle = data_config.common.max_recycling_iters
        self.seed, self.dp_rank, self.dp_size = seed, dp_rank, dp_size

    def __len__(self):
        return max(1, len(self.tags) // self.dp_size)

    def get(self, epoch, i):
        idx = (i * self.dp_size + self.dp_rank) % len(self.tags)
        tag = self.tags[idx]
        prot = protein.from_pdb_string(open(os.path.join(self.data_dir, tag + ".pdb")).read())
        seq = "".join(rc.restypes_with_x[a] for a in prot.aatype)
        aln = os.path.join(self.alignment_dir, tag) if self.alignment_dir else None
        raw = dict(self.pipeline.process_sequence(seq, tag, aln))
        raw.update({"all_atom_positions": prot.atom_positions.astype(np.float32), "all_atom_mask": prot.atom_mask.astype(np.float32),
                    "resolution": np.array(1.0, np.float32), "use_clamped_fape": np.array(1.0, np.float32),
                    "is_distillation": np.array(0.0, np.float32)})
        feats = self.features.process_features(raw, self.mode, seed=self.seed + epoch * 100003 + idx)
        g = torch.Generator().manual_seed(self.seed + epoch * len(self) + i)
        feats["no_recycling_iters"] = torch.tensor([int(torch.randint(0, self.n_recycle + 1, (1,), generator=g))])
        return feats


# ---------------------------------------------------------------------------
# Training data modules: per-chain dataset, filtered mixture, collator, loader
# (same roles as fastfold/data/data_modules.py:34-639; no torch DataLoader subclassing, no DistributedSampler -
# data-parallel sharding follows this package's DAP x DP mesh)
# ---------------------------------------------------------------------------
import json
import logging
from typing import Any, List, Optional, Sequence


class OpenFoldSingleDataset(torch.utils.data.Dataset):
    """Chains of one data source.  ``alignment_dir`` holds one sub-directory per chain (``<file id>_<chain id>`` or
    ``<file id>``) with ``.a3m`` / ``.sto`` / ``.hhr`` files; ``data_dir`` holds ``<file id>.cif`` or ``.pdb`` (train /
    eval) or ``<name>/<name>.fasta`` (predict).  ``_output_raw`` returns the numpy feature dict (the collator then runs
    the tensor pipeline, so that worker processes do the expensive part in parallel)."""

    def __init__(self, data_dir, alignment_dir, template_mmcif_dir=None, max_template_date="2100-01-01", config=None,
                 kalign_binary_path="/usr/bin/kalign", max_template_hits=4, obsolete_pdbs_file_path=None,
                 template_release_dates_cache_path=None, shuffle_top_k_prefiltered=None, treat_pdb_as_distillation=True,
                 mapping_path=None, mode="train", _output_raw=False, _alignment_index=None):
        if mode not in ("train", "eval", "predict"):
            raise ValueError("mode must be one of train / eval / predict")
        self.data_dir, self.alignment_dir, self.config, self.mode = data_dir, alignment_dir, config, mode
        self.treat_pdb_as_distillation = treat_pdb_as_distillation
        self._output_raw = _output_raw
        self._alignment_index = _alignment_index
        if _alignment_index is not None:
            self._chain_ids = list(_alignment_index.keys())
        elif mapping_path is not None:
            self._chain_ids = [ln.strip() for ln in open(mapping_path) if ln.strip()]
        else:
            self._chain_ids = sorted(os.listdir(alignment_dir))
        self._index_of = {c: i for i, c in enumerate(self._chain_ids)}
        featurizer = None
        if template_mmcif_dir and os.path.isdir(template_mmcif_dir):
            from .templates import TemplateHitFeaturizer
            featurizer = TemplateHitFeaturizer(mmcif_dir=template_mmcif_dir, max_template_date=max_template_date, max_hits=max_template_hits,
                                               kalign_binary_path=kalign_binary_path, release_dates_path=template_release_dates_cache_path,
                                               obsolete_pdbs_path=obsolete_pdbs_file_path)
        self.data_pipeline = DataPipeline(template_featurizer=featurizer)
        self.feature_pipeline = None if _output_raw else FeaturePipeline(config)

    def chain_id_to_idx(self, chain_id):
        return self._index_of[chain_id]

    def idx_to_chain_id(self, idx):
        return self._chain_ids[int(idx)]

    def __len__(self):
        return len(self._chain_ids)

    def raw(self, idx):
        name = self.idx_to_chain_id(idx)
        aln, index = os.path.join(self.alignment_dir, name), None
        if self._alignment_index is not None:
            # all targets' search outputs live in concatenated files under alignment_dir; the index says where
            aln, index = self.alignment_dir, self._alignment_index[name]
        if self.mode == "predict":
            return self.data_pipeline.process_fasta(os.path.join(self.data_dir, name, name + ".fasta"), aln, _alignment_index=index)
        file_id, chain_id = (name.rsplit("_", 1) + [None])[:2] if "_" in name else (name, None)
        base = os.path.join(self.data_dir, file_id)
        if os.path.exists(base + ".cif"):
            from . import mmcif_parsing
            res = mmcif_parsing.parse(file_id=file_id, mmcif_string=open(base + ".cif").read())
            if res.mmcif_object is None:
                raise list(res.errors.values())[0]
            return self.data_pipeline.process_mmcif(res.mmcif_object, aln, chain_id, _alignment_index=index)
        if os.path.exists(base + ".core"):
            return self.data_pipeline.process_core(base + ".core", aln, _alignment_index=index)
        if os.path.exists(base + ".pdb"):
            return self.data_pipeline.process_pdb(base + ".pdb", aln, is_distillation=self.treat_pdb_as_distillation, chain_id=chain_id,
                                                  _alignment_index=index)
        raise ValueError("no .cif, .core or .pdb file for %r under %s" % (name, self.data_dir))

    def __getitem__(self, idx):
        data = self.raw(idx)
        if self._output_raw:
            return data
        # a fresh seed per item (from the global generator, so torch.manual_seed makes a run repeatable): row sampling, masking,
        # cropping and template subsampling must differ from sample to sample and from epoch to epoch
        seed = int(torch.randint(0, 2 ** 31 - 1, (1,)))
        return self.feature_pipeline.process_features(data, self.mode, seed=seed)


def deterministic_train_filter(entry, max_resolution=9.0, max_single_aa_prop=0.8):
    """Hard filters of AlphaFold's training set: resolution and single-residue dominance
    (fastfold/data/data_modules.py:227-246)."""
    res = entry.get("resolution")
    if res is not None and res > max_resolution:
        return False
    seq = entry["seq"]
    return max(seq.count(a) for a in set(seq)) / len(seq) <= max_single_aa_prop


def get_stochastic_train_filter_prob(entry):
    """Acceptance probability of a chain: inverse cluster size times a length term clamped to [256, 512] / 512."""
    p = 1.0
    cs = entry.get("cluster_size")
    if cs is not None and cs > 0:
        p /= cs
    return p * max(min(len(entry["seq"]), 512), 256) / 512.0


class OpenFoldDataset(torch.utils.data.Dataset):
    """Epoch of ``epoch_len`` samples drawn from several ``OpenFoldSingleDataset``s with the given mixture probabilities,
    each candidate passing the hard filters and an acceptance draw.  ``reroll()`` draws a new epoch.  Each source walks
    its own endless stream of shuffled indices, so no chain repeats before the source is exhausted."""

    def __init__(self, datasets, probabilities, epoch_len, chain_data_cache_paths=None, generator=None, _roll_at_init=True, chain_data_caches=None):
        self.datasets, self.probabilities, self.epoch_len = list(datasets), [float(p) for p in probabilities], int(epoch_len)
        self.generator = generator if generator is not None else torch.Generator()
        if chain_data_caches is None:
            chain_data_caches = [json.load(open(p)) if p else None for p in (chain_data_cache_paths or [None] * len(self.datasets))]
        self.chain_data_caches = chain_data_caches
        self._streams = [self._accepted(i) for i in range(len(self.datasets))]
        self.datapoints = []
        if _roll_at_init:
            self.reroll()

    def _shuffled(self, n):
        while True:
            for i in torch.randperm(n, generator=self.generator).tolist():
                yield i

    def _accepted(self, k):
        ds, cache = self.datasets[k], self.chain_data_caches[k]
        for idx in self._shuffled(len(ds)):
            entry = cache.get(ds.idx_to_chain_id(idx)) if cache is not None else None
            if entry is None:            # no metadata: nothing to filter on
                yield idx
                continue
            if not deterministic_train_filter(entry):
                continue
            if float(torch.rand((), generator=self.generator)) < get_stochastic_train_filter_prob(entry):
                yield idx

    def reroll(self):
        choice = torch.multinomial(torch.tensor(self.probabilities), self.epoch_len, replacement=True, generator=self.generator).tolist()
        self.datapoints = [(k, next(self._streams[k])) for k in choice]

    def __len__(self):
        return self.epoch_len

    def __getitem__(self, idx):
        k, i = self.datapoints[idx]
        return self.datasets[k][i]


class OpenFoldBatchCollator:
    """Runs the tensor feature pipeline on raw examples.  Batch size one yields tensors WITHOUT a batch dimension
    (fastfold/data/data_modules.py:379-384); larger batches are stacked on a new leading axis."""

    def __init__(self, config, stage="train"):
        self.stage = stage
        self.feature_pipeline = FeaturePipeline(config)
        self._n = 0

    def __call__(self, raw_prots):
        out = []
        for prot in raw_prots:
            self._n += 1
            out.append(self.feature_pipeline.process_features(prot, self.stage, seed=self._n))
        if len(out) == 1:
            return out[0]
        return {k: torch.stack([o[k] for o in out], dim=0) for k in out[0]}


class OpenFoldDataLoader:
    """Iterates a dataset in this rank's data-parallel share and adds the per-batch training properties: whether the
    backbone FAPE is clamped (``use_clamped_fape`` ~ Bernoulli(clamp_prob)) and the number of recycling iterations
    (uniform over 0..max when ``uniform_recycling``), truncating every feature's trailing recycling axis to that number
    + 1 (fastfold/data/data_modules.py:386-476).  All ranks share the generator seed, so the ranks of a step agree on
    both draws.  ``num_workers > 0`` fetches ahead on a thread pool."""

    def __init__(self, dataset, config, stage="train", generator=None, batch_size=1, num_workers=0, collate_fn=None, dp_rank=0, dp_size=1,
                 shuffle=False):
        if batch_size != 1:
            raise ValueError("Only support batch size equals to 1")
        self.dataset, self.config, self.stage = dataset, config, stage
        self.generator = generator if generator is not None else torch.Generator()
        self.num_workers, self.collate_fn = num_workers, collate_fn
        self.dp_rank, self.dp_size, self.shuffle = dp_rank, dp_size, shuffle
        sc = config[stage] if stage in config else config["eval"]
        n_rec = config.common.max_recycling_iters
        self.clamp_prob = config.supervised.clamp_prob if sc.supervised else None
        self.recycling_probs = [1.0 / (n_rec + 1)] * (n_rec + 1) if sc.get("uniform_recycling", False) else [0.0] * n_rec + [1.0]

    def __len__(self):
        return len(self.dataset) // self.dp_size

    def _add_batch_properties(self, batch):
        n_rec = int(torch.multinomial(torch.tensor(self.recycling_probs), 1, generator=self.generator))
        r = batch["aatype"].shape[-1]
        if self.clamp_prob is not None:
            clamped = float(torch.rand((), generator=self.generator) < self.clamp_prob)
            batch["use_clamped_fape"] = torch.full((r,), clamped)
        batch["no_recycling_iters"] = torch.full((r,), n_rec, dtype=torch.int64)
        return {k: v[..., :n_rec + 1] for k, v in batch.items()}

    def _fetch(self, i):
        item = self.dataset[i]
        return self.collate_fn([item]) if self.collate_fn is not None else item

    def __iter__(self):
        order = torch.randperm(len(self.dataset), generator=self.generator).tolist() if self.shuffle else list(range(len(self.dataset)))
        mine = order[self.dp_rank::self.dp_size][:len(self)]
        if self.num_workers > 0:
            from concurrent.futures import ThreadPoolExecutor
            with ThreadPoolExecutor(self.num_workers) as pool:
                ahead = [pool.submit(self._fetch, i) for i in mine[:self.num_workers]]
                for j in range(len(mine)):
                    batch = ahead.pop(0).result()
                    if j + self.num_workers < len(mine):
                        ahead.append(pool.submit(self._fetch, mine[j + self.num_workers]))
                    yield self._add_batch_properties(batch)
        else:
            for i in mine:
                yield self._add_batch_properties(self._fetch(i))


def SetupTrainDataset(config, template_mmcif_dir=None, max_template_date="2100-01-01", train_data_dir=None, train_alignment_dir=None,
                      train_chain_data_cache_path=None, distillation_data_dir=None, distillation_alignment_dir=None,
                      distillation_chain_data_cache_path=None, val_data_dir=None, val_alignment_dir=None, kalign_binary_path="/usr/bin/kalign",
                      train_mapping_path=None, distillation_mapping_path=None, obsolete_pdbs_file_path=None,
                      template_release_dates_cache_path=None, train_epoch_len=50000, _alignment_index_path=None, **kwargs):
    """``(train_dataset, eval_dataset or None)``; ``config`` is the ``data`` sub-tree of ``model_config``."""
    if train_data_dir is None or train_alignment_dir is None:
        raise ValueError("train_data_dir and train_alignment_dir must be specified")
    if val_data_dir is not None and val_alignment_dir is None:
        raise ValueError("If val_data_dir is specified, val_alignment_dir must be specified as well")
    index = json.load(open(_alignment_index_path)) if _alignment_index_path else None

    def make(**kw):
        return OpenFoldSingleDataset(template_mmcif_dir=template_mmcif_dir, max_template_date=max_template_date, config=config,
                                     kalign_binary_path=kalign_binary_path, template_release_dates_cache_path=template_release_dates_cache_path,
                                     obsolete_pdbs_file_path=obsolete_pdbs_file_path, _output_raw=True, **kw)

    sources = [make(data_dir=train_data_dir, alignment_dir=train_alignment_dir, mapping_path=train_mapping_path,
                    max_template_hits=config.train.max_template_hits, shuffle_top_k_prefiltered=config.train.get("shuffle_top_k_prefiltered"),
                    treat_pdb_as_distillation=False, mode="train", _alignment_index=index)]
    probs, caches = [1.0], [train_chain_data_cache_path]
    if distillation_data_dir is not None:
        sources.append(make(data_dir=distillation_data_dir, alignment_dir=distillation_alignment_dir, mapping_path=distillation_mapping_path,
                            max_template_hits=config.train.max_template_hits, treat_pdb_as_distillation=True, mode="train"))
        d = config.train.distillation_prob
        probs, caches = [1.0 - d, d], caches + [distillation_chain_data_cache_path]
    train = OpenFoldDataset(sources, probs, train_epoch_len, caches, _roll_at_init=False)
    val = None
    if val_data_dir is not None:
        val = make(data_dir=val_data_dir, alignment_dir=val_alignment_dir, mapping_path=None, max_template_hits=config.eval.max_template_hits,
                   mode="eval")
    return train, val


def TrainDataLoader(config, train_dataset, test_dataset=None, batch_seed=None, dp_rank=None, dp_size=None):
    """Loaders over ``SetupTrainDataset``'s datasets; every data-parallel replica reads its own share of the epoch (DAP
    ranks of one replica read the same samples)."""
    if config.data_module.data_loaders.batch_size != 1:
        raise ValueError("Only support batch size equals to 1")
    if dp_rank is None:
        from ..parallel import core
        dp_rank, dp_size = core.get_dp_rank(), core.get_dp_size()
    gen = torch.Generator()
    if batch_seed is not None:
        gen.manual_seed(batch_seed)
    workers = config.data_module.data_loaders.num_workers
    train_dataset.reroll()
    train = OpenFoldDataLoader(train_dataset, config, "train", gen, 1, workers, OpenFoldBatchCollator(config, "train"), dp_rank, dp_size)
    test = None
    if test_dataset is not None:
        test = OpenFoldDataLoader(test_dataset, config, "eval", gen, 1, workers, OpenFoldBatchCollator(config, "eval"), dp_rank, dp_size)
    return train, test
