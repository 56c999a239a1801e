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
