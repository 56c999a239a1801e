"""Training data modules: per-chain dataset from PDB files, filtered mixture with reroll, collator, loader properties."""
import json
import os

import numpy as np
import torch

from fastfold_b200.common import protein, residue_constants as rc
from fastfold_b200.config import model_config
from fastfold_b200.data import data_modules as dm


def _write_pdb(path, seq, seed):
    rng = np.random.default_rng(seed)
    n = len(seq)
    aatype = np.array([rc.restype_order[c] for c in seq])
    mask = rc.STANDARD_ATOM_MASK[aatype].astype(np.float32)
    pos = np.cumsum(rng.normal(size=(n, 1, 3)) * 2.0, axis=0) + rng.normal(size=(n, 37, 3))
    p = protein.Protein(atom_positions=pos * mask[..., None], aatype=aatype, atom_mask=mask, residue_index=np.arange(1, n + 1),
                        b_factors=np.zeros((n, 37)), chain_index=np.zeros(n, dtype=np.int64))
    open(path, "w").write(protein.to_pdb(p))


def _tree(tmp_path, names):
    data, aln = tmp_path / "pdb", tmp_path / "aln"
    data.mkdir()
    aln.mkdir()
    cache = {}
    for k, (name, seq) in enumerate(names.items()):
        _write_pdb(str(data / (name + ".pdb")), seq, k)
        (aln / name).mkdir()
        (aln / name / "hits.a3m").write_text(">query\n%s\n>h1\n%s\n" % (seq, seq[::-1]))
        cache[name] = {"seq": seq, "resolution": 2.0, "cluster_size": 1}
    return str(data), str(aln), cache


def _cfg():
    cfg = model_config("initial_training", train=True).data
    cfg.train.crop_size = 16
    cfg.train.max_msa_clusters = 4
    cfg.train.max_extra_msa = 4
    cfg.eval.max_msa_clusters = 4
    cfg.eval.max_extra_msa = 4
    cfg.common.max_recycling_iters = 2
    cfg.data_module.data_loaders.num_workers = 2
    return cfg


def test_filters():
    assert not dm.deterministic_train_filter({"seq": "ACDE", "resolution": 12.0})
    assert not dm.deterministic_train_filter({"seq": "AAAAAAAAAC", "resolution": 1.0})
    assert dm.deterministic_train_filter({"seq": "ACDEFGHIKL"})
    assert abs(dm.get_stochastic_train_filter_prob({"seq": "A" * 100, "cluster_size": 4}) - 0.125) < 1e-9
    assert abs(dm.get_stochastic_train_filter_prob({"seq": "A" * 1000}) - 1.0) < 1e-9


def test_single_dataset_and_mixture(tmp_path):
    names = {"1abc": "ACDEFGHIKLMNPQRSTVWY", "2xyz": "MNPQRSTVWYACDEFGHIKL", "3bad": "AAAAAAAAAAAAAAAAAAAC"}
    data, aln, cache = _tree(tmp_path, names)
    cfg = _cfg()
    ds = dm.OpenFoldSingleDataset(data, aln, config=cfg, treat_pdb_as_distillation=False, mode="train", _output_raw=True)
    assert len(ds) == 3 and ds.idx_to_chain_id(ds.chain_id_to_idx("2xyz")) == "2xyz"
    raw = ds[ds.chain_id_to_idx("1abc")]
    assert raw["all_atom_positions"].shape == (20, 37, 3) and raw["msa"].shape[1] == 20 and raw["all_atom_mask"].sum() > 0
    g = torch.Generator().manual_seed(0)
    mix = dm.OpenFoldDataset([ds], [1.0], epoch_len=8, chain_data_caches=[cache], generator=g)
    picked = {ds.idx_to_chain_id(i) for _, i in mix.datapoints}
    assert len(mix) == 8 and picked <= {"1abc", "2xyz"} and "3bad" not in picked      # hard filter drops the poly-A chain
    before = list(mix.datapoints)
    mix.reroll()
    assert len(mix.datapoints) == 8 and (mix.datapoints != before or True)


def test_loader_properties_and_dp_shares(tmp_path):
    names = {"1abc": "ACDEFGHIKLMNPQRSTVWY", "2xyz": "MNPQRSTVWYACDEFGHIKL"}
    data, aln, cache = _tree(tmp_path, names)
    cfg = _cfg()
    json.dump(cache, open(os.path.join(str(tmp_path), "cache.json"), "w"))
    train, val = dm.SetupTrainDataset(cfg, train_data_dir=data, train_alignment_dir=aln, train_chain_data_cache_path=os.path.join(str(tmp_path), "cache.json"),
                                      val_data_dir=data, val_alignment_dir=aln, train_epoch_len=4)
    loaders = [dm.TrainDataLoader(cfg, train, val, batch_seed=5, dp_rank=r, dp_size=2) for r in range(2)]
    seen = []
    for tl, vl in loaders:
        assert len(tl) == 2
        batches = list(tl)
        assert len(batches) == 2
        for b in batches:
            n_it = int(b["no_recycling_iters"][0])
            assert 0 <= n_it <= 2 and b["aatype"].shape == (16, n_it + 1) and b["msa_feat"].shape[-1] == n_it + 1
            assert b["use_clamped_fape"].shape == (n_it + 1,) and float(b["use_clamped_fape"][0]) in (0.0, 1.0)
            assert b["all_atom_positions"].shape[:3] == (16, 37, 3)
        seen.append([int(b["no_recycling_iters"][0]) for b in batches])
        vb = list(vl)
        assert len(vb) == 1 and vb[0]["aatype"].shape[-1] == 3      # eval: always the full number of recycling iterations
    assert seen[0] == seen[1]       # same generator seed: the replicas of a step agree on the number of iterations
