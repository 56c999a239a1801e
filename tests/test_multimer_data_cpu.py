"""Multimer feature assembly: assembly ids, species pairing, block-diagonal merging."""
import numpy as np

from fastfold_b200.common import residue_constants as rc
from fastfold_b200.data import msa_pairing as mp
from fastfold_b200.data.data_pipeline import DataPipeline, DataPipelineMultimer


def test_identifiers():
    assert mp.get_identifiers("tr|A0A146SKV9|A0A146SKV9_FUNHE/2-98 some text").species_id == "FUNHE"
    assert mp.get_identifiers("sp|P0C2L1|A3X1_LOXLA").species_id == "LOXLA"
    assert mp.get_identifiers("UniRef90_XYZ").species_id == ""


def _chain(seq, rows, species, ent):
    ids = lambda s: [rc.HHBLITS_AA_TO_ID[c] for c in s]
    n = len(seq)
    return {"aatype": np.eye(21)[[rc.restype_order_with_x[c] for c in seq]], "sequence": np.array([seq.encode()], dtype=object),
            "seq_length": np.array([n] * n), "residue_index": np.arange(n), "between_segment_residues": np.zeros(n, np.int32),
            "msa": np.array([ids(seq)] + [ids(r) for r in rows[:1]], dtype=np.int32), "deletion_matrix_int": np.zeros((1 + len(rows[:1]), n), np.int32),
            "num_alignments": np.array([2] * n), "msa_all_seq": np.array([ids(seq)] + [ids(r) for r in rows], dtype=np.int32),
            "deletion_matrix_int_all_seq": np.zeros((1 + len(rows), n), np.int32),
            "msa_species_identifiers_all_seq": np.array([b""] + [s.encode() for s in species], dtype=object)}


def test_pair_and_merge_heteromer():
    a = _chain("ACDEFGHIKL", ["ACDEFGHIKV", "ACDEYGHIKL", "AADEFGHIKL"], ["HUMAN", "MOUSE", "YEAST"], 1)
    b = _chain("MNPQRSTV", ["MNPQRSTA", "MNPQKSTV"], ["MOUSE", "HUMAN"], 2)
    chains = mp.add_assembly_features({"0_A": a, "1_B": b})
    assert sorted(chains) == ["A_1", "B_1"]
    table = mp.pair_sequences(mp.process_unmerged_features(list(chains.values())))
    # row 0 pairs the queries; HUMAN and MOUSE exist in both chains, YEAST only in the first
    assert table.shape == (3, 2) and (table[0] == 0).all()
    ex = mp.pair_and_merge(chains)
    n = 18
    assert ex["aatype"].shape == (n,) and ex["msa"].shape[1] == n
    assert list(np.unique(ex["asym_id"])) == [1, 2] and list(np.unique(ex["entity_id"])) == [1, 2] and list(np.unique(ex["sym_id"])) == [1]
    assert ex["seq_mask"].sum() == n
    # paired rows come first: 3 of them; the remaining rows are block-diagonal (gaps for the other chain)
    gap = mp.MSA_GAP_IDX
    tail = ex["msa"][3:]
    assert all(((row[:10] == gap).all() or (row[10:] == gap).all()) for row in tail)
    assert not any(((row[:10] == gap).all() or (row[10:] == gap).all()) for row in ex["msa"][:3])


def test_homomer_is_not_paired_and_pipeline(tmp_path):
    fasta = tmp_path / "c.fasta"
    fasta.write_text(">A first\nACDEFGHIKL\n>B second\nACDEFGHIKL\n")
    ex = DataPipelineMultimer(DataPipeline()).process_fasta(str(fasta))
    assert ex["aatype"].shape == (20,) and list(np.unique(ex["sym_id"])) == [1, 2] and list(np.unique(ex["entity_id"])) == [1]
    assert ex["msa"].shape[0] >= 512 and ex["msa"].shape[1] == 20


def test_multimer_tensor_pipeline():
    import torch
    from fastfold_b200.config import model_config
    from fastfold_b200.data import data_transforms_multimer as dtm
    a = _chain("ACDEFGHIKL", ["ACDEFGHIKV", "ACDEYGHIKL", "AADEFGHIKL"], ["HUMAN", "MOUSE", "YEAST"], 1)
    b = _chain("MNPQRSTV", ["MNPQRSTA", "MNPQKSTV"], ["MOUSE", "HUMAN"], 2)
    ex = mp.pair_and_merge(mp.add_assembly_features({"0_A": a, "1_B": b}))
    cfg = model_config("multimer")
    cfg.data.predict.max_msa_clusters = 3
    cfg.data.predict.max_extra_msa = 4
    tens = {k: torch.tensor(np.asarray(v)) for k, v in ex.items() if np.asarray(v).dtype != object}
    out = dtm.process_tensors(tens, cfg.data.common, cfg.data.predict, seed=1)
    assert out["msa_feat"].shape == (3, 18, 49) and out["target_feat"].shape == (18, 21)
    assert out["extra_msa"].shape[0] <= 4 and out["extra_has_deletion"].shape == out["extra_msa"].shape
    assert torch.isfinite(out["msa_feat"]).all()
    # the query row is always the first cluster centre
    assert (out["true_msa"][0] == tens["msa"][0]).all()
    prof = out["msa_feat"][..., 25:48]
    assert torch.allclose(prof.sum(-1)[out["msa_mask"] > 0], torch.ones_like(prof.sum(-1)[out["msa_mask"] > 0]), atol=1e-3)


def test_multimer_fasta_to_structure(tmp_path):
    """All chains of the FASTA file reach the model: features of a two-chain complex -> multimer model -> coordinates."""
    import torch
    from fastfold_b200.config import model_config
    from fastfold_b200.data.data_pipeline import FeaturePipeline
    from fastfold_b200.models.hub import AlphaFold
    from fastfold_b200.utils.inject_fastnn import inject_fastnn
    from fastfold_b200.common import protein
    fasta = tmp_path / "c.fasta"
    fasta.write_text(">A first\nACDEFGHIKL\n>B second\nMNPQRSTVWY\n")
    raw = DataPipelineMultimer(DataPipeline()).process_fasta(str(fasta))
    cfg = model_config("multimer")
    cfg.data.predict.max_msa_clusters = 8
    cfg.data.predict.max_extra_msa = 8
    cfg.data.common.max_recycling_iters = 1
    feats = FeaturePipeline(cfg.data).process_features(raw, mode="predict", seed=0)
    assert feats["aatype"].shape == (20, 2) and feats["msa_feat"].shape == (8, 20, 49, 2)
    assert sorted(set(feats["asym_id"][..., 0].tolist())) == [1, 2]
    cfg.model.evoformer_stack.no_blocks = 1
    cfg.model.extra_msa.extra_msa_stack.no_blocks = 1
    torch.manual_seed(0)
    model = inject_fastnn(AlphaFold(cfg)).eval()
    with torch.no_grad():
        out = model(feats)
    assert out["final_atom_positions"].shape == (20, 37, 3) and torch.isfinite(out["final_atom_positions"]).all()
    f = {"aatype": feats["aatype"][..., 0].numpy(), "residue_index": feats["residue_index"][..., 0].numpy(), "asym_id": feats["asym_id"][..., 0].numpy()}
    pdb = protein.to_pdb(protein.from_prediction(f, {k: v.numpy() for k, v in out.items() if isinstance(v, torch.Tensor)}))
    chains = {ln[21] for ln in pdb.splitlines() if ln.startswith("ATOM")}
    assert chains == {"A", "B"}


def test_lean_multimer_embedders_match_reference_modules():
    """``inject_fastnn`` swaps in the lean multimer embedders (table-lookup relative positions, stacked single-channel
    projections, in-place template accumulation); outputs equal the OpenFold-layout modules'."""
    import copy
    import torch
    from fastfold_b200.config import model_config
    from fastfold_b200.models.fastnn import embedders_multimer as fmm
    from fastfold_b200.models.hub import AlphaFold
    from fastfold_b200.utils.inject_fastnn import inject_fastnn
    from fastfold_b200.utils.synthetic import random_features
    cfg = model_config("multimer")
    cfg.model.evoformer_stack.no_blocks = 1
    cfg.model.extra_msa.extra_msa_stack.no_blocks = 1
    torch.manual_seed(0)
    base = AlphaFold(cfg).eval()
    with torch.no_grad():
        for p in base.parameters():
            if p.dim() >= 2 and float(p.abs().sum()) == 0.0:
                p.normal_(0.0, 0.05)
    fast = inject_fastnn(copy.deepcopy(base)).eval()
    assert isinstance(fast.input_embedder, fmm.InputEmbedderMultimer)
    assert isinstance(fast.template_embedder, fmm.TemplateEmbedderMultimer)
    feats = random_features(20, 6, 8, n_templ=2, n_recycle=0, seed=1, chains=[12, 8])
    one = {k: v[..., 0] for k, v in feats.items()}
    with torch.no_grad():
        m0, z0 = base.input_embedder(one)
        m1, z1 = fast.input_embedder(one)
        assert torch.allclose(m0, m1, atol=1e-5) and torch.allclose(z0, z1, atol=1e-5)
        out0, out1 = base(feats), fast(feats)
    assert torch.allclose(out0["final_atom_positions"], out1["final_atom_positions"], atol=5e-3)
    assert torch.allclose(out0["pair"], out1["pair"], atol=2e-3)


def test_cluster_bias_and_bert_masks_follow_the_block_structure():
    """fastfold/data/msa_pairing.py:287-330 and data_transforms_multimer.py:83-119, 253-289."""
    import torch
    from fastfold_b200.config import model_config
    from fastfold_b200.data import data_transforms_multimer as dtm
    a = _chain("ACDEFGHIKL", ["ACDEFGHIKV", "ACDEYGHIKL", "AADEFGHIKL"], ["HUMAN", "MOUSE", "YEAST"], 1)
    b = _chain("MNPQRSTV", ["MNPQRSTA", "MNPQKSTV"], ["MOUSE", "HUMAN"], 2)
    ex = mp.pair_and_merge(mp.add_assembly_features({"0_A": a, "1_B": b}))
    # paired: only the first row is pinned; paired rows may be scored everywhere, block rows only inside their own chain
    assert ex["cluster_bias_mask"][0] == 1 and ex["cluster_bias_mask"][1:].sum() == 0
    assert (ex["bert_mask"][:3] == 1).all()
    gap = mp.MSA_GAP_IDX
    for row, scored in zip(ex["msa"][3:], ex["bert_mask"][3:]):
        own = slice(0, 10) if (row[10:] == gap).all() else slice(10, 18)
        assert scored[own].all() and scored.sum() == (own.stop - own.start)
    # homo-dimer: copies of one sequence share their rows - the MSA is dense (both copies side by side), one pinned row
    dense = mp.pair_and_merge(mp.add_assembly_features({"0_A": _chain("ACDEFGHIKL", ["ACDEFGHIKV"], ["HUMAN"], 1),
                                                         "1_B": _chain("ACDEFGHIKL", ["ACDEFGHIKV"], ["HUMAN"], 1)}))
    assert dense["msa"].shape == (2, 20) and (dense["msa"][:, :10] == dense["msa"][:, 10:]).all() and (dense["bert_mask"] == 1).all()
    assert list(np.nonzero(dense["cluster_bias_mask"])[0]) == [0] and (dense["seq_length"] == 20).all()
    # two different chains without species-tagged rows: nothing to pair, one block per chain, each block's first row pinned
    def unpaired(seq, rows):
        return {k: v for k, v in _chain(seq, rows, ["HUMAN"] * len(rows), 1).items() if "_all_seq" not in k}
    h = mp.pair_and_merge(mp.add_assembly_features({"0_A": unpaired("ACDEFGHIKL", ["ACDEFGHIKV"]), "1_B": unpaired("MNPQRSTVWY", ["MNPQRSTVWA"])}))
    pinned = np.nonzero(h["cluster_bias_mask"])[0]
    assert len(pinned) == 2 and pinned[0] == 0 and (h["msa"][pinned[1]][:10] == gap).all()
    # sampling: pinned rows always come first, empty (padding) rows always last, whatever the seed
    padded = mp.pad_msa(h, 12)
    t = {k: torch.tensor(np.asarray(v)) for k, v in padded.items() if np.asarray(v).dtype != object}
    t["msa_mask"] = torch.cat([torch.ones(h["msa"].shape), torch.zeros(12 - h["msa"].shape[0], 20)])
    n_real = h["msa"].shape[0]
    for seed in range(5):
        s = dtm.sample_msa({k: v.clone() for k, v in t.items()}, max_seq=n_real, max_extra_msa_seq=4, seed=seed)
        assert s["msa_mask"].sum(-1).min() > 0 and s["extra_msa_mask"].sum() == 0          # every real row before any padding row
        first_two = {tuple(r.tolist()) for r in s["msa"][:2]}
        assert first_two == {tuple(h["msa"][p].tolist()) for p in pinned}
    # corruption: positions outside a row's own chain are never scored
    cfg = model_config("multimer")
    tens = {k: torch.tensor(np.asarray(v)) for k, v in ex.items() if np.asarray(v).dtype != object}
    tens = dtm.make_msa_profile(tens)
    out = dtm.make_masked_msa(tens, cfg.data.common.masked_msa, replace_fraction=0.9, seed=0)
    assert (out["bert_mask"] <= torch.tensor(ex["bert_mask"])).all() and out["bert_mask"].sum() > 0
