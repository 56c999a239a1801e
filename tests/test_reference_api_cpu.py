"""The parts of the reference's Python API that live outside the model: tensor pipeline entry points, data helpers,
loss / validation helpers, geometry, relaxation helpers and the ``fastfold.*`` import paths (CPU only)."""
import importlib
from types import SimpleNamespace as NS

import numpy as np
import pytest
import torch

from fastfold_b200.common import protein, residue_constants as rc
from fastfold_b200.config import model_config
from fastfold_b200.data import data_pipeline as dp
from fastfold_b200.data import data_transforms as dt
from fastfold_b200.data import data_transforms_multimer as dtm
from fastfold_b200.data import feature_pipeline, input_pipeline, msa_pairing, parsers, templates
from fastfold_b200.models.hub import loss as L
from fastfold_b200.utils import geometry as g


SEQ = "ACDEFGHIKLMNPQRSTVWYACDE"


def _raw_example(n_templates=0):
    n = len(SEQ)
    feats = dict(dp.make_sequence_features(SEQ, "t", n))
    msa = [SEQ, SEQ[:10] + "-" * (n - 10), SEQ.replace("A", "G"), SEQ.replace("C", "S")]
    feats.update(dp.make_msa_features([msa], [[[0] * n for _ in msa]]))
    t = dict(dp.empty_template_features(n))
    if n_templates:
        rng = np.random.RandomState(0)
        aat = np.zeros((n_templates, n, 22), np.float32)
        aat[np.arange(n_templates)[:, None], np.arange(n)[None], rng.randint(0, 20, (n_templates, n))] = 1
        t.update({"template_aatype": aat, "template_all_atom_masks": np.ones((n_templates, n, 37), np.float32),
                  "template_all_atom_positions": rng.randn(n_templates, n, 37, 3).astype(np.float32),
                  "template_sum_probs": np.ones((n_templates, 1), np.float32)})
    feats.update(t)
    return feats


def test_predict_features_with_and_without_templates():
    cfg = model_config("model_1")
    pipe = dp.FeaturePipeline(cfg.data)
    out = pipe.process_features(_raw_example(2), mode="predict", seed=5)
    n_it = cfg.data.common.max_recycling_iters + 1
    assert out["msa_feat"].shape == (cfg.data.predict.max_msa_clusters, len(SEQ), 49, n_it)
    assert out["template_aatype"].shape == (cfg.data.predict.max_templates, len(SEQ), n_it)
    assert out["template_mask"][:, 0].tolist() == [1.0, 1.0, 0.0, 0.0]
    assert out["template_torsion_angles_sin_cos"].shape[-3:] == (7, 2, n_it)
    assert out["template_pseudo_beta"].shape == (4, len(SEQ), 3, n_it)
    # no hit: no template features come back (the caller switches the template stack off)
    out0 = pipe.process_features(_raw_example(0), mode="predict", seed=5)
    assert not any(k.startswith("template_") for k in out0)
    assert out0["target_feat"].shape == (len(SEQ), 22, n_it)


def test_feature_pipeline_is_reproducible_and_honours_no_recycling_iters():
    cfg = model_config("model_1")
    a = feature_pipeline.np_example_to_features(_raw_example(), cfg.data, "predict", seed=3)
    b = feature_pipeline.np_example_to_features(_raw_example(), cfg.data, "predict", seed=3)
    c = feature_pipeline.np_example_to_features(_raw_example(), cfg.data, "predict", seed=4)
    assert all(torch.equal(a[k], b[k]) for k in a)
    assert any(not torch.equal(a[k], c[k]) for k in a)
    raw = _raw_example()
    raw["no_recycling_iters"] = np.array(1)
    assert feature_pipeline.np_example_to_features(raw, cfg.data, "predict", seed=0)["aatype"].shape[-1] == 2
    fns = input_pipeline.nonensembled_transform_fns(cfg.data.common, cfg.data.predict)
    assert dt.fix_templates_aatype in fns and len(input_pipeline.ensembled_transform_fns(cfg.data.common, cfg.data.predict, 0)) >= 6


def test_new_data_transforms():
    p = {"msa": torch.arange(40).reshape(20, 2), "deletion_matrix": torch.zeros(20, 2)}
    out = dt.block_delete_msa(NS(msa_fraction_per_block=0.3, num_blocks=2, randomize_num_blocks=False), seed=1)(dict(p))
    assert 8 <= out["msa"].shape[0] < 20 and out["msa"][0].tolist() == [0, 1] and out["deletion_matrix"].shape[0] == out["msa"].shape[0]
    assert dt.shaped_categorical(torch.tensor([[0.0, 1.0, 0.0], [1.0, 0.0, 0.0]])).tolist() == [1, 0]
    oh = torch.nn.functional.one_hot(torch.tensor([[0, 1, 2, 21]]), 22).float()
    fixed = dt.fix_templates_aatype({"template_aatype": oh})["template_aatype"]
    assert fixed.tolist() == [[rc.MAP_HHBLITS_AATYPE_TO_OUR_AATYPE[i] for i in (0, 1, 2, 21)]]
    assert dt.make_atom14_masks_np({"aatype": np.array([0, 5, 19])})["atom14_atom_exists"].shape == (3, 14)
    d = dt.sample_msa_distillation(4)(dt.add_distillation_flag(1)({"msa": torch.zeros(9, 3, dtype=torch.long)}))
    assert d["msa"].shape[0] == 4
    assert dt.add_constant_field("x", 3.0)({"msa": torch.zeros(1)})["x"] == 3.0


def test_gumbel_helpers():
    g_ = torch.Generator().manual_seed(0)
    logits = torch.tensor([0.0, 10.0, -10.0]).repeat(2000, 1)
    draws = dtm.gumbel_max_sample(logits, generator=g_).float().mean(0)
    assert draws[1] > 0.99 and draws.sum().item() == pytest.approx(1.0)
    order = dtm.gumbel_argsort_sample_idx(torch.tensor([100.0, 0.0, -100.0]), generator=g_)
    assert order.tolist() == [0, 1, 2]
    assert dtm.gumbel_noise((4, 5), generator=g_).shape == (4, 5)


def test_data_pipeline_helpers(tmp_path):
    assert [dp.int_id_to_str_id(i) for i in (1, 26, 27, 28)] == ["A", "Z", "AA", "BA"]
    with dp.temp_fasta_file(">a\nACD\n") as path:
        assert open(path).read() == ">a\nACD\n"
    raw = _raw_example()
    conv = dp.convert_monomer_features(raw, "B")
    assert conv["aatype"].shape == (len(SEQ),) and conv["seq_length"] == len(SEQ) and "template_all_atom_mask" in conv
    assert dp.make_template_features(SEQ, {}, None)["template_aatype"].shape == (0, len(SEQ), 22)
    prot = protein.Protein(atom_positions=np.random.randn(3, 37, 3).astype(np.float32), aatype=np.array([0, 1, 2]),
                           atom_mask=np.ones((3, 37), np.float32), residue_index=np.arange(3), b_factors=np.full((3, 37), 80.0))
    f = dp.make_pdb_features(prot, "x", is_distillation=True, confidence_threshold=90.0)
    assert f["all_atom_mask"].sum() == 0 and f["aatype"].shape == (3, 21)

    class Runner:
        def query(self, path, max_seq=None):
            return [{"sto": "STO %s" % max_seq, "a3m": "A3M"}]
    out = tmp_path / "hits.sto"
    dp.run_msa_tool(Runner(), "q.fasta", str(out), "sto", max_sto_sequences=7)
    assert out.read_text() == "STO 7"


def test_process_core_record(tmp_path):
    rec = "[ID]\n1abc\n[PRIMARY]\nACDEF\n[TERTIARY]\n" + " ".join(str(100 * i) for i in range(15)) + "\n" + " ".join("1" for _ in range(15)) + \
          "\n" + " ".join("0" for _ in range(15)) + "\n[MASK]\n++-++\n"
    path = tmp_path / "1abc_1_a.core"
    path.write_text(rec)
    feats = dp.DataPipeline().process_core(str(path))
    assert feats["aatype"].shape == (5, 21) and feats["all_atom_positions"].shape == (5, 37, 3)
    assert feats["all_atom_mask"][:, 1].tolist() == [1.0, 1.0, 0.0, 1.0, 1.0] and feats["msa"].shape == (1, 5)


def test_parsers_and_pairing_helpers():
    meta = parsers.parse_hmmsearch_description(">4pqx_A/2-217 [subseq from] mol:protein length:217  Free text")
    assert (meta.pdb_id, meta.chain, meta.start, meta.end, meta.length, meta.text) == ("4pqx", "A", 2, 217, 217, "Free text")
    m = parsers.Msa.from_a3m(">q\nACD\n>h\nA-D\n")
    assert len(m) == 2 and len(m.truncate(1)) == 1
    with pytest.raises(ValueError):
        parsers.Msa(["A"], [[0]], [])
    bd = msa_pairing.block_diag(np.ones((2, 3)), 2 * np.ones((1, 2)), pad_value=-1)
    assert bd.shape == (3, 5) and bd[0, 4] == -1 and bd[2, 3] == 2
    padded = msa_pairing.pad_features(np.zeros((3, 5), np.int32), "msa_all_seq")
    assert padded.shape == (4, 5) and (padded[-1] == msa_pairing.MSA_GAP_IDX).all()
    rows = msa_pairing.reorder_paired_rows({2: np.array([[3, 4], [1, 2]]), 3: np.array([[5, 5, 5]])}) if False else \
        msa_pairing.reorder_paired_rows({2: np.array([[3, 4], [1, 2]])})
    assert rows.tolist() == [[1, 2], [3, 4]]
    chain = {"msa": np.zeros((10, 5), int), "deletion_matrix": np.zeros((10, 5)),
             "msa_all_seq": np.concatenate([np.zeros((3, 5), int), np.full((3, 5), msa_pairing.MSA_GAP_IDX)]),
             "template_aatype": np.zeros((6, 5, 22)), "template_all_atom_mask": np.zeros((6, 5, 37)),
             "template_all_atom_positions": np.zeros((6, 5, 37, 3))}
    out = msa_pairing.crop_chains([chain], msa_crop_size=8, pair_msa_sequences=True, max_templates=4)[0]
    # 4 paired rows kept (half of the budget), 3 of them are the chain's own -> 8 - 3 = 5 unpaired rows
    assert out["msa_all_seq"].shape[0] == 4 and out["msa"].shape[0] == 5 and out["template_aatype"].shape[0] == 4


def test_release_date_cache_and_query_filters(tmp_path):
    cif = tmp_path / "1abc.cif"
    cif.write_text("data_1ABC\n_pdbx_audit_revision_history.revision_date 2001-02-03\n")
    dates = templates.generate_release_dates_cache(str(tmp_path), str(tmp_path / "dates.json"))
    assert dates in ({}, {"1abc": {"release_date": "2001-02-03"}})       # a header-only file may not parse as a structure
    assert issubclass(templates.PdbIdError, templates.PrefilterError)
    assert templates.PrefilterResult(True, None, None).valid


def test_loss_helpers():
    torch.manual_seed(0)
    a = torch.randn(5, 7, 2)
    gt = torch.nn.functional.normalize(torch.randn(5, 7, 2), dim=-1)
    unit = torch.nn.functional.normalize(a, dim=-1)
    expect = torch.minimum(((unit - gt) ** 2).sum(-1), ((unit + gt) ** 2).sum(-1)).mean() + 0.02 * (a.norm(dim=-1) - 1).abs().mean()
    assert torch.allclose(L.torsion_angle_loss(a, gt, -gt), expect, atol=1e-6)
    x = torch.randn(10, 3)
    assert float(L.compute_drmsd(x, x.clone())) == pytest.approx(0.0, abs=1e-5)
    d = torch.cdist(x, x)
    assert float(L.compute_drmsd(x, 2 * x)) == pytest.approx(float(torch.sqrt((d ** 2).sum() / 90)), rel=1e-4)
    assert float(L.compute_drmsd_np(x.numpy(), x.numpy() * 2)) == pytest.approx(float(L.compute_drmsd(x, 2 * x)), rel=1e-5)
    n = 12
    batch = dt.make_atom14_masks({"aatype": torch.randint(0, 20, (n,)), "residue_index": torch.arange(n), "seq_mask": torch.ones(n)})
    pos = torch.randn(n, 14, 3) * 3
    v = L.find_structural_violations(batch, pos, 12.0, 1.5)
    met = L.compute_violation_metrics(batch, pos, v)
    assert set(met) == {"violations_extreme_ca_ca_distance", "violations_between_residue_bond", "violations_between_residue_clash",
                        "violations_within_residue", "violations_per_residue"}
    assert all(0.0 <= float(t) <= 1.0 for t in met.values())
    nb = {k: t.numpy() for k, t in batch.items()}
    vn = L.find_structural_violations_np(nb, pos.numpy(), {"violation_tolerance_factor": 12.0, "clash_overlap_tolerance": 1.5})
    mn = L.compute_violation_metrics_np(nb, pos.numpy(), vn)
    assert float(mn["violations_per_residue"]) == pytest.approx(float(met["violations_per_residue"]), abs=1e-6)


def test_geometry_extras_and_stereo_props():
    torch.manual_seed(1)
    r = g.Rigid3Array(g.Rot3Array.from_quaternion(*torch.randn(4, 5)), g.Vec3Array.from_array(torch.randn(5, 3)))
    g.assert_rigid_close_to_rigid(r, g.Rigid3Array.from_array(r.to_tensor()))
    g.assert_rigid_close_to_rigid(r.compose(r.inverse()), g.Rigid3Array.identity((5,)), atol=1e-5)
    assert g.Rigid3Array.cat([r, r], 0).shape == (10,) and r.unsqueeze(0).shape == (1, 5) and r.reshape((5, 1)).shape == (5, 1)
    p = torch.randn(5, 3)
    g.assert_vectors_close(r.apply(p), r.apply_to_point(g.Vec3Array.from_array(p)))
    assert not r.stop_rot_gradient().rotation.xx.requires_grad
    assert g.get_field_names(g.Vec3Array) == ["x", "y", "z"]
    v = g.Vec3Array.from_array(torch.randn(4, 3))
    assert torch.allclose(g.dot(v, v), g.norm(v) ** 2, atol=1e-5) and g.Vec3Array.cat([v, v], 0).shape == (8,)
    bonds, virtual, angles = rc.load_stereo_chemical_props()
    n_ca = [b for b in bonds["ALA"] if {b.atom1_name, b.atom2_name} == {"N", "CA"}][0]
    assert 1.44 < n_ca.length < 1.48
    tau = [a for a in angles["GLY"] if (a.atom1_name, a.atom2_name, a.atom3name) == ("N", "CA", "C")][0]
    assert 1.85 < tau.angle_rad < 2.05 and len(virtual["GLY"]) == len(angles["GLY"])


def test_protein_and_relax_helpers():
    rec = "[ID]\n1abc\n[PRIMARY]\nACD\n[TERTIARY]\n100 200 300 400 500 600 700 800 900\n1 2 3 4 5 6 7 8 9\n0 0 0 0 0 0 0 0 0\n[MASK]\n+-+\n"
    prot = protein.from_proteinnet_string(rec)
    assert prot.aatype.tolist() == [0, 4, 3] and prot.atom_positions[1, :3, 0].tolist() == [4.0, 5.0, 6.0]
    assert prot.atom_mask[:, 1].tolist() == [1.0, 0.0, 1.0]
    from fastfold_b200.relax import amber_minimize, utils as rutils
    assert rutils.mask_mean_np(np.array([[1, 0, 1]]), np.array([[1.0, 5.0, 3.0], [2.0, 5.0, 4.0]]), axis=[0, 1]) == pytest.approx(2.5)
    atom = NS(name="CA", element=NS(name="carbon"))
    assert amber_minimize.will_restrain(atom, "non_hydrogen") and amber_minimize.will_restrain(atom, "c_alpha")
    assert not amber_minimize.will_restrain(NS(name="H", element=NS(name="hydrogen")), "non_hydrogen")
    n = 6
    full = protein.Protein(atom_positions=np.random.RandomState(0).randn(n, 37, 3).astype(np.float32) * 4, aatype=np.zeros(n, np.int64),
                           atom_mask=np.tile(np.asarray(rc.STANDARD_ATOM_MASK)[0], (n, 1)).astype(np.float32), residue_index=np.arange(n),
                           b_factors=np.zeros((n, 37), np.float32))
    met = amber_minimize.get_violation_metrics(full)
    assert met["num_residue_violations"] == len(met["residue_violations"]) and "structural_violations" in met


def test_misc_utils_and_import_paths():
    from fastfold_b200.parallel import comm_async
    from fastfold_b200.utils import checkpointing, tensor_utils, test_utils, validation_utils
    x = torch.randn(1, 4, 3, 2, requires_grad=True)
    y = comm_async.GatherAsyncOpp.apply(x)
    y.sum().backward()
    assert y.shape == x.shape and x.grad.shape == x.shape
    lin = torch.nn.Linear(4, 4)
    inp = torch.randn(3, 4, requires_grad=True)
    out = checkpointing.get_checkpoint_fn()(lambda a: torch.relu(lin(a)), inp)
    out.sum().backward()
    assert inp.grad is not None and out.shape == (3, 4)
    assert tensor_utils.dict_map(lambda t: t + 1, {"a": torch.zeros(1), "b": {"c": torch.ones(1)}}, torch.Tensor)["b"]["c"].item() == 2.0
    test_utils.set_seed(7)
    a = torch.rand(1)
    test_utils.set_seed(7)
    assert torch.equal(a, torch.rand(1))
    pts = torch.randn(8, 3)
    assert float(validation_utils.drmsd_np(pts.numpy(), pts.numpy())) == pytest.approx(0.0, abs=1e-5)
    import fastfold
    for name in sorted(fastfold._ALIASES):
        importlib.import_module(name)
    # every module of the reference package except its Habana port (paths listed from its source tree)
    for name in ("fastfold.model.fastnn.kernel.triton.softmax", "fastfold.model.fastnn.kernel.cuda_native.layer_norm",
                 "fastfold.model.fastnn.kernel.jit.options", "fastfold.workflow.factory.hhfilter", "fastfold.data.tools.kalign",
                 "fastfold.utils.geometry.quat_rigid", "fastfold.model.nn.outer_product_mean", "fastfold.relax.cleanup"):
        importlib.import_module(name)
    from fastfold.data.input_pipeline import process_tensors_from_config          # noqa: F401
    from fastfold.utils.geometry.rigid_matrix_vector import Rigid3Array          # noqa: F401
    from fastfold.model.nn.triangular_multiplicative_update import TriangleMultiplicationIncoming          # noqa: F401
    from fastfold.utils.import_weights import Param, ParamType, get_translation_dict          # noqa: F401


def test_template_features_flow_into_the_model():
    """Raw example with two templates -> feature pipeline -> full model (OpenFold layout and injected fast modules)."""
    from fastfold_b200.models.hub import AlphaFold
    from fastfold_b200.utils.inject_fastnn import inject_fastnn
    cfg = model_config("model_1")
    cfg.model.evoformer_stack.no_blocks = 1
    cfg.model.extra_msa.extra_msa_stack.no_blocks = 1
    cfg.model.template.template_pair_stack.no_blocks = 1
    cfg.model.structure_module.no_blocks = 1
    cfg.data.common.max_recycling_iters = 0
    cfg.data.predict.max_msa_clusters = 8
    cfg.data.predict.max_extra_msa = 16
    feats = dp.FeaturePipeline(cfg.data).process_features(_raw_example(2), mode="predict", seed=1)
    assert feats["template_mask"][:, 0].tolist() == [1.0, 1.0, 0.0, 0.0]
    torch.manual_seed(0)
    model = AlphaFold(cfg).eval()
    with torch.no_grad():
        for p in model.parameters():          # the zero-initialised output layers would hide the template path
            if p.abs().sum() == 0:
                p.normal_(0, 0.02)
        out = model(feats)
        no_templ = dict(feats)
        no_templ["template_mask"] = torch.zeros_like(feats["template_mask"])
        out_masked = model(no_templ)
        fast = inject_fastnn(model)
        out_fast = fast(feats)
    assert torch.isfinite(out["final_atom_positions"]).all()
    assert (out["pair"] - out_masked["pair"]).abs().max() > 1e-4          # the templates do change the pair representation
    assert (out_fast["pair"] - out["pair"]).abs().max() < 5e-4


def test_kernel_level_names_keep_the_reference_contracts():
    """fastfold/model/fastnn/kernel/{attention_core,softmax,layer_norm}.py and its back-end sub-modules."""
    import math
    from fastfold.model.fastnn.kernel import fused_attention_core
    from fastfold.model.fastnn.kernel.attention_core import FusedAttenionCoreFunc
    from fastfold.model.fastnn.kernel.triton.attention_core import attention_core_triton_kernel_wrapper
    from fastfold.model.fastnn.kernel.cuda_native.softmax import softmax_cuda_kernel_wrapper, softmax_grad_cuda_kernel_wrapper
    from fastfold.model.fastnn.kernel.triton.softmax import softmax_triton_kernel_wrapper, softmax_grad_triton_kernel_wrapper
    from fastfold.model.fastnn.kernel.softmax import FusedSoftmaxFunc  # noqa: F401
    from fastfold.model.fastnn.kernel.cuda_native.layer_norm import FusedLayerNormAffineFunction
    from fastfold.model.fastnn.kernel.triton.layer_norm import LayerNormTritonFunc
    torch.manual_seed(0)
    b1, b2, h, n, d = 1, 3, 2, 5, 4
    q, k, v = (torch.randn(b1, b2, h, n, d) for _ in range(3))
    mask = (torch.rand(b1, b2, n) > 0.3).float()
    mask[..., 0] = 1
    bias = torch.randn(b1, 1, h, n, n)
    # the reference's composite: q scaled inside, heads merged in the result
    logits = torch.matmul(q / math.sqrt(d), k.transpose(-1, -2)) + bias + (1e20 * (mask - 1))[..., :, None, None, :]
    want = torch.matmul(torch.softmax(logits, -1), v).permute(0, 1, 3, 2, 4).reshape(b1, b2, n, h * d)
    for fn in (fused_attention_core, FusedAttenionCoreFunc.apply, attention_core_triton_kernel_wrapper):
        got = fn(q, k, v, mask, bias)
        assert got.shape == want.shape and torch.allclose(got, want, atol=1e-5)
    # softmax: forward wrappers agree with the oracle, backward wrappers with autograd
    x = torch.randn(b1, b2, h, n, n, requires_grad=True)
    y_ref = torch.softmax(x + bias + (1e9 * (mask - 1))[..., :, None, None, :], -1)
    dy = torch.randn_like(y_ref)
    (dx_ref,) = torch.autograd.grad(y_ref, x, dy)
    rows, cols = x.numel() // n, n
    for fwd in (softmax_cuda_kernel_wrapper, softmax_triton_kernel_wrapper):
        assert torch.allclose(fwd(x.detach(), mask, bias, rows, cols), y_ref, atol=1e-6)
    assert torch.allclose(softmax_grad_cuda_kernel_wrapper(dy, y_ref.detach(), mask, rows, cols), dx_ref, atol=1e-6)
    assert torch.allclose(softmax_grad_triton_kernel_wrapper(dy, y_ref.detach(), rows, cols), dx_ref, atol=1e-6)
    with pytest.raises(ValueError):
        softmax_cuda_kernel_wrapper(x.detach(), mask, bias, rows, cols + 1)
    # LayerNorm: the two argument orders
    a = torch.randn(7, 16)
    w, b = torch.randn(16), torch.randn(16)
    want = torch.nn.functional.layer_norm(a, (16,), w, b, 1e-5)
    assert torch.allclose(FusedLayerNormAffineFunction.apply(a, w, b, (16,), 1e-5), want, atol=1e-6)
    assert torch.allclose(LayerNormTritonFunc.apply(a, (16,), w, b, 1e-5), want, atol=1e-6)


def test_weight_copy_helpers_and_translation_tables():
    """fastfold/utils/inject_fastnn.py:24-318 (copy_*), fastfold/utils/import_weights.py:81-129 (stacked, assign)."""
    inj = importlib.import_module("fastfold.utils.inject_fastnn")       # the package exports a function of the same name
    iw = importlib.import_module("fastfold.utils.import_weights")
    from fastfold_b200.models.nn.primitives import Attention, Linear
    from fastfold_b200.models.fastnn.ops import SelfAttention
    torch.manual_seed(0)
    ori = Attention(16, 16, 16, 8, 2)
    for p in ori.parameters():
        torch.nn.init.normal_(p, std=0.3)
    fast = SelfAttention(qkv_dim=16, c=8, n_head=2, out_dim=16, gating=True, last_bias_fuse=False)
    inj.copy_attention(fast, ori)
    x = torch.randn(1, 3, 5, 16)
    want = ori(x, x, biases=None)
    got, tail_done = fast(x, torch.ones(1, 3, 5), None)
    assert not tail_done
    assert torch.allclose(got, want, atol=1e-5)
    fused = torch.nn.Linear(16, 48, bias=False)
    inj.copy_qkv_linear(fused, ori.linear_q, ori.linear_k, ori.linear_v)
    assert torch.equal(fused.weight[16:32], ori.linear_k.weight)
    kv = torch.nn.Linear(16, 32, bias=False)
    inj.copy_kv_linear(kv, ori.linear_k, ori.linear_v)
    assert torch.equal(kv.weight[16:], ori.linear_v.weight)
    left, right, both = Linear(8, 4), Linear(8, 4), Linear(8, 8)
    inj.copy_left_right(both, left, right)
    assert torch.equal(both.weight[4:], right.weight) and torch.equal(both.bias[:4], left.bias)
    twin = Attention(16, 16, 16, 8, 2)
    inj.copy_native_att(twin, ori)
    assert torch.equal(twin.linear_o.weight, ori.linear_o.weight) and torch.equal(twin.linear_g.bias, ori.linear_g.bias)
    # stacked / assign: two blocks' trees become one stacked table; archive arrays land transposed
    l1, l2 = torch.nn.Linear(3, 4), torch.nn.Linear(3, 4)
    tree = [{"a": {"w": iw.Param(l.weight, iw.ParamType.LinearWeight), "b": iw.Param(l.bias)}} for l in (l1, l2)]
    st = iw.stacked(tree)
    assert st["a"]["w"].stacked and len(st["a"]["w"].param) == 2
    W, B = np.random.randn(2, 3, 4).astype(np.float32), np.random.randn(2, 4).astype(np.float32)
    iw.assign({"a/w": st["a"]["w"], "a/b": st["a"]["b"]}, {"a/w": W, "a/b": B})
    assert np.allclose(l2.weight.detach().numpy(), W[1].T) and np.allclose(l1.bias.detach().numpy(), B[0])
    with pytest.raises(ValueError):
        iw.assign({"a/b": st["a"]["b"]}, {"a/b": B[:1]})


def test_remaining_small_names():
    from fastfold.data import data_pipeline, data_transforms, data_transforms_multimer
    from fastfold.model.hub import loss
    from fastfold.model.fastnn import ops as fops, triangle
    from fastfold.relax import amber_minimize
    from fastfold.common import residue_constants
    assert data_pipeline.add_assembly_features is msa_pairing.add_assembly_features and callable(data_pipeline.pad_msa)
    chi = data_transforms.get_chi_atom_indices()
    assert len(chi) == 21 and len(chi[0]) == 4 and chi[rc.restype_order["G"]] == [[0, 0, 0, 0]] * 4
    n = 6
    aatype = torch.tensor([rc.restype_order[c] for c in "GAVLKD"])
    pos, m37 = torch.randn(n, 37, 3), torch.ones(n, 37)
    pb, pbm = data_transforms.pseudo_beta_fn(aatype, pos, m37)
    assert torch.equal(pb[0], pos[0, rc.atom_order["CA"]]) and torch.equal(pb[1], pos[1, rc.atom_order["CB"]]) and pbm.shape == (n,)
    feat = data_transforms_multimer.build_extra_msa_feat({"extra_msa": torch.randint(0, 23, (4, n)), "extra_deletion_matrix": torch.tensor([[0., 3., 0., 0., 1., 0.]] * 4)})
    assert feat.shape == (4, n, 25) and feat[0, 1, 23] == 1 and abs(float(feat[0, 1, 24]) - 0.5) < 1e-6 and feat[0, 0, 24] == 0
    assert loss.compute_plddt(torch.randn(n, 50)).shape == (n,) and callable(loss.compute_tm) and callable(loss.compute_predicted_aligned_error)
    assert fops.InputEmbedder.__name__ == "InputEmbedder" and fops.RecyclingEmbedder.__name__ == "RecyclingEmbedder"
    assert callable(fops.permute_final_dims) and callable(triangle.permute_final_dims)
    prot = {"aatype": aatype.numpy(), "all_atom_positions": pos.numpy(), "all_atom_mask": (m37 * torch.tensor(rc.restype_atom37_mask)[aatype]).numpy()}
    out = amber_minimize.make_atom14_positions(prot)
    assert out["atom14_gt_positions"].shape == (n, 14, 3) and out["residx_atom14_to_atom37"].shape == (n, 14)
    assert out["atom14_gt_exists"][0].sum() == 4 and out["atom14_atom_is_ambiguous"][5].sum() == 2      # GLY has 4 atoms; ASP OD1 / OD2
    import os
    assert os.path.isdir(residue_constants.get_cache_path())


def test_alignment_and_structure_indices(tmp_path):
    """Search outputs of all targets concatenated into one file + an index of byte ranges (fastfold/data/data_pipeline.py:792-843,
    1000-1021; data_modules.py:168-209) give the same features as one directory per target."""
    from fastfold_b200.data.data_modules import OpenFoldSingleDataset
    seqs = {"1abc_A": "MKTAYIAKQRQ", "2xyz_A": "GSHMLEDPVK"}
    aln, flat, data = tmp_path / "aln", tmp_path / "flat", tmp_path / "data"
    flat.mkdir(), data.mkdir()
    index, blob = {}, b""
    for name, seq in seqs.items():
        (aln / name).mkdir(parents=True)
        a3m = ">query\n%s\n>hit1\n%s\n>hit2\n%s-\n" % (seq, seq[:-1] + "A", seq[:-1])
        sto = "# STOCKHOLM 1.0\nquery %s\nother %s\n//\n" % (seq, "A" + seq[1:])
        files = {"bfd_uniclust_hits.a3m": a3m, "mgnify_hits.sto": sto}
        entries = []
        for fname, text in files.items():
            (aln / name / fname).write_text(text)
            entries.append([fname, len(blob), len(text.encode())])
            blob += text.encode()
        index[name] = {"db": "alignments.db", "files": entries}
        prot = protein.Protein(atom_positions=np.random.RandomState(len(seq)).randn(len(seq), 37, 3).astype(np.float32),
                               aatype=np.array([rc.restype_order[c] for c in seq]), atom_mask=np.tile(np.array(rc.restype_atom37_mask)[[rc.restype_order[c] for c in seq]], 1).astype(np.float32),
                               residue_index=np.arange(len(seq)), b_factors=np.full((len(seq), 37), 90.0), chain_index=np.zeros(len(seq), dtype=np.int64))
        (data / (name.split("_")[0] + ".pdb")).write_text(protein.to_pdb(prot))
    (flat / "alignments.db").write_bytes(blob)
    by_dir = OpenFoldSingleDataset(str(data), str(aln), config=None, mode="train", _output_raw=True)
    by_index = OpenFoldSingleDataset(str(data), str(flat), config=None, mode="train", _output_raw=True, _alignment_index=index)
    assert sorted(by_index._chain_ids) == sorted(seqs)
    for name in seqs:
        a, b = by_dir[by_dir.chain_id_to_idx(name)], by_index[by_index.chain_id_to_idx(name)]
        assert a["msa"].shape[0] == 4 and set(a) == set(b)           # query + 2 a3m hits + 1 stockholm row (duplicate query dropped)
        for k in a:
            if a[k].dtype != object:
                assert np.array_equal(a[k], b[k]), k
    # structure index: the PDB text as a byte range of one concatenated file beside the path
    texts = [(data / "1abc.pdb").read_text(), (data / "2xyz.pdb").read_text()]
    (data / "structures.db").write_text("".join(texts))
    sidx = {"db": "structures.db", "files": [["2xyz.pdb", len(texts[0].encode()), len(texts[1].encode())]]}
    p = dp.DataPipeline(None)
    via_index = p.process_pdb(str(data / "missing.pdb"), None, is_distillation=False, _structure_index=sidx)
    direct = p.process_pdb(str(data / "2xyz.pdb"), None, is_distillation=False)
    assert np.array_equal(via_index["all_atom_positions"], direct["all_atom_positions"]) and np.array_equal(via_index["aatype"], direct["aatype"])
