"""Full-model training step on CPU (tiny config): every loss term is finite, gradients reach the trunk, and the
single Evoformer block reproduces the OpenFold-layout block in forward and backward (fp32)."""
import copy

import torch

from fastfold_b200.config import model_config, set_shared
from fastfold_b200.models.hub import AlphaFold, AlphaFoldLoss, AlphaFoldLRScheduler
from fastfold_b200.utils.inject_fastnn import inject_fastnn
from fastfold_b200.utils.synthetic import random_features
from fastfold_b200.utils.tensor_utils import tensor_tree_map


def _tiny(name="model_3_ptm"):
    c = model_config(name, train=True)
    c.model.evoformer_stack.no_blocks = 2
    c.model.extra_msa.extra_msa_stack.no_blocks = 1
    c.model.structure_module.no_blocks = 2
    c.loss.violation.weight = 1.0
    c.loss.experimentally_resolved.weight = 0.01
    return c


def test_train_step_all_loss_terms_finite():
    torch.manual_seed(0)
    c = _tiny()
    model = inject_fastnn(AlphaFold(c)).train()
    batch = random_features(10, 5, 6, n_recycle=1, seed=2, supervised=True)
    out = model(batch)
    last = tensor_tree_map(lambda t: t[..., -1], batch)
    loss, parts = AlphaFoldLoss(c.loss)(out, last, _return_breakdown=True)
    assert torch.isfinite(loss)
    for k in ("distogram", "fape", "lddt", "masked_msa", "supervised_chi", "violation", "experimentally_resolved", "tm"):
        assert k in parts and torch.isfinite(parts[k]), k
    loss.backward()
    g = [p.grad for n, p in model.named_parameters() if n.startswith("evoformer.") and p.grad is not None]
    assert len(g) > 50 and all(torch.isfinite(x).all() for x in g)


def test_lr_schedule():
    class Opt:
        lr = 0.0
    s = AlphaFoldLRScheduler(Opt(), warmup_no_steps=10, start_decay_after_n_steps=20, decay_every_n_steps=5)
    lrs = [s.step() for _ in range(40)]
    assert abs(lrs[9] - 1e-3) < 1e-9 and abs(lrs[15] - 1e-3) < 1e-12 and lrs[-1] < 1e-3 * 0.95 ** 3
    assert s.state_dict()["last_epoch"] == 40


def test_single_block_forward_backward_matches_reference_layout():
    """Single Evoformer block, fp32, m [32, 64, 256] / z [64, 64, 128] scaled down to keep CPU time low."""
    from fastfold_b200.models.nn.evoformer import EvoformerStack as RefStack
    from fastfold_b200.models.fastnn import EvoformerStack as FastStack
    from fastfold_b200.utils.inject_fastnn import copy_evoformer_block, _copy_linear
    torch.manual_seed(0)
    ref = RefStack(256, 128, 32, 32, 128, 32, 384, 8, 4, 1, 4, 0.15, 0.25, None, 1e9, 1e-8).eval()
    with torch.no_grad():
        for p in ref.parameters():
            if p.dim() >= 2 and float(p.abs().sum()) == 0.0:
                p.normal_(std=0.05)
    fast = FastStack(256, 128, 384, 1, None).eval()
    copy_evoformer_block(fast.blocks[0], ref.blocks[0])
    _copy_linear(fast.linear, ref.linear)
    S, N = 8, 16
    m = torch.randn(S, N, 256, requires_grad=True)
    z = torch.randn(N, N, 128, requires_grad=True)
    mm, pm = torch.ones(S, N), torch.ones(N, N)
    outs = []
    for mod in (ref, fast):
        m_, z_ = m.detach().clone().requires_grad_(True), z.detach().clone().requires_grad_(True)
        om, oz, s = mod(m_, z_, mm, pm, None)
        (om.pow(2).mean() + oz.pow(2).mean() + s.pow(2).mean()).backward()
        outs.append((om.detach(), oz.detach(), m_.grad, z_.grad))
    for a, b in zip(*outs):
        assert (a - b).abs().max() < 1e-4 * max(1.0, b.abs().max().item())


def test_block_permuted_gemm_reference_layouts():
    """CPU oracle of the block-permuted GEMM output: both layouts used by the outer-product-mean module."""
    import torch
    from fastfold_b200.ops import gemm
    torch.manual_seed(0)
    S, ni, N = 16, 2, 64
    l2, r2 = torch.randn(S, ni * 32), torch.randn(S, N * 32)
    o4 = gemm(l2, r2, a_mn=True, b_mn=True, block_out=((ni, N, 32, 32), 1, N * 1024, 0, 1024))
    ref = (l2.t() @ r2).reshape(ni, 32, N, 32).permute(0, 2, 1, 3)
    assert torch.allclose(o4, ref, atol=1e-4)
    dy, w = torch.randn(ni * N, 8), torch.randn(8, 1024)
    do = gemm(dy, w, b_mn=True, block_out=((ni * 32, N * 32), N // 32, N * 1024, 1024, 32 * N))
    ref = (dy @ w).reshape(ni, N, 32, 32).permute(0, 2, 1, 3).reshape(ni * 32, N * 32)
    assert torch.allclose(do, ref, atol=1e-4)


def test_multimer_preset_forward():
    """The multimer preset builds (chain-aware input embedder, multimer template embedder, split IPA projections)
    and runs on synthetic two-chain features."""
    import torch
    from fastfold_b200.config import model_config
    from fastfold_b200.models.hub import AlphaFold
    from fastfold_b200.utils.synthetic import random_features
    cfg = model_config("multimer")
    cfg.model.evoformer_stack.no_blocks = 1
    cfg.model.extra_msa.extra_msa_stack.no_blocks = 1
    cfg.model.template.template_pair_stack.no_blocks = 1
    cfg.model.structure_module.no_blocks = 2
    torch.manual_seed(0)
    model = AlphaFold(cfg).eval()
    assert hasattr(model.structure_module.ipa, "linear_k_points") and not hasattr(model.structure_module.ipa, "linear_kv")
    batch = random_features(n_res=20, n_seq=6, n_extra=8, n_templ=2, n_recycle=1, chains=[12, 8])
    with torch.no_grad():
        out = model(batch)
    assert out["final_atom_positions"].shape == (20, 37, 3)
    assert torch.isfinite(out["final_atom_positions"]).all() and torch.isfinite(out["pair"]).all()
    assert out["masked_msa_logits"].shape[-1] == 22


def test_global_attention_reference_matches_module_math():
    """``global_attention_ref`` (the oracle of the fused kernel) is the module's composite path."""
    import torch
    from fastfold_b200 import ops
    from fastfold_b200.models.fastnn.ops import GlobalAttention
    torch.manual_seed(0)
    ga = GlobalAttention(16, 4, 2, 16)
    with torch.no_grad():
        for p in ga.parameters():
            p.copy_(torch.randn_like(p) * 0.3)
    m = torch.randn(1, 5, 7, 16)
    mask = (torch.rand(1, 5, 7) > 0.3).float()
    mask[0, 2] = 0
    want = ga(m, mask)
    mk = mask
    q = torch.sum(m * mk.unsqueeze(-1), dim=-2) / (torch.sum(mk, dim=-1)[..., None] + ga.eps)
    q = ga.to_q(q * ga.scaling).view(5, 2, 4)
    core = ops.global_attention_ref(q, ga.to_kv(m)[0], mask[0], ga.gating_linear(m)[0], ga.gating_bias)
    got = ga.o_linear(core.unsqueeze(0))
    assert torch.allclose(got, want, atol=1e-5)


def test_recycle_pair_embed_reference_matches_module():
    """The oracle of the fused recycling pair update equals the recycling embedder's composite forward."""
    import torch
    from fastfold_b200.models.fastnn.embedders import RecyclingEmbedder
    from fastfold_b200.ops import embed
    torch.manual_seed(0)
    emb = RecyclingEmbedder(c_m=32, c_z=16, min_bin=3.25, max_bin=20.75, no_bins=15, inf=1e8)
    m, z, x = torch.randn(10, 32), torch.randn(10, 10, 16), torch.randn(10, 3) * 8
    _, want = emb(m, z, x)
    bins = torch.linspace(3.25, 20.75, 15) ** 2
    got = embed.recycle_pair_embed(z, x, bins, 1e8, emb.linear.weight, emb.linear.bias, emb.layer_norm_z.weight, emb.layer_norm_z.bias, emb.layer_norm_z.eps)
    assert torch.allclose(got, want, atol=1e-5)


def test_lean_input_embedder_relpos_lookup_matches_one_hot():
    """The lean input embedder's relative-position term (a table lookup on integer offsets) equals the one-hot + Linear
    of the OpenFold-layout embedder."""
    import torch
    from fastfold_b200.models.fastnn.embedders import InputEmbedder as Lean
    from fastfold_b200.models.nn.embedders import InputEmbedder as Ref
    torch.manual_seed(0)
    ref = Ref(tf_dim=22, msa_dim=49, c_z=16, c_m=24, relpos_k=32)
    lean = Lean(tf_dim=22, msa_dim=49, c_z=16, c_m=24, relpos_k=32)
    lean.load_state_dict(ref.state_dict())
    n = 300
    tf, msa = torch.randn(n, 22), torch.randn(5, n, 49)
    ri = torch.arange(n)
    ri[150:] += 200                      # a chain break: offsets far outside the clipping range
    m1, z1 = ref(tf, ri, msa)
    m2, z2 = lean(tf, ri, msa)
    assert torch.allclose(m1, m2, atol=1e-6) and torch.allclose(z1, z2, atol=1e-5)


def test_padded_head_weights_reproduce_the_layer():
    """Zero-padding every attention head to the fused kernel's 32 channels leaves projections and output unchanged."""
    import torch
    from fastfold_b200.models.fastnn.ops import SelfAttention
    torch.manual_seed(0)
    att = SelfAttention(16, 8, 2, 16, gating=True).eval()      # the cache below applies to eval mode only
    with torch.no_grad():
        for p in att.parameters():
            p.copy_(torch.randn_like(p))
    wq, wg, bg, wo = att._padded_heads()
    x = torch.randn(5, 16)
    qkv = (x @ att.to_qkv.weight.t()).reshape(5, 3, 2, 8)
    qkv_p = (x @ wq.t()).reshape(5, 3, 2, 32)
    assert torch.equal(qkv_p[..., :8], qkv) and float(qkv_p[..., 8:].abs().max()) == 0.0
    o = torch.randn(5, 2, 8)
    o_p = torch.zeros(5, 2, 32)
    o_p[..., :8] = o
    assert torch.allclose(o_p.reshape(5, -1) @ wo.t(), o.reshape(5, -1) @ att.o_linear.weight.t(), atol=1e-5)
    assert torch.equal(bg.reshape(2, 32)[:, :8].reshape(-1), att.gating_bias) and float(bg.reshape(2, 32)[:, 8:].abs().max()) == 0.0
    assert torch.equal(wg.reshape(2, 32, 16)[:, :8].reshape(16, 16), att.gating_linear.weight)
    assert att._padded_heads()[0] is wq                      # cached until a weight changes
    with torch.no_grad():
        att.to_qkv.weight.mul_(2.0)
    assert att._padded_heads()[0] is not wq
    # in training mode nothing is cached: an optimiser that writes the parameters through raw pointers bumps no version
    att.train()
    first = att._padded_heads()[0]
    att.to_qkv.weight.data.view(-1)[0] = 123.0
    again = att._padded_heads()[0]
    assert again is not first and float(again.reshape(-1)[0]) == 123.0


def test_full_model_train_step_matches_reference_layout(monkeypatch):
    """One optimiser step of the whole model with the fast trunk against the OpenFold-layout model: loss, every gradient
    (fused / re-laid-out parameters compared after mapping back to the OpenFold names) and the updated parameters.  The
    reference's tests/test_train.py:60-106 compares identically named parameters only; dropout is switched off here because
    the two layouts draw their masks differently."""
    from functools import partial
    from fastfold_b200.models.fastnn import evoformer as fast_evoformer
    from fastfold_b200.utils.inject_fastnn import extract_fastnn
    # the fast trunk's dropout rates are constants (0.15 / 0.25, as in the reference's fast modules): draw keep-all masks
    monkeypatch.setattr(fast_evoformer, "draw_block_dropout", partial(fast_evoformer.draw_block_dropout, p_msa=0.0, p_pair=0.0))
    c = _tiny("model_1_ptm")
    c.model.template.template_pair_stack.dropout_rate = 0.0
    for stack in (c.model.evoformer_stack, c.model.extra_msa.extra_msa_stack):
        stack.msa_dropout = 0.0
        stack.pair_dropout = 0.0
    c.model.structure_module.dropout_rate = 0.0
    torch.manual_seed(0)
    ref = AlphaFold(c)
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for p in ref.parameters():
            if float(p.abs().sum()) == 0.0:
                p.copy_(torch.randn(p.shape, generator=g) * (0.02 if p.dim() < 2 else 0.5 / p.shape[-1] ** 0.5))
    fast = inject_fastnn(copy.deepcopy(ref))
    batch = random_features(10, 5, 6, n_templ=2, n_recycle=1, seed=2, supervised=True)
    last = tensor_tree_map(lambda t: t[..., -1], batch)
    crit = AlphaFoldLoss(c.loss)
    state = {}
    for name, model in (("ref", ref), ("fast", fast)):
        model.train()
        opt = torch.optim.Adam(model.parameters(), lr=1e-3, eps=1e-6)
        loss = crit(model(batch), last)
        loss.backward()
        if name == "fast":
            # gradients and parameters of the swapped stacks under their OpenFold names
            live = dict(model.named_parameters())
            for p in live.values():
                p.data, p.grad = p.grad, p.data
            grads = {k: v.clone() for k, v in extract_fastnn(model).items()}
            for p in live.values():
                p.data, p.grad = p.grad, p.data
        else:
            grads = {k: p.grad.clone() for k, p in model.named_parameters() if p.grad is not None}
        opt.step()
        params = extract_fastnn(model) if name == "fast" else {k: p.detach() for k, p in model.named_parameters()}
        state[name] = (float(loss), grads, params)
    (l0, g0, p0), (l1, g1, p1) = state["ref"], state["fast"]
    assert abs(l0 - l1) < 1e-4 * abs(l0)
    trunk = [k for k in g0 if k.startswith(("evoformer.", "extra_msa_stack.", "template_embedder.template_pair_stack."))]
    assert len(trunk) > 150 and all(k in g1 for k in trunk), [k for k in trunk if k not in g1][:5]
    scale = max(float(v.abs().max()) for v in g0.values())
    for k, v in g0.items():
        if k in g1:
            assert (g1[k] - v).abs().max() < 5e-3 * max(scale * 1e-2, float(v.abs().max())), k
    moved = 0
    for k, v in p0.items():
        if k in p1:
            assert (p1[k] - v).abs().max() < 1e-3, k
            moved += 1
    assert moved > 200
