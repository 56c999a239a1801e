"""LayerNorm / softmax / fused elementwise kernels against fp32 PyTorch references.

Shapes and tolerances follow the reference's kernel tests
(tests/test_fastnn/test_layernorm.py:20, tests/test_fastnn/test_softmax.py:14).
"""
import pytest
import torch

from fastfold_b200 import ops
from fastfold_b200.ops.layer_norm import layer_norm_transposed
from fastfold_b200.ops.softmax import softmax_ref

pytestmark = pytest.mark.gpu
DEV = "cuda"
LN_TOL = {torch.float32: 1e-4, torch.float16: 1e-1, torch.bfloat16: 1e-1}
# output rounding alone is half an ulp at values in [0.5, 1): 2.4e-4 (fp16), 2e-3 (bf16)
SM_TOL = {torch.float32: 1e-6, torch.float16: 5e-4, torch.bfloat16: 4e-3}


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("cols", [64, 128, 129, 256, 384, 1024, 2048])
def test_layernorm(dtype, cols, device_status):
    torch.manual_seed(0)
    x = torch.randn(3, 64, cols, device=DEV, dtype=dtype, requires_grad=True)
    ln = ops.LayerNorm(cols).to(DEV, dtype)
    with torch.no_grad():
        ln.weight.copy_(torch.randn(cols) * 0.5 + 1)
        ln.bias.copy_(torch.randn(cols) * 0.1)
    y = ln(x)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    wr = ln.weight.detach().float().requires_grad_(True)
    br = ln.bias.detach().float().requires_grad_(True)
    yr = torch.nn.functional.layer_norm(xr, (cols,), wr, br, ln.eps)
    yr.backward(g.float())
    tol = LN_TOL[dtype]
    assert (y.float() - yr).abs().max() < tol
    assert (x.grad.float() - xr.grad).abs().max() < tol
    rel = lambda a, b: ((a.float() - b).abs().max() / (b.abs().max() + 1e-6)).item()
    assert rel(ln.weight.grad, wr.grad) < (1e-4 if dtype == torch.float32 else 2e-2)
    assert rel(ln.bias.grad, br.grad) < (1e-4 if dtype == torch.float32 else 2e-2)


def test_layernorm_transposed(device_status):
    x = torch.randn(128, 1000, device=DEV, dtype=torch.bfloat16)
    w = torch.randn(128, device=DEV, dtype=torch.bfloat16)
    b = torch.randn(128, device=DEV, dtype=torch.bfloat16)
    y = layer_norm_transposed(x, w, b, 1e-5)
    yr = torch.nn.functional.layer_norm(x.float().t(), (128,), w.float(), b.float(), 1e-5)
    assert (y.float() - yr).abs().max() < 1e-1


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16])
@pytest.mark.parametrize("seq", [31, 32, 128, 129, 256, 259, 512, 700, 1024, 1500])
def test_softmax(dtype, seq, device_status):
    torch.manual_seed(1)
    x = torch.randn(2, 3, 4, seq, seq, device=DEV, dtype=dtype, requires_grad=True)
    mask = (torch.rand(2, 3, seq, device=DEV) > 0.2).to(dtype)
    mask[..., 0] = 1
    bias = torch.randn(2, 1, 4, seq, seq, device=DEV, dtype=dtype, requires_grad=True)
    y = ops.fused_softmax(x, mask, bias)
    g = torch.randn_like(y)
    y.backward(g)
    xr = x.detach().float().requires_grad_(True)
    br = bias.detach().float().requires_grad_(True)
    yr = softmax_ref(xr, mask.float(), br)
    yr.backward(g.float())
    tol = SM_TOL[dtype]
    assert (y.float() - yr).abs().max() < tol
    assert (x.grad.float() - xr.grad).abs().max() < tol * 10
    assert (bias.grad.float() - br.grad).abs().max() < tol * 30


def test_softmax_global_attention_shape(device_status):
    # 4-D logits [b1, b2, H, S]: the mask row must follow b2, not row // (H * S)
    x = torch.randn(1, 7, 8, 300, device=DEV, dtype=torch.bfloat16)
    mask = (torch.rand(1, 7, 300, device=DEV) > 0.3).to(torch.bfloat16)
    mask[..., 0] = 1
    y = ops.fused_softmax(x, mask)
    assert (y.float() - softmax_ref(x.float(), mask.float())).abs().max() < 1e-3


def _check_grads(fn_fast, fn_ref, tensors, tol=3e-2):
    fast = [t.detach().clone().requires_grad_(t.is_floating_point() and t.requires_grad) for t in tensors]
    ref = [t.detach().float().requires_grad_(t.requires_grad) for t in tensors]
    yf, yr = fn_fast(*fast), fn_ref(*ref)
    g = torch.randn_like(yr)
    yf.backward(g.to(yf.dtype))
    yr.backward(g)
    assert (yf.float() - yr).abs().max() < tol * (1 + yr.abs().max())
    for a, b in zip(fast, ref):
        if b.grad is not None:
            assert a.grad is not None
            assert (a.grad.float() - b.grad).abs().max() < tol * (1 + b.grad.abs().max()), (a.shape,)


def test_fused_elementwise(device_status):
    torch.manual_seed(2)
    bf = torch.bfloat16
    R = lambda *s: torch.randn(*s, device=DEV, dtype=bf).requires_grad_(True)
    y, bias, z = R(1, 16, 24, 256), R(256), R(1, 16, 24, 256)
    _check_grads(ops.bias_sigmod_ele, lambda y, b, z: torch.sigmoid(y + b) * z, [y, bias, z])
    mask_row = ((torch.rand(1, 1, 24, 256, device=DEV) > 0.15).to(bf) / 0.85)
    mask_col = ((torch.rand(1, 16, 1, 256, device=DEV) > 0.25).to(bf) / 0.75)
    x, res = R(1, 16, 24, 256), R(1, 16, 24, 256)
    for mk in (mask_row, mask_col, None):
        _check_grads(lambda x, b, r: ops.bias_dropout_add(x, b, mk, r, 0.0, True),
                     lambda x, b, r: r + (x + b) * (1 if mk is None else mk.float()), [x, bias, res])
    ab, g = R(1, 16, 24, 256), R(1, 16, 24, 256)
    _check_grads(lambda ab, b, g, r: ops.bias_ele_dropout_residual(ab, b, g, mask_row, r, 0.0, True),
                 lambda ab, b, g, r: r + mask_row.float() * (g * (ab + b)), [ab, bias, g, res])
    p, q = R(1, 16, 24, 256), R(1, 16, 24, 256)
    rm = (torch.rand(1, 16, 24, device=DEV) > 0.2).to(bf)
    _check_grads(lambda p, q: ops.glu_mask(p, q, rm), lambda p, q: rm.float().unsqueeze(-1) * p * torch.sigmoid(q), [p, q])


def test_channel_major_ops_match_references(device_status):
    """linear_t, glu_mask_t and layer_norm_transposed (forward + backward) against fp32 PyTorch."""
    from fastfold_b200 import ops as K
    torch.manual_seed(21)
    R, d, c = 4096 + 64, 128, 128
    x = (torch.randn(R, d, device="cuda") * 0.5).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(4 * c, d, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_(True)
    b = (torch.randn(4 * c, device="cuda") * 0.1).to(torch.bfloat16).requires_grad_(True)
    mask = (torch.rand(R, device="cuda") > 0.2).to(torch.bfloat16)
    gam = (1 + 0.1 * torch.randn(c, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    bet = (0.1 * torch.randn(c, device="cuda")).to(torch.bfloat16).requires_grad_(True)
    lo, hi = K.glu_mask_t(K.linear_t(x, w, b), mask, split=c)
    y = K.layer_norm_transposed(lo * hi, gam, bet, 1e-5)                  # [R, c]
    g = torch.randn_like(y)
    y.backward(g)
    xf, wf, bf, gf, btf = (t.detach().float().requires_grad_(True) for t in (x, w, b, gam, bet))
    pre = (xf @ wf.t() + bf).t()
    glu = pre[:2 * c] * torch.sigmoid(pre[2 * c:]) * mask.float().unsqueeze(0)
    prod = (glu[:c].bfloat16().float() * glu[c:].bfloat16().float())     # the kernel path rounds the gated values to bf16
    ref = torch.nn.functional.layer_norm(prod.t(), (c,), gf, btf, 1e-5)
    ref.backward(g.float())
    assert (y.float() - ref).abs().max() < 0.08
    for got, want, name in ((x, xf, "x"), (w, wf, "w"), (b, bf, "b"), (gam, gf, "gamma"), (bet, btf, "beta")):
        err = (got.grad.float() - want.grad).abs().max().item()
        assert err < 0.05 * max(1.0, want.grad.abs().max().item()), (name, err, want.grad.abs().max().item())


def test_trainer_gradient_sink_matches_autograd_accumulation(device_status):
    """Weight / bias gradients added straight into the trainer's fp32 sink give the same step as autograd accumulation."""
    import copy
    from fastfold_b200.models.fastnn import EvoformerStack
    from fastfold_b200.runtime import FlatAdamTrainer
    torch.manual_seed(0)
    base = EvoformerStack(256, 128, 384, 1, blocks_per_ckpt=1)
    with torch.no_grad():
        for p in base.parameters():
            if p.dim() >= 2 and float(p.abs().sum()) == 0.0:
                p.copy_(torch.randn_like(p) * 0.02)
    S, N = 32, 64
    m = torch.randn(S, N, 256, device="cuda").to(torch.bfloat16)
    z = torch.randn(N, N, 128, device="cuda").to(torch.bfloat16)
    mm, pm = torch.ones(S, N, device="cuda", dtype=torch.bfloat16), torch.ones(N, N, device="cuda", dtype=torch.bfloat16)

    def loss_fn(mod, m, z, mm, pm):
        om, oz, s = mod(m, z, mm, pm, None)
        return om.float().pow(2).mean() + oz.float().pow(2).mean() + s.float().pow(2).mean()

    grads = []
    for sink in (True, False):
        model = copy.deepcopy(base).to("cuda", torch.bfloat16).train()
        tr = FlatAdamTrainer(model, loss_fn, use_graph=False, grad_sink=sink)
        tr.flat_g.zero_()
        if tr.flat_g32 is not None:
            tr.flat_g32.zero_()
        torch.manual_seed(123)                     # same dropout masks in both runs
        loss_fn(model, m, z, mm, pm).backward()
        g = tr.flat_g.float().clone()
        if tr.flat_g32 is not None:
            assert float(tr.flat_g32.abs().sum()) > 0
            g = g + tr.flat_g32
        grads.append(g)
    err = (grads[0] - grads[1]).abs().max().item()
    scale = grads[1].abs().max().item()
    assert err < 2e-2 * max(scale, 1e-3), (err, scale)


@pytest.mark.parametrize("rows,C", [(65536, 128), (4099, 256), (777, 384), (5000, 1024), (300, 8), (1000, 6)])
def test_colsum(rows, C, device_status):
    from fastfold_b200.ops.fused_ops import colsum
    torch.manual_seed(rows)
    x = torch.randn(rows, C, device="cuda").to(torch.bfloat16)
    got = colsum(x)
    want = x.float().sum(0)
    assert (got - want).abs().max() < 1e-2 * max(1.0, want.abs().max().item())
    acc = torch.ones(C, device="cuda")
    colsum(x, out=acc)
    assert (acc - 1 - want).abs().max() < 1e-2 * max(1.0, want.abs().max().item())


@pytest.mark.parametrize("R,S,H,c", [(37, 300, 8, 8), (5, 20, 4, 16), (3, 1000, 8, 32), (150, 1024, 8, 8)])
def test_global_attention_core(R, S, H, c, device_status):
    """One-kernel global column attention (softmax over the sequences with one query per head, value aggregation, gate)
    against the fp32 reference; includes a fully masked column (uniform weights) and S smaller than the 32 sequence lanes."""
    from fastfold_b200.ops.fused_ops import global_attention_supported
    torch.manual_seed(R + S)
    q = (torch.randn(R, H, c, device=DEV) * 0.8).bfloat16()
    kv = torch.randn(R, S, 2 * c, device=DEV).bfloat16()
    mask = (torch.rand(R, S, device=DEV) > 0.2).bfloat16()
    mask[1] = 0
    gate = torch.randn(R, S, H * c, device=DEV).bfloat16()
    gb = torch.randn(H * c, device=DEV).bfloat16()
    with torch.no_grad():
        assert global_attention_supported(q, kv, gate)
        out = ops.global_attention_core(q, kv, mask, gate, gb)
    ref = ops.global_attention_ref(q, kv, mask, gate, gb)
    assert out.shape == gate.shape and out.dtype == torch.bfloat16
    assert (out.float() - ref).abs().max() < 2e-2


@pytest.mark.parametrize("R,S,H,c", [(9, 300, 8, 8), (5, 45, 4, 16), (3, 700, 8, 32)])
def test_global_attention_core_backward(R, S, H, c, device_status):
    """Backward kernel of the global column attention (d q, d kv, d gate, d gate-bias) against autograd through the fp32
    reference; includes a fully masked column."""
    torch.manual_seed(R * S)
    q = (torch.randn(R, H, c, device=DEV) * 0.8).bfloat16().requires_grad_(True)
    kv = torch.randn(R, S, 2 * c, device=DEV).bfloat16().requires_grad_(True)
    mask = (torch.rand(R, S, device=DEV) > 0.2).bfloat16()
    mask[1] = 0
    gate = torch.randn(R, S, H * c, device=DEV).bfloat16().requires_grad_(True)
    gb = torch.randn(H * c, device=DEV).bfloat16().requires_grad_(True)
    dout = torch.randn(R, S, H * c, device=DEV).bfloat16()
    out = ops.global_attention_core(q, kv, mask, gate, gb)
    assert out.grad_fn is not None and "GlobalAttention" in type(out.grad_fn).__name__
    out.backward(dout)
    got = [t.grad.float().clone() for t in (q, kv, gate, gb)]
    ref_in = [t.detach().float().requires_grad_(True) for t in (q, kv, gate, gb)]
    ops.global_attention_ref(ref_in[0], ref_in[1], mask, ref_in[2], ref_in[3]).backward(dout.float())
    for name, a, b in zip(("dq", "dkv", "dgate", "dgate_bias"), got, [t.grad for t in ref_in]):
        tol = 3e-2 * max(1.0, b.abs().max().item())
        assert (a - b).abs().max().item() <= tol, "%s: max err %g (ref max %g)" % (name, (a - b).abs().max().item(), b.abs().max().item())


def test_global_attention_module_matches_composite(device_status):
    """The fastnn GlobalAttention module gives the same result with the fused inference kernel (no grad) as with its
    composite path (grad enabled)."""
    from fastfold_b200.models.fastnn.ops import GlobalAttention
    torch.manual_seed(0)
    ga = GlobalAttention(64, 8, 8, 64).to(DEV, torch.bfloat16)
    with torch.no_grad():
        for p in ga.parameters():
            p.copy_(torch.randn_like(p) * 0.2)
    m = torch.randn(1, 24, 200, 64, device=DEV).bfloat16()
    mask = (torch.rand(1, 24, 200, device=DEV) > 0.1).bfloat16()
    with torch.no_grad():
        fused = ga(m, mask)
    trained = ga(m, mask)                       # grad enabled: forward kernel under the autograd wrapper
    comp = ga.float().cpu()(m.float().cpu(), mask.float().cpu()).detach()
    assert (fused.float().cpu() - comp).abs().max() < 3e-2 * max(1.0, comp.abs().max().item())
    assert (trained.detach().float().cpu() - comp).abs().max() < 3e-2 * max(1.0, comp.abs().max().item())


@pytest.mark.parametrize("N", [64, 200])
def test_recycle_pair_embed(N, device_status):
    """Gather-add form of the recycling embedder's pair update against the one-hot composite.  A distance that sits
    within rounding of a bin edge may fall into the neighbouring bin, so a handful of rows may differ by one weight column."""
    from fastfold_b200.ops import embed
    torch.manual_seed(N)
    z = torch.randn(N, N, 128, device=DEV).bfloat16()
    x = torch.randn(N, 3, device=DEV) * 8.0
    bins = torch.linspace(3.25, 20.75, 15, device=DEV) ** 2
    w = (torch.randn(128, 15, device=DEV) * 0.5).bfloat16()
    b = (torch.randn(128, device=DEV) * 0.1).bfloat16()
    g = (torch.randn(128, device=DEV) * 0.3 + 1).bfloat16()
    be = (torch.randn(128, device=DEV) * 0.1).bfloat16()
    with torch.no_grad():
        assert embed.recycle_pair_embed_supported(z, x)
        out = embed.recycle_pair_embed(z, x, bins, 1e8, w, b, g, be, 1e-5)
        ref = embed.recycle_pair_embed_ref(z.float(), x, bins, 1e8, w.float(), b.float(), g.float(), be.float(), 1e-5)
    err = (out.float() - ref).abs().amax(dim=-1)
    assert (err > 6e-2).float().mean().item() < 1e-3, err.max().item()
    assert torch.isfinite(out.float()).all()


def test_recycling_embedder_module_uses_fused_pair_update(device_status):
    from fastfold_b200.models.fastnn.embedders import RecyclingEmbedder
    torch.manual_seed(1)
    emb = RecyclingEmbedder(c_m=256, c_z=128, min_bin=3.25, max_bin=20.75, no_bins=15, inf=1e8).to(DEV, torch.bfloat16)
    with torch.no_grad():
        for p in emb.parameters():
            p.copy_(torch.randn_like(p) * 0.3)
    m = torch.randn(96, 256, device=DEV).bfloat16()
    z = torch.randn(96, 96, 128, device=DEV).bfloat16()
    x = torch.randn(96, 3, device=DEV) * 8.0
    with torch.no_grad():
        m1, z1 = emb(m, z, x)
    m2, z2 = emb(m, z, x)                    # grad enabled: composite path
    assert torch.equal(m1, m2.detach())
    err = (z1.float() - z2.detach().float()).abs().amax(dim=-1)
    assert (err > 8e-2).float().mean().item() < 1e-3, err.max().item()
