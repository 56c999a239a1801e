"""tcgen05 GEMM against an fp32 PyTorch reference: every operand layout, tails, batching, split-K and each epilogue."""
import pytest
import torch

from fastfold_b200.ops import gemm, gemm_ref, linear, bmm_nt

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _rand(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def _close(out, ref, K):
    # bf16 inputs, fp32 accumulation, bf16 output rounding: error grows like sqrt(K) * eps_bf16
    tol = 2e-2 * max(1.0, (K / 64) ** 0.5)
    ref_max = ref.float().abs().max().item()
    tol = tol + ref_max * 2.0 ** -7          # bf16 output rounding (half an ulp, relative) with slack
    err = (out.float() - ref.float()).abs().max().item()
    scale = ref.float().abs().max().item() + 1e-6
    assert err <= tol * max(1.0, scale / 8), "max abs err %g (ref max %g, K=%d)" % (err, scale, K)


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 128, 256), (384, 640, 128), (200, 72, 136), (1024, 1024, 256), (130, 64, 64), (4096, 256, 1024)])
def test_kmajor(M, N, K, device_status):
    a, b = _rand(M, K), _rand(N, K)
    out = gemm(a, b)
    _close(out, gemm_ref(a, b, out_dtype=torch.float32), K)


@pytest.mark.parametrize("bn", [64, 128, 256])
def test_tile_widths(bn, device_status):
    a, b = _rand(512, 192), _rand(512, 192)
    _close(gemm(a, b, bn=bn), gemm_ref(a, b, out_dtype=torch.float32), 192)


@pytest.mark.parametrize("M,N,K", [(256, 128, 256), (384, 256, 128), (200, 192, 72)])
def test_b_mn_major(M, N, K, device_status):
    a, b = _rand(M, K), _rand(K, N)          # B stored [K, N]: data-gradient layout
    out = gemm(a, b, b_mn=True)
    _close(out, gemm_ref(a, b, b_mn=True, out_dtype=torch.float32), K)


@pytest.mark.parametrize("M,N,K", [(256, 128, 512), (128, 256, 4096), (192, 320, 200)])
def test_both_mn_major_splitk(M, N, K, device_status):
    a, b = _rand(K, M), _rand(K, N)          # weight-gradient layout: contraction over tokens
    ref = gemm_ref(a, b, a_mn=True, b_mn=True, out_dtype=torch.float32)
    _close(gemm(a, b, a_mn=True, b_mn=True), ref, K)
    acc = torch.zeros(M, N, device=DEV)
    gemm(a, b, a_mn=True, b_mn=True, out=acc, accumulate=True, splits=4)
    _close(acc, ref, K)


def test_a_mn_only(device_status):
    a, b = _rand(256, 192), _rand(128, 256)  # A stored [K=256, M=192]
    _close(gemm(a, b, a_mn=True), gemm_ref(a, b, a_mn=True, out_dtype=torch.float32), 256)


def test_batched_and_broadcast(device_status):
    a, b = _rand(8, 128, 64), _rand(8, 192, 64)
    _close(gemm(a, b), gemm_ref(a, b, out_dtype=torch.float32), 64)
    w = _rand(128, 64)
    _close(gemm(a, w), gemm_ref(a, w, out_dtype=torch.float32), 64)
    at, bt = _rand(8, 64, 128), _rand(8, 64, 192)
    _close(gemm(at, bt, a_mn=True, b_mn=True), gemm_ref(at, bt, a_mn=True, b_mn=True, out_dtype=torch.float32), 64)


def test_epilogues(device_status):
    M, N, K = 512, 256, 128
    a, b = _rand(M, K), _rand(N, K, scale=0.2)
    bias = _rand(N)
    mul = _rand(M, N)
    resid = _rand(M, N)
    rowscale = torch.rand(M, device=DEV)
    for act in (None, "relu", "sigmoid"):
        _close(gemm(a, b, bias=bias, act=act), gemm_ref(a, b, bias=bias, act=act, out_dtype=torch.float32), K)
    _close(gemm(a, b, bias=bias, act="sigmoid", mul=mul), gemm_ref(a, b, bias=bias, act="sigmoid", mul=mul, out_dtype=torch.float32), K)
    # dropout mask shared along "rows of 64" (mask row = m % 64) and along columns (mask row = m // 64)
    dm = (torch.rand(64, N, device=DEV) > 0.25).to(torch.bfloat16) / 0.75
    _close(gemm(a, b, bias=bias, dmask=(dm, 1, 64), resid=resid), gemm_ref(a, b, bias=bias, dmask=(dm, 1, 64), resid=resid, out_dtype=torch.float32), K)
    dm2 = (torch.rand(8, N, device=DEV) > 0.25).to(torch.bfloat16) / 0.75
    _close(gemm(a, b, mul=mul, dmask=(dm2, 64, 8), resid=resid), gemm_ref(a, b, mul=mul, dmask=(dm2, 64, 8), resid=resid, out_dtype=torch.float32), K)
    _close(gemm(a, b, bias=bias, rowscale=rowscale, resid=resid), gemm_ref(a, b, bias=bias, rowscale=rowscale, resid=resid, out_dtype=torch.float32), K)
    # gated linear unit on interleaved (value, gate) columns, transposed (channel-major) store
    out = gemm(a, b, bias=bias, glu=True, rowscale=rowscale, trans_out=True)
    assert out.shape == (N // 2, M)
    _close(out, gemm_ref(a, b, bias=bias, glu=True, rowscale=rowscale, trans_out=True, out_dtype=torch.float32), K)
    _close(gemm(a, b, out_dtype=torch.float32), gemm_ref(a, b, out_dtype=torch.float32), K)


def test_epilogues_many_tiles(device_status):
    """Several tiles per CTA and the 256-wide tile (two column chunks per epilogue warp): the mul / residual tiles of a
    warp's first chunk are requested before the accumulator is complete, those of its second chunk after the first."""
    torch.manual_seed(11)
    M, N, K = 19200, 512, 128
    a, b = _rand(M, K), _rand(N, K, scale=0.2)
    bias, mul, resid = _rand(N), _rand(M, N), _rand(M, N)
    rowscale = torch.rand(M, device=DEV)
    _close(gemm(a, b, bias=bias, act="sigmoid", mul=mul), gemm_ref(a, b, bias=bias, act="sigmoid", mul=mul, out_dtype=torch.float32), K)
    _close(gemm(a, b, bias=bias, resid=resid), gemm_ref(a, b, bias=bias, resid=resid, out_dtype=torch.float32), K)
    _close(gemm(a, b, bias=bias, mul=mul, rowscale=rowscale, resid=resid),
           gemm_ref(a, b, bias=bias, mul=mul, rowscale=rowscale, resid=resid, out_dtype=torch.float32), K)
    for bn in (128, 256):
        out = gemm(a, b, bias=bias, glu=True, rowscale=rowscale, trans_out=True, bn=bn)
        assert out.shape == (N // 2, M)
        _close(out, gemm_ref(a, b, bias=bias, glu=True, rowscale=rowscale, trans_out=True, out_dtype=torch.float32), K)
        _close(gemm(a, b, bias=bias, rowscale=rowscale, trans_out=True, bn=bn),
               gemm_ref(a, b, bias=bias, rowscale=rowscale, trans_out=True, out_dtype=torch.float32), K)
    # in place: the residual tile is read and the result written through the same storage
    r2 = resid.clone()
    ref = gemm_ref(a, b, bias=bias, resid=resid, out_dtype=torch.float32)
    _close(gemm(a, b, bias=bias, resid=r2, out=r2), ref, K)


def test_linear_autograd(device_status):
    x = _rand(4, 96, 256).requires_grad_(True)
    w = _rand(512, 256, scale=0.05).requires_grad_(True)
    bias = _rand(512).requires_grad_(True)
    y = linear(x, w, bias, act="relu")
    gy = _rand(4, 96, 512)
    y.backward(gy)
    xf, wf, bf = (t.detach().float().requires_grad_(True) for t in (x, w, bias))
    yf = torch.relu(torch.nn.functional.linear(xf, wf, bf))
    yf.backward(gy.float())
    _close(y, yf, 256)
    _close(x.grad, xf.grad, 512)
    _close(w.grad, wf.grad, 384)
    _close(bias.grad, bf.grad, 384)


def test_bmm_autograd(device_status):
    a = _rand(16, 128, 64).requires_grad_(True)
    b = _rand(16, 192, 64).requires_grad_(True)
    out = bmm_nt(a, b)
    g = _rand(16, 128, 192)
    out.backward(g)
    af, bf = a.detach().float().requires_grad_(True), b.detach().float().requires_grad_(True)
    of = torch.matmul(af, bf.transpose(-1, -2))
    of.backward(g.float())
    _close(out, of, 64)
    _close(a.grad, af.grad, 192)
    _close(b.grad, bf.grad, 128)


def test_block_permuted_output(device_status):
    """Outer-product layouts: [(i d), (j e)] stored as [i, j, d, e], and [(i j), (d e)] stored as [(i d), (j e)]."""
    torch.manual_seed(3)
    S, ni, N = 128, 64, 96
    l2 = torch.randn(S, ni * 32, device="cuda").to(torch.bfloat16)
    r2 = torch.randn(S, N * 32, device="cuda").to(torch.bfloat16)
    o4 = gemm(l2, r2, a_mn=True, b_mn=True, block_out=((ni, N, 32, 32), 1, N * 1024, 0, 1024))
    ref = (l2.float().t() @ r2.float()).reshape(ni, 32, N, 32).permute(0, 2, 1, 3)
    assert (o4.float() - ref).abs().max() < 0.25 and (o4.float() - ref).abs().mean() < 0.03
    dy = (torch.randn(ni * N, 128, device="cuda") * 0.1).to(torch.bfloat16)
    w = torch.randn(128, 1024, device="cuda").to(torch.bfloat16)
    do = gemm(dy, w, b_mn=True, block_out=((ni * 32, N * 32), N // 32, N * 1024, 1024, 32 * N))
    ref = (dy.float() @ w.float()).reshape(ni, N, 32, 32).permute(0, 2, 1, 3).reshape(ni * 32, N * 32)
    err = (do.float() - ref).abs().max().item()
    assert err < 2e-2 * max(1.0, ref.abs().max().item()), err


def test_outer_product_mean_core_gradients(device_status):
    """The hand-written backward of the fused outer-product-mean tail against autograd on the fp32 composite."""
    from fastfold_b200.models.fastnn.ops import _OpmCore
    torch.manual_seed(4)
    S, ni, N, cz = 64, 32, 64, 128
    mk = lambda *shape, s=1.0: (torch.randn(*shape, device="cuda") * s).to(torch.bfloat16).requires_grad_(True)
    l2, r2, w, b, z2 = mk(S, ni * 32, s=0.5), mk(S, N * 32, s=0.5), mk(cz, 1024, s=0.05), mk(cz, s=0.1), mk(ni * N, cz)
    inv = (torch.rand(ni * N, device="cuda") + 0.5).float()
    out = _OpmCore.apply(l2, r2, w, b, inv, z2)
    g = torch.randn_like(out)
    out.backward(g)
    fl = [t.detach().float().requires_grad_(True) for t in (l2, r2, w, b, z2)]
    o = (fl[0].t() @ fl[1]).reshape(ni, 32, N, 32).permute(0, 2, 1, 3).reshape(ni * N, 1024)
    ref = fl[4] + (o @ fl[2].t() + fl[3]) * inv.unsqueeze(-1)
    ref.backward(g.float())
    assert (out.float() - ref).abs().max() < 0.05 * max(1.0, ref.abs().max().item())
    for got, want, name in zip((l2, r2, w, b, z2), fl, "l r w b z".split()):
        err = (got.grad.float() - want.grad).abs().max().item()
        assert err < 3e-2 * max(1.0, want.grad.abs().max().item()), (name, err)


@pytest.mark.parametrize("heads,tokens", [(8, 4096), (4, 2048), (8, 520)])
def test_narrow_channel_major_projection(heads, tokens, device_status):
    """Pair-bias projection stored channel-major (``[H, tokens]``), forward and all three gradients, H < 64."""
    from fastfold_b200.ops import linear_t
    c = 128
    x = _rand(tokens, c).requires_grad_(True)
    w = _rand(heads, c, scale=0.1).requires_grad_(True)
    y = linear_t(x, w)
    assert y.shape == (heads, tokens) and y.is_contiguous()
    ref = (x.detach().float() @ w.detach().float().t()).t()
    _close(y, ref, c)
    dy = _rand(heads, tokens)
    y.backward(dy)
    dx_ref = dy.float().t() @ w.detach().float()
    dw_ref = dy.float() @ x.detach().float()
    _close(x.grad, dx_ref, heads)
    _close(w.grad, dw_ref, tokens)


def test_pair_bias_hqk_matches_permuted_projection(device_status):
    from fastfold_b200.models.fastnn.ops import pair_bias_hqk
    zn = _rand(1, 64, 64, 128)
    w = _rand(8, 128, scale=0.1)
    b = pair_bias_hqk(zn, w)
    ref = torch.einsum("bqkc,hc->bhqk", zn.float(), w.float())
    assert b is not None and b.shape == (1, 8, 64, 64)
    _close(b, ref, 128)
