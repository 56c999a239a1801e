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
