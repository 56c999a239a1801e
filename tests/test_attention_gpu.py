"""Fused tcgen05 attention against an fp32 PyTorch reference of the same op."""
import pytest
import torch

from fastfold_b200.ops.attention import attention_core, attention_core_ref
from fastfold_b200.ops import flash

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _qkv(B, n, H, d=32):
    qkv = torch.randn(1, B, n, 3, H, d, device=DEV).to(torch.bfloat16)
    return tuple(qkv[:, :, :, i].permute(0, 1, 3, 2, 4) for i in range(3))


@pytest.mark.parametrize("B,n,H,use_bias,use_mask", [
    (4, 128, 8, True, True), (128, 256, 8, True, True), (37, 256, 4, True, False), (256, 128, 8, False, True),
    (3, 384, 4, True, True), (2, 200, 4, True, True), (5, 1024, 4, True, True), (9, 72, 8, False, False),
    (3, 40, 4, True, True), (300, 256, 4, True, False),
])
def test_forward(B, n, H, use_bias, use_mask, device_status):
    torch.manual_seed(B * 1000 + n)
    q, k, v = _qkv(B, n, H)
    bias = torch.randn(1, 1, H, n, n, device=DEV).to(torch.bfloat16) if use_bias else None
    mask = None
    if use_mask:
        mask = (torch.rand(1, B, n, device=DEV) > 0.2).to(torch.bfloat16)
        mask[..., 0] = 1
        if B > 1:
            mask[0, 1] = 0            # one fully masked row: uniform weights, as in the reference kernels
    assert flash.supported(q, k, v, mask, bias)
    with torch.no_grad():
        out = attention_core(q, k, v, mask, bias)
    ref = attention_core_ref(q.float(), k.float(), v.float(), None if mask is None else mask.float(), None if bias is None else bias.float())
    err = (out.float() - ref).abs().max().item()
    assert err < 2e-2, "max abs err %g" % err


@pytest.mark.parametrize("B,n,H,use_bias,use_mask", [
    (4, 128, 8, True, True), (16, 256, 8, True, True), (7, 256, 4, False, True), (5, 384, 4, True, False), (3, 200, 4, True, True),
    (6, 512, 4, True, True),
])
def test_backward(B, n, H, use_bias, use_mask, device_status):
    torch.manual_seed(B * 77 + n)
    qkv = (torch.randn(1, B, n, 3, H, 32, device=DEV) * 0.7).to(torch.bfloat16).requires_grad_(True)
    bias = torch.randn(1, 1, H, n, n, device=DEV).to(torch.bfloat16).requires_grad_(True) if use_bias else None
    mask = None
    if use_mask:
        mask = (torch.rand(1, B, n, device=DEV) > 0.2).to(torch.bfloat16)
        mask[..., 0] = 1
    q, k, v = (qkv[:, :, :, i].permute(0, 1, 3, 2, 4) for i in range(3))
    assert flash.supported(q, k, v, mask, bias)
    out = attention_core(q, k, v, mask, bias)
    g = torch.randn_like(out)
    out.backward(g)
    qkv_r = qkv.detach().float().requires_grad_(True)
    bias_r = bias.detach().float().requires_grad_(True) if use_bias else None
    qr, kr, vr = (qkv_r[:, :, :, i].permute(0, 1, 3, 2, 4) for i in range(3))
    ref = attention_core_ref(qr, kr, vr, None if mask is None else mask.float(), bias_r)
    ref.backward(g.float())
    assert (out.float() - ref).abs().max() < 2e-2
    gerr = (qkv.grad.float() - qkv_r.grad).abs().max().item()
    gmax = qkv_r.grad.abs().max().item()
    assert gerr < 3e-2 * max(1.0, gmax), "dqkv err %g (max %g)" % (gerr, gmax)
    if use_bias:
        berr = (bias.grad.float() - bias_r.grad).abs().max().item()
        bmax = bias_r.grad.abs().max().item()
        assert berr < 3e-2 * max(1.0, bmax), "dbias err %g (max %g)" % (berr, bmax)


def test_backward_fully_masked_row_stays_finite(device_status):
    """A batch row whose keys are all masked (a padded MSA row) must not poison the other rows' gradients."""
    torch.manual_seed(5)
    B, n, H = 6, 256, 4
    qkv = (torch.randn(1, B, n, 3, H, 32, device=DEV) * 0.7).to(torch.bfloat16).requires_grad_(True)
    bias = torch.randn(1, 1, H, n, n, device=DEV).to(torch.bfloat16).requires_grad_(True)
    mask = torch.ones(1, B, n, device=DEV, dtype=torch.bfloat16)
    mask[0, 2] = 0
    q, k, v = (qkv[:, :, :, i].permute(0, 1, 3, 2, 4) for i in range(3))
    out = attention_core(q, k, v, mask, bias)
    g = torch.randn_like(out)
    g[:, 2] = 0                      # the model multiplies masked rows away downstream
    out.backward(g)
    assert torch.isfinite(out.float()).all()
    assert torch.isfinite(qkv.grad.float()).all() and torch.isfinite(bias.grad.float()).all()
    qkv_r = qkv.detach().float().requires_grad_(True)
    bias_r = bias.detach().float().requires_grad_(True)
    qr, kr, vr = (qkv_r[:, :, :, i].permute(0, 1, 3, 2, 4) for i in range(3))
    ref = attention_core_ref(qr, kr, vr, mask.float(), bias_r)
    ref.backward(g.float())
    keep = [0, 1, 3, 4, 5]
    gerr = (qkv.grad.float()[:, keep] - qkv_r.grad[:, keep]).abs().max().item()
    assert gerr < 3e-2 * max(1.0, qkv_r.grad.abs().max().item())
    berr = (bias.grad.float() - bias_r.grad).abs().max().item()
    assert berr < 3e-2 * max(1.0, bias_r.grad.abs().max().item())
