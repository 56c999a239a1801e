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


@pytest.mark.parametrize("n", [256, 200])
def test_backward_fully_masked_row_is_exact(n, device_status):
    """A batch row whose keys are all masked (a padded MSA row) has uniform attention weights; its gradients must be
    those of the uniform softmax (a backward pass that is off by a constant factor there grows exponentially through a
    deep stack), and the other rows must be unaffected."""
    torch.manual_seed(5)
    B, H = 6, 4
    qkv = (torch.randn(1, B, n, 3, H, 32, device=DEV) * 0.7).to(torch.bfloat16).requires_grad_(True)
    bias = torch.randn(1, 1, H, n, n, device=DEV).to(torch.bfloat16).requires_grad_(True)
    mask = torch.ones(1, B, n, device=DEV, dtype=torch.bfloat16)
    mask[0, 2] = 0
    mask[0, 4] = 0
    q, k, v = (qkv[:, :, :, i].permute(0, 1, 3, 2, 4) for i in range(3))
    out = attention_core(q, k, v, mask, bias)
    g = torch.randn_like(out)
    out.backward(g)
    assert torch.isfinite(out.float()).all()
    assert torch.isfinite(qkv.grad.float()).all() and torch.isfinite(bias.grad.float()).all()
    qkv_r = qkv.detach().float().requires_grad_(True)
    bias_r = bias.detach().float().requires_grad_(True)
    qr, kr, vr = (qkv_r[:, :, :, i].permute(0, 1, 3, 2, 4) for i in range(3))
    ref = attention_core_ref(qr, kr, vr, mask.float(), bias_r)
    ref.backward(g.float())
    assert (out.float() - ref).abs().max().item() < 2e-2
    gerr = (qkv.grad.float() - qkv_r.grad).abs().max().item()
    assert gerr < 3e-2 * max(1.0, qkv_r.grad.abs().max().item()), gerr
    # the masked rows on their own: dV there is mean(dO) / 1, small numbers that a factor-n error would swamp
    merr = (qkv.grad.float()[:, [2, 4]] - qkv_r.grad[:, [2, 4]]).abs().max().item()
    assert merr < 3e-2 * max(0.05, qkv_r.grad[:, [2, 4]].abs().max().item()), merr
    berr = (bias.grad.float() - bias_r.grad).abs().max().item()
    assert berr < 3e-2 * max(1.0, bias_r.grad.abs().max().item())


@pytest.mark.parametrize("B,n,H,use_bias", [(6, 256, 4, True), (5, 128, 8, False), (3, 200, 4, True)])
def test_packed_qkv_path(B, n, H, use_bias, device_status):
    """The packed entry (one QKV tensor in, one gradient tensor out) against the fp32 reference."""
    torch.manual_seed(B + n)
    qkv = (torch.randn(1, B, n, 3, H, 32, device=DEV) * 0.7).to(torch.bfloat16).requires_grad_(True)
    bias = torch.randn(1, 1, H, n, n, device=DEV).to(torch.bfloat16).requires_grad_(True) if use_bias else None
    mask = (torch.rand(1, B, n, device=DEV) > 0.2).to(torch.bfloat16)
    mask[..., 0] = 1
    assert flash.packed_supported(qkv, mask, bias)
    out = flash.flash_attention_packed(qkv, mask, bias, 32 ** -0.5)
    g = torch.randn_like(out)
    out.backward(g)
    qkv_r = qkv.detach().float().requires_grad_(True)
    bias_r = bias.detach().float().requires_grad_(True) if use_bias else None
    qr, kr, vr = (qkv_r[:, :, :, i].permute(0, 1, 3, 2, 4) for i in range(3))
    ref = attention_core_ref(qr, kr, vr, mask.float(), bias_r).permute(0, 1, 3, 2, 4).reshape(out.shape)
    ref.backward(g.float())
    assert (out.float() - ref).abs().max() < 2e-2
    gerr = (qkv.grad.float() - qkv_r.grad).abs().max().item()
    assert gerr < 3e-2 * max(1.0, qkv_r.grad.abs().max().item())
    if use_bias:
        berr = (bias.grad.float() - bias_r.grad).abs().max().item()
        assert berr < 3e-2 * max(1.0, bias_r.grad.abs().max().item())


def test_ending_node_strided_matches_transposed_reference(device_status):
    """Triangle attention around the ending node: GPU path (row / batch strides, no transposes; fused tail under
    no_grad, autograd under grad) against the same module in fp32 on the CPU (explicit transposes)."""
    from fastfold_b200.models.fastnn.ops import ChunkTriangleAttentionEndingNode
    torch.manual_seed(11)
    N, c = 64, 128
    ref = ChunkTriangleAttentionEndingNode(c, p_drop=0.25, c=32, n_head=4)
    with torch.no_grad():
        for p in ref.parameters():
            p.copy_(torch.randn_like(p) * 0.1)
    gpu = ChunkTriangleAttentionEndingNode(c, p_drop=0.25, c=32, n_head=4)
    gpu.load_state_dict(ref.state_dict())
    gpu = gpu.to(DEV, torch.bfloat16)
    ref.eval(); gpu.eval()
    z = torch.randn(1, N, N, c)
    mask = (torch.rand(1, N, N) > 0.1).float()
    mask[:, 0, :] = 1
    zg = z.to(DEV, torch.bfloat16)
    zr = zg.float().cpu().requires_grad_(True)
    with torch.no_grad():
        for p, q in zip(ref.parameters(), gpu.parameters()):
            p.copy_(q.float().cpu())
    out_ref = ref(zr, mask)
    assert gpu.strided(zg)
    with torch.no_grad():
        out_nograd = gpu(zg, mask.to(DEV, torch.bfloat16))
    assert (out_nograd.float().cpu() - out_ref.detach()).abs().max() < 0.06
    zg2 = zg.clone().requires_grad_(True)
    out_grad = gpu(zg2, mask.to(DEV, torch.bfloat16))
    assert (out_grad.float().cpu() - out_ref.detach()).abs().max() < 0.06
    g = torch.randn_like(out_ref)
    out_ref.backward(g)
    out_grad.backward(g.to(DEV, torch.bfloat16))
    err = (zg2.grad.float().cpu() - zr.grad).abs().max().item()
    assert err < 0.05 * max(1.0, zr.grad.abs().max().item()), err
    for (n_, p), q in zip(ref.named_parameters(), gpu.parameters()):
        e = (q.grad.float().cpu() - p.grad).abs().max().item()
        assert e < 0.06 * max(1.0, p.grad.abs().max().item()), (n_, e)


@pytest.mark.parametrize("B,n,H,use_bias,transposed", [(3, 640, 4, True, False), (2, 1024, 4, True, False), (2, 1024, 8, False, True),
                                                        (1, 2048, 4, True, False)])
def test_packed_backward_long_rows(B, n, H, use_bias, transposed, device_status):
    """Rows longer than the 512 queries whose gradient fits tensor memory: backward runs in blocks of 512 queries and sums
    the key / value gradients across the blocks; forward and all gradients against the fp32 reference."""
    torch.manual_seed(B * 31 + n)
    shape = (1, n, B, 3, H, 32) if transposed else (1, B, n, 3, H, 32)
    qkv = (torch.randn(*shape, device=DEV) * 0.7).to(torch.bfloat16).requires_grad_(True)
    bias = (torch.randn(1, 1, H, n, n, device=DEV)).to(torch.bfloat16).requires_grad_(True) if use_bias else None
    mask = (torch.rand(1, B, n, device=DEV) > 0.2).to(torch.bfloat16)
    mask[..., 0] = 1
    assert flash.packed_supported(qkv, mask, bias, transposed=transposed)
    out = flash.flash_attention_packed(qkv, mask, bias, 32 ** -0.5, transposed=transposed)
    g = torch.randn_like(out)
    out.backward(g)
    qkv_r = qkv.detach().float().requires_grad_(True)
    bias_r = bias.detach().float().requires_grad_(True) if use_bias else None
    src = qkv_r.transpose(1, 2) if transposed else qkv_r
    qr, kr, vr = (src[:, :, :, i].permute(0, 1, 3, 2, 4) for i in range(3))
    ref = attention_core_ref(qr, kr, vr, mask.float(), bias_r).permute(0, 1, 3, 2, 4).reshape(1, B, n, H * 32)
    if transposed:
        ref = ref.transpose(1, 2)
    ref.backward(g.float())
    assert (out.float() - ref).abs().max() < 2e-2
    gerr = (qkv.grad.float() - qkv_r.grad).abs().max().item()
    assert gerr < 3e-2 * max(1.0, qkv_r.grad.abs().max().item()), gerr
    if use_bias:
        berr = (bias.grad.float() - bias_r.grad).abs().max().item()
        assert berr < 3e-2 * max(1.0, bias_r.grad.abs().max().item()), berr


@pytest.mark.parametrize("c,heads", [(8, 8), (16, 4)])
def test_narrow_heads_train_on_the_fused_kernels(c, heads, device_status):
    """Gated self attention with 8- / 16-channel heads (extra-MSA rows, template triangles) under autograd: the module runs
    the fused kernels through differentiably zero-padded weights; outputs and every gradient against fp32 on the CPU."""
    from fastfold_b200.models.fastnn.ops import SelfAttention
    from fastfold_b200.ops import _lib
    torch.manual_seed(c)
    att = SelfAttention(64, c, heads, 64, gating=True)
    with torch.no_grad():
        for p in att.parameters():
            p.copy_(torch.randn_like(p) * 0.2)
    gpu = SelfAttention(64, c, heads, 64, gating=True)
    gpu.load_state_dict(att.state_dict())
    gpu = gpu.to(DEV, torch.bfloat16)
    with torch.no_grad():
        for p, q in zip(att.parameters(), gpu.parameters()):
            p.copy_(q.float().cpu())
    x = torch.randn(1, 6, 72, 64)
    xg = x.to(DEV, torch.bfloat16).requires_grad_(True)
    xr = xg.detach().float().cpu().requires_grad_(True)
    mask = (torch.rand(1, 6, 72) > 0.2).float()
    mask[..., 0] = 1
    bias = torch.randn(1, heads, 72, 72)
    n0 = _lib.LAUNCHES[0]
    out, _ = gpu(xg, mask.to(DEV, torch.bfloat16), (bias.to(DEV, torch.bfloat16), -1))
    assert _lib.LAUNCHES[0] - n0 >= 3
    ref, _ = att(xr, mask, (bias, -1))
    assert (out.float().cpu() - ref.detach()).abs().max() < 6e-2 * max(1.0, ref.abs().max().item())
    g = torch.randn_like(ref)
    ref.backward(g)
    out.backward(g.to(DEV, torch.bfloat16))
    assert (xg.grad.float().cpu() - xr.grad).abs().max() < 6e-2 * max(1.0, xr.grad.abs().max().item())
    for (name, p), q in zip(att.named_parameters(), gpu.parameters()):
        e = (q.grad.float().cpu() - p.grad).abs().max().item()
        assert e < 8e-2 * max(1.0, p.grad.abs().max().item()), (name, e)
