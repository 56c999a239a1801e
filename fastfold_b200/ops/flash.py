"""Fused tcgen05 attention (csrc/attention_tcgen05.cu): dispatch, autograd wrapper.

``q, k, v`` arrive as ``[1, B, H, n, d]`` views of the fused QKV projection output ``[1, B, n, 3, H, d]``; the
kernel reads them in place through TMA (no head transposes) and writes ``[1, B, n, H*d]``, which is returned as
the ``[1, B, H, n, d]`` view the callers expect, so their ``permute + reshape`` back is free.
"""
import torch

from . import _lib

HEAD_DIM = 32


def _layout(t):
    """(pointer tensor, batch stride, row stride) if ``t [1, B, H, n, d]`` is addressable as (b, i, h, c) -> b*bs + i*rs + h*d + c."""
    if t.stride(-1) != 1 or t.stride(2) != t.shape[-1]:
        return None
    bs, rs = t.stride(1), t.stride(3)
    if bs % 8 or rs % 8 or t.data_ptr() % 16:
        return None
    return bs, rs


def supported(q, k, v, mask, bias):
    if not (q.is_cuda and q.dtype == torch.bfloat16 and q.dim() == 5 and q.shape[0] == 1 and q.shape[-1] == HEAD_DIM):
        return False
    if not _lib.has("ffb_attention_fwd"):
        return False
    if torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad or (bias is not None and bias.requires_grad)):
        if not _lib.has("ffb_attention_bwd"):
            return False
        if max(q.shape[3], k.shape[3]) > 512:
            return False
    n_k = k.shape[3]
    if n_k % 8:
        return False
    if bias is not None and (bias.shape[0] != 1 or bias.shape[1] != 1):
        return False
    return True


def _prep(q, k, v):
    outs = []
    for t in (q, k, v):
        lay = _layout(t)
        if lay is None:
            # re-pack as [1, B, n, H, d] contiguous, viewed back as [1, B, H, n, d]
            t = t.permute(0, 1, 3, 2, 4).contiguous().permute(0, 1, 3, 2, 4)
            lay = _layout(t)
        outs.append((t, lay))
    return outs


def _fwd(q, k, v, mask, bias, scale, want_lse):
    lib = _lib.get()
    (q, (qbs, qrs)), (k, (kbs, krs)), (v, (vbs, vrs)) = _prep(q, k, v)
    if (kbs, krs) != (vbs, vrs):
        v = v.permute(0, 1, 3, 2, 4).contiguous().permute(0, 1, 3, 2, 4)
        k = k.permute(0, 1, 3, 2, 4).contiguous().permute(0, 1, 3, 2, 4)
        kbs, krs = _layout(k)
    _, B, H, n_q, d = q.shape
    n_k = k.shape[3]
    out = torch.empty(1, B, n_q, H * d, device=q.device, dtype=q.dtype)
    lse = torch.empty(B, H, n_q, device=q.device, dtype=torch.float32) if want_lse else None
    b3 = bias.reshape(H, n_q, n_k).contiguous() if bias is not None else None
    m2 = mask.reshape(B, n_k).to(torch.bfloat16).contiguous() if mask is not None else None
    rc = lib.ffb_attention_fwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), qbs, qrs, kbs, krs, _lib.ptr(b3), _lib.ptr(m2), n_k,
                               _lib.ptr(out), n_q * H * d, H * d, _lib.ptr(lse), B, H, n_q, n_k, d, float(scale), _lib.stream_ptr())
    _lib.check(rc, "ffb_attention_fwd(B=%d,H=%d,n=%d/%d)" % (B, H, n_q, n_k))
    return out, lse, (q, k, v, b3, m2)


class _FlashFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, mask, bias, scale):
        out, lse, (q, k, v, b3, m2) = _fwd(q, k, v, mask, bias, scale, True)
        ctx.save_for_backward(q, k, v, b3, m2, out, lse)
        ctx.scale = scale
        ctx.bias_shape = None if bias is None else tuple(bias.shape)
        _, B, n_q, HD = out.shape
        H = q.shape[2]
        return out.view(1, B, n_q, H, HD // H).permute(0, 1, 3, 2, 4)

    @staticmethod
    def backward(ctx, do):
        lib = _lib.get()
        q, k, v, b3, m2, out, lse = ctx.saved_tensors
        _, B, H, n_q, d = q.shape
        n_k = k.shape[3]
        do_c = do.permute(0, 1, 3, 2, 4).contiguous()            # [1, B, n_q, H, d]
        dqkv = torch.empty(3, B, max(n_q, n_k), H * d, device=q.device, dtype=q.dtype)
        ds = torch.empty(B, H, n_q, n_k, device=q.device, dtype=q.dtype) if b3 is not None else None
        qbs, qrs = _layout(q)
        kbs, krs = _layout(k)
        rc = lib.ffb_attention_bwd(_lib.ptr(q), _lib.ptr(k), _lib.ptr(v), qbs, qrs, kbs, krs, _lib.ptr(b3), _lib.ptr(m2), n_k,
                                   _lib.ptr(out), _lib.ptr(do_c), _lib.ptr(lse), _lib.ptr(dqkv), _lib.ptr(ds), B, H, n_q, n_k, d,
                                   float(ctx.scale), _lib.stream_ptr())
        _lib.check(rc, "ffb_attention_bwd(q=%s strides=%s ptr=%x k strides=%s B=%d H=%d n=%d/%d)" % (
            tuple(q.shape), q.stride(), q.data_ptr(), k.stride(), B, H, n_q, n_k))
        dq = dqkv[0, :, :n_q].view(1, B, n_q, H, d).permute(0, 1, 3, 2, 4)
        dk = dqkv[1, :, :n_k].view(1, B, n_k, H, d).permute(0, 1, 3, 2, 4)
        dv = dqkv[2, :, :n_k].view(1, B, n_k, H, d).permute(0, 1, 3, 2, 4)
        dbias = None
        if ds is not None and ctx.needs_input_grad[4]:
            dbias = ds.sum(dim=0).reshape(ctx.bias_shape)
        return dq, dk, dv, None, dbias, None


def flash_attention(q, k, v, mask, bias, scale):
    need_grad = torch.is_grad_enabled() and (q.requires_grad or k.requires_grad or v.requires_grad or
                                             (bias is not None and bias.requires_grad))
    if need_grad:
        return _FlashFn.apply(q, k, v, mask, bias, scale)
    out, _, _ = _fwd(q, k, v, mask, bias, scale, False)
    _, B, n_q, HD = out.shape
    H = q.shape[2]
    return out.view(1, B, n_q, H, HD // H).permute(0, 1, 3, 2, 4)
