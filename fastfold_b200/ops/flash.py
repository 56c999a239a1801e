"""Fused tcgen05 attention (csrc/attention_tcgen05.cu): dispatch, autograd wrapper.

``q, k, v`` arrive as ``[1, B, H, n, d]`` views of the fused QKV projection output ``[1, B, n, 3, H, d]``; the
kernel reads them in place through TMA (no head transposes) and writes ``[1, B, n, H*d]``, which is returned as
the ``[1, B, H, n, d]`` view the callers expect, so their ``permute + reshape`` back is free.
"""
import torch

from . import _lib

HEAD_DIM = 32
MAX_BWD_QUERIES = 512      # queries of one (row, head) whose gradient the backward kernel holds in tensor memory


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


# ---------------------------------------------------------------------------
# Packed path: the fused QKV projection output goes in as one tensor and its gradient comes back as one tensor,
# written in place by the backward kernel (no per-slice zero-fill / copy / accumulate in autograd).  With
# ``transposed=True`` the attention runs along dim 1 of ``qkv [1, n, B, 3, H, d]`` (batch = dim 2): the kernels take
# row / batch strides, so the triangle attention around the ending node needs no transposed copy of the pair tensor.
# ---------------------------------------------------------------------------
def packed_supported(qkv, mask, bias, transposed=False):
    """``qkv [1, B, n, 3, H, d]`` (or ``[1, n, B, 3, H, d]``) contiguous bf16 on a GPU, self attention."""
    if not (qkv.is_cuda and qkv.dtype == torch.bfloat16 and qkv.dim() == 6 and qkv.shape[0] == 1 and qkv.shape[3] == 3
            and qkv.shape[-1] == HEAD_DIM and qkv.is_contiguous() and qkv.data_ptr() % 16 == 0):
        return False
    if not (_lib.has("ffb_attention_fwd") and _lib.has("ffb_attention_bwd_strided")):
        return False
    n = qkv.shape[1] if transposed else qkv.shape[2]
    if n % 8:
        return False
    if bias is not None and (bias.dim() != 5 or bias.shape[0] != 1 or bias.shape[1] != 1):
        return False
    return True


def _packed_geometry(qkv, transposed):
    """B, n, H, d and the (batch, row) strides of the q/k/v slabs and of the output."""
    if transposed:
        _, n, B, _, H, d = qkv.shape
        HD = H * d
        return B, n, H, d, (3 * HD, B * 3 * HD), (HD, B * HD)
    _, B, n, _, H, d = qkv.shape
    HD = H * d
    return B, n, H, d, (n * 3 * HD, 3 * HD), (n * HD, HD)


def _packed_fwd(qkv, mask, bias, scale, want_lse, transposed):
    lib = _lib.get()
    B, n, H, d, (bs, rs), (obs, ors) = _packed_geometry(qkv, transposed)
    HD = H * d
    out = torch.empty((1, n, B, HD) if transposed else (1, B, n, HD), device=qkv.device, dtype=qkv.dtype)
    lse = torch.empty(B, H, n, device=qkv.device, dtype=torch.float32) if want_lse else None
    b3 = bias.reshape(H, n, n).contiguous() if bias is not None else None
    m2 = mask.reshape(B, n).to(torch.bfloat16).contiguous() if mask is not None else None
    base = qkv.data_ptr()
    rc = lib.ffb_attention_fwd(base, base + 2 * HD, base + 4 * HD, bs, rs, bs, rs, _lib.ptr(b3), _lib.ptr(m2), n,
                               _lib.ptr(out), obs, ors, _lib.ptr(lse), B, H, n, n, d, float(scale), _lib.stream_ptr())
    _lib.check(rc, "ffb_attention_fwd packed (B=%d,H=%d,n=%d)" % (B, H, n))
    return out, lse, b3, m2


class _FlashPackedFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, mask, bias, scale, transposed):
        out, lse, b3, m2 = _packed_fwd(qkv, mask, bias, scale, True, transposed)
        ctx.save_for_backward(qkv, b3, m2, out, lse)
        ctx.scale, ctx.transposed = scale, transposed
        ctx.bias_shape = None if bias is None else tuple(bias.shape)
        return out

    @staticmethod
    def backward(ctx, do):
        lib = _lib.get()
        qkv, b3, m2, out, lse = ctx.saved_tensors
        B, n, H, d, (bs, rs), (obs, ors) = _packed_geometry(qkv, ctx.transposed)
        HD = H * d
        do = do.contiguous()
        dqkv = torch.empty_like(qkv)
        base, gbase = qkv.data_ptr(), dqkv.data_ptr()
        want_dbias = b3 is not None and ctx.needs_input_grad[2]
        if n <= MAX_BWD_QUERIES:
            ds = torch.empty(B, H, n, n, device=qkv.device, dtype=qkv.dtype) if b3 is not None else None
            rc = lib.ffb_attention_bwd_strided(base, base + 2 * HD, base + 4 * HD, bs, rs, bs, rs, _lib.ptr(b3), _lib.ptr(m2), n, _lib.ptr(out),
                                               _lib.ptr(do), obs, ors, _lib.ptr(lse), gbase, gbase + 2 * HD, gbase + 4 * HD, bs, rs, bs, rs,
                                               _lib.ptr(ds), B, H, n, n, d, float(ctx.scale), _lib.stream_ptr())
            _lib.check(rc, "ffb_attention_bwd_strided (B=%d,H=%d,n=%d)" % (B, H, n))
            dbias = ds.sum(dim=0).reshape(ctx.bias_shape) if want_dbias else None
            return dqkv, None, dbias, None, None
        # Long rows: the kernel keeps the query gradients of one (row, head) in tensor memory, which holds 512 queries.
        # Longer rows go through it in blocks of 512 queries against ALL keys: each call writes its block of dq in place
        # and a partial dk / dv over the whole row, which are summed in fp32 across the blocks.
        es = qkv.element_size()
        part = torch.empty(2, B, n, HD, device=qkv.device, dtype=qkv.dtype)
        acc = torch.zeros(2, B, n, HD, device=qkv.device, dtype=torch.float32)
        dbias = torch.empty(H, n, n, device=qkv.device, dtype=qkv.dtype) if want_dbias else None
        for c0 in range(0, n, MAX_BWD_QUERIES):
            nq = min(MAX_BWD_QUERIES, n - c0)
            lse_c = lse[:, :, c0:c0 + nq].contiguous()
            b_c = b3[:, c0:c0 + nq].contiguous() if b3 is not None else None
            ds = torch.empty(B, H, nq, n, device=qkv.device, dtype=qkv.dtype) if b3 is not None else None
            rc = lib.ffb_attention_bwd_strided(base + c0 * rs * es, base + 2 * HD, base + 4 * HD, bs, rs, bs, rs, _lib.ptr(b_c), _lib.ptr(m2), n,
                                               out.data_ptr() + c0 * ors * es, do.data_ptr() + c0 * ors * es, obs, ors, _lib.ptr(lse_c),
                                               gbase + c0 * rs * es, _lib.ptr(part[0]), _lib.ptr(part[1]), bs, rs, n * HD, HD, _lib.ptr(ds),
                                               B, H, nq, n, d, float(ctx.scale), _lib.stream_ptr())
            _lib.check(rc, "ffb_attention_bwd_strided (B=%d,H=%d,n=%d, queries %d..%d)" % (B, H, n, c0, c0 + nq))
            acc += part
            if want_dbias:
                dbias[:, c0:c0 + nq] = ds.sum(dim=0)
            del ds
        # dk / dv slabs of the packed gradient: element (b, i, h, c) at gbase + (1 | 2) * HD + b * bs + i * rs
        gk = torch.as_strided(dqkv, (2, B, n, HD), (HD, bs, rs, 1), storage_offset=dqkv.storage_offset() + HD)
        gk.copy_(acc)
        return dqkv, None, (dbias.reshape(ctx.bias_shape) if want_dbias else None), None, None


def flash_attention_packed(qkv, mask, bias, scale, transposed=False):
    """``qkv [1, B, n, 3, H, d]`` -> ``[1, B, n, H*d]`` (heads side by side, ready for gating / output projection);
    ``transposed``: ``qkv [1, n, B, 3, H, d]`` -> ``[1, n, B, H*d]``, ``mask [.., B, n]``."""
    need_grad = torch.is_grad_enabled() and (qkv.requires_grad or (bias is not None and bias.requires_grad))
    if need_grad:
        return _FlashPackedFn.apply(qkv, mask, bias, scale, transposed)
    return _packed_fwd(qkv, mask, bias, scale, False, transposed)[0]
