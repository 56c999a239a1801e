"""Fused elementwise regions (csrc/elementwise.cu) with hand-written gradients.

API of the reference's ``fastfold.model.fastnn.kernel`` JIT ops
(kernel/jit/fused_ops.py:5-22) is kept:

* ``bias_sigmod_ele(y, bias, z)``            -> ``sigmoid(y + bias) * z``
* ``bias_dropout_add(x, bias, dropmask, residual, prob, training)``
* ``bias_ele_dropout_residual(ab, b, g, dropout_mask, Z_raw, prob, training)``

In the reference ``dropmask`` is a tensor of ones shaped like one slice of the
activation and the op applies ``F.dropout`` to it.  Here the same call works
(ones in, dropout applied inside), and in addition a ready-made mask (values in
``{0, 1/(1-p)}``) can be passed with ``prob=0``: the trunk draws all masks of a
step up front so that activation-checkpoint recomputation and every DAP rank
see identical masks without touching RNG state.
"""
import torch
import torch.nn.functional as F

from . import _lib


def _bf16_cuda(*ts):
    return all(t is None or (t.is_cuda and t.dtype == torch.bfloat16) for t in ts)


def _rows_c(t):
    C = t.shape[-1]
    return t.numel() // C, C


def _mask_index(x, mask):
    """Maps a broadcastable mask ([.., 1, N, C] or [.., N, 1, C]) to (mask2d, div, mod) over flattened rows."""
    C = x.shape[-1]
    a, b = x.shape[-3], x.shape[-2]
    assert mask.shape[-1] == C
    lead = 1
    for s in mask.shape[:-3]:
        lead *= s
    assert lead == 1, "dropout mask must not have leading batch extent"
    ma, mb = (mask.shape[-3] if mask.dim() >= 3 else 1), mask.shape[-2]
    if ma == 1 and mb == b:          # shared along rows: mask index = row % b
        return mask.reshape(b, C), 1, b
    if ma == a and mb == 1:          # shared along columns: mask index = row // b
        return mask.reshape(a, C), b, a
    if ma == 1 and mb == 1:
        return mask.reshape(1, C), 1, 1
    raise ValueError("unsupported dropout mask shape %s for activation %s" % (tuple(mask.shape), tuple(x.shape)))


# ---------------------------------------------------------------------------
class _BiasSigmoidMul(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, bias, o):
        lib = _lib.get()
        gc, oc, bc = g.contiguous(), o.contiguous(), bias.contiguous()
        rows, C = _rows_c(gc)
        y = torch.empty_like(gc)
        _lib.check(lib.ffb_bias_sigmoid_mul_fwd(_lib.ptr(gc), _lib.ptr(bc), _lib.ptr(oc), _lib.ptr(y), rows, C, _lib.stream_ptr()),
                   "bias_sigmoid_mul_fwd")
        ctx.save_for_backward(gc, bc, oc)
        ctx.bias_param = bias
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib.get()
        gc, bc, oc = ctx.saved_tensors
        rows, C = _rows_c(gc)
        dg = torch.empty_like(gc)
        do = torch.empty_like(oc)
        dyc = dy.contiguous()
        _lib.check(lib.ffb_bias_sigmoid_mul_bwd(_lib.ptr(dyc), _lib.ptr(gc), _lib.ptr(bc), _lib.ptr(oc), _lib.ptr(dg), _lib.ptr(do),
                                                rows, C, _lib.stream_ptr()), "bias_sigmoid_mul_bwd")
        db = _bias_grad(ctx.bias_param, dg.reshape(rows, C), bc.dtype) if ctx.needs_input_grad[1] else None
        return dg, db, do


def bias_sigmod_ele(y, bias, z):
    if _bf16_cuda(y, bias, z) and y.shape == z.shape and y.shape[-1] % 8 == 0 and bias.numel() == y.shape[-1]:
        return _BiasSigmoidMul.apply(y, bias, z)
    return torch.sigmoid(y + bias) * z


# ---------------------------------------------------------------------------
class _BiasDropoutAdd(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, bias, m2, div, mod, resid):
        lib = _lib.get()
        xc, rc = x.contiguous(), resid.contiguous()
        rows, C = _rows_c(xc)
        y = torch.empty_like(xc)
        _lib.check(lib.ffb_bias_dropout_add_fwd(_lib.ptr(xc), _lib.ptr(bias), _lib.ptr(m2), _lib.ptr(rc), _lib.ptr(y), rows, C,
                                                div, mod, _lib.stream_ptr()), "bias_dropout_add_fwd")
        ctx.save_for_backward(m2)
        ctx.dm = (div, mod)
        ctx.has_bias = bias is not None
        ctx.bias_param = bias
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib.get()
        (m2,) = ctx.saved_tensors
        dyc = dy.contiguous()
        rows, C = _rows_c(dyc)
        if m2 is not None:
            dx = torch.empty_like(dyc)
            _lib.check(lib.ffb_mask_mul(_lib.ptr(dyc), _lib.ptr(m2), _lib.ptr(dx), rows, C, ctx.dm[0], ctx.dm[1], _lib.stream_ptr()),
                       "mask_mul")
        else:
            dx = dyc
        db = _bias_grad(ctx.bias_param, dx.reshape(rows, C), dyc.dtype) if (ctx.has_bias and ctx.needs_input_grad[1]) else None
        return dx, db, None, None, None, dyc


def bias_dropout_add(x, bias, dropmask, residual, prob, training=True):
    if dropmask is not None and training and prob > 0.0:
        dropmask = F.dropout(dropmask, p=prob, training=True)
    elif dropmask is not None and not training:
        dropmask = None
    if _bf16_cuda(x, bias, dropmask, residual) and x.shape == residual.shape and x.shape[-1] % 8 == 0 and x.dim() >= 3:
        if dropmask is not None:
            m2, div, mod = _mask_index(x, dropmask)
            m2 = m2.contiguous()
        else:
            m2, div, mod = None, 1, 1
        return _BiasDropoutAdd.apply(x, bias.contiguous() if bias is not None else None, m2, div, mod, residual)
    out = x if bias is None else x + bias
    if dropmask is not None:
        out = out * dropmask
    return residual + out


# ---------------------------------------------------------------------------
class _BiasEleDropoutRes(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ab, b, g, m2, div, mod, resid):
        lib = _lib.get()
        abc, gc, rc, bc = ab.contiguous(), g.contiguous(), resid.contiguous(), b.contiguous()
        rows, C = _rows_c(abc)
        y = torch.empty_like(abc)
        _lib.check(lib.ffb_bias_ele_dropout_res_fwd(_lib.ptr(abc), _lib.ptr(bc), _lib.ptr(gc), _lib.ptr(m2), _lib.ptr(rc), _lib.ptr(y),
                                                    rows, C, div, mod, _lib.stream_ptr()), "bias_ele_dropout_res_fwd")
        ctx.save_for_backward(abc, bc, gc, m2)
        ctx.dm = (div, mod)
        ctx.bias_param = b
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib.get()
        abc, bc, gc, m2 = ctx.saved_tensors
        dyc = dy.contiguous()
        rows, C = _rows_c(dyc)
        dab = torch.empty_like(abc)
        dg = torch.empty_like(gc)
        _lib.check(lib.ffb_bias_ele_dropout_res_bwd(_lib.ptr(dyc), _lib.ptr(abc), _lib.ptr(bc), _lib.ptr(gc), _lib.ptr(m2),
                                                    _lib.ptr(dab), _lib.ptr(dg), rows, C, ctx.dm[0], ctx.dm[1], _lib.stream_ptr()),
                   "bias_ele_dropout_res_bwd")
        db = _bias_grad(ctx.bias_param, dab.reshape(rows, C), bc.dtype) if ctx.needs_input_grad[1] else None
        return dab, db, dg, None, None, None, dyc


def bias_ele_dropout_residual(ab, b, g, dropout_mask, Z_raw, prob, training=True):
    if dropout_mask is not None and training and prob > 0.0:
        dropout_mask = F.dropout(dropout_mask, p=prob, training=True)
    elif dropout_mask is not None and not training:
        dropout_mask = None
    if _bf16_cuda(ab, b, g, dropout_mask, Z_raw) and ab.shape == Z_raw.shape == g.shape and ab.shape[-1] % 8 == 0 and ab.dim() >= 3:
        if dropout_mask is not None:
            m2, div, mod = _mask_index(ab, dropout_mask)
            m2 = m2.contiguous()
        else:
            m2, div, mod = None, 1, 1
        return _BiasEleDropoutRes.apply(ab, b, g, m2, div, mod, Z_raw)
    out = g * (ab + b)
    if dropout_mask is not None:
        out = out * dropout_mask
    return Z_raw + out


# ---------------------------------------------------------------------------
class _GluMask(torch.autograd.Function):
    @staticmethod
    def forward(ctx, p, q, rowmask):
        lib = _lib.get()
        pc, qc = p.contiguous(), q.contiguous()
        rows, C = _rows_c(pc)
        y = torch.empty_like(pc)
        rm = rowmask.to(torch.bfloat16).contiguous() if rowmask is not None else None
        _lib.check(lib.ffb_glu_mask_fwd(_lib.ptr(pc), _lib.ptr(qc), _lib.ptr(rm), _lib.ptr(y), rows, C, _lib.stream_ptr()), "glu_mask_fwd")
        ctx.save_for_backward(pc, qc, rm)
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib.get()
        pc, qc, rm = ctx.saved_tensors
        rows, C = _rows_c(pc)
        dyc = dy.contiguous()
        dp = torch.empty_like(pc)
        dq = torch.empty_like(qc)
        _lib.check(lib.ffb_glu_mask_bwd(_lib.ptr(dyc), _lib.ptr(pc), _lib.ptr(qc), _lib.ptr(rm), _lib.ptr(dp), _lib.ptr(dq), rows, C,
                                        _lib.stream_ptr()), "glu_mask_bwd")
        return dp, dq, None


def glu_mask(p, q, rowmask=None):
    """``rowmask[..., None] * p * sigmoid(q)``; ``rowmask`` has the shape of ``p`` without its last dim."""
    if _bf16_cuda(p, q) and p.shape == q.shape and p.shape[-1] % 8 == 0 and (rowmask is None or rowmask.numel() == p.numel() // p.shape[-1]):
        return _GluMask.apply(p, q, rowmask)
    out = p * torch.sigmoid(q)
    if rowmask is not None:
        out = out * rowmask.unsqueeze(-1).to(out.dtype)
    return out


# ---------------------------------------------------------------------------
class _GluMaskT(torch.autograd.Function):
    """Channel-major gated projection: ``pre [2 C2, R]`` (values, then gates) -> ``pre[:C2] * sigmoid(pre[C2:]) * mask[R]``,
    returned as its first ``split`` channels and the rest (two views of one buffer, so that autograd does not
    zero-fill and accumulate per slice)."""

    @staticmethod
    def forward(ctx, pre, mask, split):
        lib = _lib.get()
        C2, R = pre.shape[0] // 2, pre.shape[1]
        out = torch.empty(C2, R, device=pre.device, dtype=pre.dtype)
        _lib.check(lib.ffb_glu_mask_t_fwd(_lib.ptr(pre), _lib.ptr(mask), _lib.ptr(out), C2, R, _lib.stream_ptr()), "glu_mask_t_fwd")
        ctx.save_for_backward(pre, mask)
        ctx.split = split
        return out[:split], out[split:]

    @staticmethod
    def backward(ctx, d_lo, d_hi):
        lib = _lib.get()
        pre, mask = ctx.saved_tensors
        C2, R = pre.shape[0] // 2, pre.shape[1]
        if d_lo is None:
            d_lo = pre.new_zeros(ctx.split, R)
        if d_hi is None:
            d_hi = pre.new_zeros(C2 - ctx.split, R)
        dout = torch.cat([d_lo.reshape(ctx.split, R), d_hi.reshape(C2 - ctx.split, R)], dim=0)
        dpre = torch.empty_like(pre)
        _lib.check(lib.ffb_glu_mask_t_bwd(_lib.ptr(dout), _lib.ptr(pre), _lib.ptr(mask), _lib.ptr(dpre), C2, R, _lib.stream_ptr()), "glu_mask_t_bwd")
        return dpre, None, None


def glu_mask_t(pre, mask, split=None):
    """``pre [2 C2, R]`` channel-major (rows ``[0, C2)`` values, ``[C2, 2 C2)`` gates), ``mask [R]`` -> the gated product
    ``[C2, R]`` as the pair ``(first split channels, remaining channels)``; ``split`` defaults to ``C2 // 2``."""
    C2 = pre.shape[0] // 2
    split = C2 // 2 if split is None else split
    if _bf16_cuda(pre) and pre.is_contiguous() and pre.shape[1] % 8 == 0 and _lib.has("ffb_glu_mask_t_fwd"):
        return _GluMaskT.apply(pre, mask.reshape(-1).to(pre.dtype).contiguous(), split)
    out = pre[:C2] * torch.sigmoid(pre[C2:]) * mask.reshape(1, -1).to(pre.dtype)
    return out[:split], out[split:]


# ---------------------------------------------------------------------------
def global_attention_ref(q, kv, mask, gate, gate_bias):
    """fp32 reference of ``global_attention_core`` in plain PyTorch."""
    c = q.shape[-1]
    k, v = kv.float()[..., :c], kv.float()[..., c:]
    logits = torch.einsum("rhc,rsc->rhs", q.float(), k)
    logits = torch.where(mask[:, None, :] == 0, logits.new_full((), -1e9), logits)
    o = torch.einsum("rhs,rsc->rhc", torch.softmax(logits, dim=-1), v).reshape(q.shape[0], 1, -1)
    return torch.sigmoid(gate.float() + gate_bias.float()) * o


def global_attention_supported(q, kv, gate):
    H, c = q.shape[-2:]
    ok = (_bf16_cuda(q) and _bf16_cuda(kv) and _bf16_cuda(gate) and c in (8, 16, 32) and 256 % H == 0 and H * c <= 256
          and _lib.has("ffb_global_attention_fwd"))
    if ok and torch.is_grad_enabled() and (q.requires_grad or kv.requires_grad or gate.requires_grad):
        # training: the backward kernel folds the heads of one sequence with warp shuffles
        ok = 32 % H == 0 and 256 % (H * c) == 0 and _lib.has("ffb_global_attention_bwd")
    return ok


def _global_attention_fwd(q, kv, mask, gate, gate_bias):
    R, H, c = q.shape
    S = kv.shape[1]
    out = torch.empty_like(gate)
    _lib.check(_lib.get().ffb_global_attention_fwd(_lib.ptr(q), _lib.ptr(kv), _lib.ptr(mask), _lib.ptr(gate), _lib.ptr(gate_bias), _lib.ptr(out),
                                                   R, S, H, c, _lib.stream_ptr()), "global_attention_fwd")
    return out


class _GlobalAttentionFn(torch.autograd.Function):
    """Forward and backward of the global-attention core on the kernels of csrc/global_attention.cu."""

    @staticmethod
    def forward(ctx, q, kv, mask, gate, gate_bias):
        q, kv, gate = q.contiguous(), kv.contiguous(), gate.contiguous()
        mask = mask.to(q.dtype).contiguous()
        gb = gate_bias.to(q.dtype).contiguous()
        ctx.save_for_backward(q, kv, mask, gate, gb)
        ctx.bias_ref = gate_bias
        return _global_attention_fwd(q, kv, mask, gate, gb)

    @staticmethod
    def backward(ctx, dout):
        import ctypes
        q, kv, mask, gate, gb = ctx.saved_tensors
        R, H, c = q.shape
        S = kv.shape[1]
        dout = dout.contiguous()
        dq = torch.empty(R, H, c, device=q.device, dtype=torch.float32)
        dkv = torch.empty_like(kv)
        dgate = torch.empty_like(gate)
        lib = _lib.get()
        P, I, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong
        lib.ffb_global_attention_bwd.argtypes = [P] * 9 + [L, I, I, I, P]
        lib.ffb_global_attention_bwd.restype = I
        _lib.check(lib.ffb_global_attention_bwd(_lib.ptr(q), _lib.ptr(kv), _lib.ptr(mask), _lib.ptr(gate), _lib.ptr(gb), _lib.ptr(dout), _lib.ptr(dq),
                                                _lib.ptr(dkv), _lib.ptr(dgate), R, S, H, c, _lib.stream_ptr()), "global_attention_bwd")
        dgb = None
        if ctx.needs_input_grad[4]:
            from .gemm import sink_bias_grad
            if not sink_bias_grad(ctx.bias_ref, dgate.reshape(-1, H * c)):
                dgb = colsum(dgate.reshape(-1, H * c)).to(ctx.bias_ref.dtype)
        return dq.to(q.dtype), dkv, None, dgate, dgb


def global_attention_core(q, kv, mask, gate, gate_bias):
    """One query per (column, head), keys / values shared by the heads:  ``q [R, H, c]`` (projected and scaled),
    ``kv [R, S, 2c]`` (keys | values), ``mask [R, S]`` (0 = masked key, logit replaced by -1e9), ``gate [R, S, H*c]``
    (gating projection before bias and sigmoid), ``gate_bias [H*c]``  ->  ``sigmoid(gate + bias) * softmax(q k^T) v``
    broadcast over S, ``[R, S, H*c]``.  One kernel forward (one pass over ``kv`` and ``gate``), one kernel backward
    (``_GlobalAttentionFn``)."""
    if not global_attention_supported(q, kv, gate):
        return global_attention_ref(q, kv, mask, gate, gate_bias).to(gate.dtype)
    if torch.is_grad_enabled() and (q.requires_grad or kv.requires_grad or gate.requires_grad or gate_bias.requires_grad):
        return _GlobalAttentionFn.apply(q, kv, mask, gate, gate_bias)
    q, kv, gate = q.contiguous(), kv.contiguous(), gate.contiguous()
    return _global_attention_fwd(q, kv, mask.to(q.dtype).contiguous(), gate, gate_bias.to(q.dtype).contiguous())


# ---------------------------------------------------------------------------
def act_backward(dy2, y2, act):
    """dy * act'(pre-activation), expressed through the saved activation output."""
    mode = 1 if act == "relu" else 2
    if _bf16_cuda(dy2, y2) and dy2.shape[-1] % 8 == 0:
        lib = _lib.get()
        dyc, yc = dy2.contiguous(), y2.contiguous()
        rows, C = _rows_c(dyc)
        dx = torch.empty_like(dyc)
        _lib.check(lib.ffb_act_bwd(_lib.ptr(dyc), _lib.ptr(yc), _lib.ptr(dx), rows, C, mode, _lib.stream_ptr()), "act_bwd")
        return dx
    if mode == 1:
        return dy2 * (y2 > 0).to(dy2.dtype)
    return dy2 * y2 * (1 - y2)


def colsum(x2, out=None):
    """fp32 column sums of a 2-D tensor; with ``out`` (fp32 ``[C]``) the sums are ADDED into it."""
    if x2.is_cuda and x2.dtype == torch.bfloat16 and x2.shape[-1] % 2 == 0:
        lib = _lib.get()
        xc = x2.contiguous()
        if out is None:
            out = torch.zeros(xc.shape[-1], device=xc.device, dtype=torch.float32)
        _lib.check(lib.ffb_colsum(_lib.ptr(xc), _lib.ptr(out), xc.shape[0], xc.shape[1], _lib.stream_ptr()), "colsum")
        return out
    r = x2.float().sum(dim=0)
    if out is not None:
        out.add_(r)
        return out
    return r


def _bias_grad(bias_param, d2, dtype):
    """Bias gradient = column sums of ``d2``: added straight into the parameter's fp32 gradient sink when the trainer
    provides one (then no gradient tensor is returned to autograd)."""
    from .gemm import grad_sink
    sink = grad_sink(bias_param) if bias_param is not None else None
    if sink is not None and d2.is_cuda and d2.dtype == torch.bfloat16:
        colsum(d2, out=sink.reshape(-1))
        return None
    return colsum(d2).to(dtype)
