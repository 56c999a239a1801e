"""bf16 matrix products on the tcgen05 GEMM kernel (csrc/gemm_tcgen05.cu).

``gemm`` is the raw launcher (operands in either storage order, fused
epilogue); ``linear`` and ``bmm`` are autograd-aware wrappers whose backward
also runs on the same kernel (data gradient with the weight read MN-major,
weight gradient with both operands MN-major and split-K fp32 accumulation).
On CPU tensors everything is computed with PyTorch in fp32, which is also the
oracle the GPU tests compare against.

Stands in for the cuBLAS calls behind ``torch.matmul`` / ``nn.Linear`` /
``torch.einsum`` in the reference (fastfold/model/fastnn/ops.py:79-82,
143-160, 275-324, 393-404).
"""
import os

import torch

from . import _lib
from ._lib import ACT_NONE, ACT_RELU, ACT_SIGMOID, OUT_BF16, OUT_F32, OUT_F32_ATOMIC

_ACT = {None: ACT_NONE, "none": ACT_NONE, "relu": ACT_RELU, "sigmoid": ACT_SIGMOID}


def _as3d(t):
    return t if t.dim() == 3 else t.unsqueeze(0)


def gemm_ref(a, b, *, a_mn=False, b_mn=False, alpha=1.0, bias=None, act=None, glu=False, rowscale=None, mul=None,
             dmask=None, resid=None, trans_out=False, out_dtype=None):
    """fp32 PyTorch statement of what the kernel computes (same argument meaning as ``gemm``)."""
    A = a.float().transpose(-1, -2) if a_mn else a.float()
    B = b.float().transpose(-1, -2) if b_mn else b.float()
    v = alpha * torch.matmul(A, B.transpose(-1, -2))
    if bias is not None:
        v = v + bias.float()
    if _ACT[act] == ACT_RELU:
        v = torch.relu(v)
    elif _ACT[act] == ACT_SIGMOID:
        v = torch.sigmoid(v)
    if glu:
        v = v[..., 0::2] * torch.sigmoid(v[..., 1::2])
    if mul is not None:
        v = v * mul.float()
    if rowscale is not None:
        v = v * rowscale.float().unsqueeze(-1)
    if dmask is not None:
        m, div, mod = dmask
        rows = torch.arange(v.shape[-2], device=v.device)
        v = v * m.float()[(rows // div) % mod]
    if resid is not None:
        v = v + resid.float()
    if trans_out:
        v = v.transpose(-1, -2)
    return v.to(out_dtype or a.dtype)


def gemm(a, b, *, a_mn=False, b_mn=False, alpha=1.0, bias=None, act=None, glu=False, rowscale=None, mul=None,
         dmask=None, resid=None, trans_out=False, out=None, out_dtype=None, splits=1, accumulate=False, bn=0, peer=None, block_out=None):
    """``C = epilogue(alpha * A @ B^T)`` with A ``[.., M, K]`` and B ``[.., N, K]``.

    ``a_mn`` / ``b_mn``: the operand is stored with the contraction index
    strided, i.e. A is given as ``[.., K, M]`` / B as ``[.., K, N]``.
    Epilogue order: ``+bias -> act -> glu -> *mul -> *rowscale -> *dmask -> +resid``.
    ``dmask=(mask[mod, N], div, mod)`` picks mask row ``(m // div) % mod``.
    ``accumulate=True`` adds into an fp32 ``out`` with atomics (allows ``splits > 1``).
    A leading batch dimension may be present on either operand (a 2-D operand is
    shared by all batches).
    ``peer=("a" | "b", [address of every rank's slab])``: that operand is the concatenation, along its M / N extent,
    of one equally shaped slab per rank; the tensor passed in is this rank's slab (it supplies shape and strides)
    and the kernel fetches every slab's tiles from the given addresses - peer GPUs' memory - with TMA.
    ``block_out=(shape, mdiv, sr2, sr1, sc1)``: the bf16 result is stored block-permuted into a new tensor of ``shape``:
    with ``m = 32 m1 + m0`` and ``n = 32 n1 + n0``, element ``(m, n)`` lands at flat index
    ``(m1 // mdiv) sr2 + (m1 % mdiv) sr1 + n1 sc1 + 32 m0 + n0`` (every 32 x 32 block contiguous).  With ``d = e = 32``:
    ``[(i d), (j e)] -> [i, j, d, e]`` is ``(1, 1024 J, 0, 1024)`` and ``[(i j), (d e)] -> [(i d), (j e)]`` is
    ``(J // 32, 1024 J, 1024, 32 J)``.  Needs ``M % 32 == 0``, ``N % 64 == 0``.
    """
    if block_out is not None:
        assert out is None and not trans_out and not glu and mul is None and resid is None and a.dim() == 2 and b.dim() == 2
    if not a.is_cuda:
        if block_out is not None:
            shape, mdiv, sr2, sr1, sc1 = block_out
            r = gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn, alpha=alpha, bias=bias, act=act, rowscale=rowscale, dmask=dmask, out_dtype=out_dtype)
            Mr, Nr = r.shape
            res = torch.empty(shape, dtype=r.dtype)
            m1 = Mr // 32
            dst = torch.as_strided(res, (m1 // mdiv, mdiv, Nr // 32, 32, 32), (sr2, sr1, sc1, 32, 1))
            dst.copy_(r.reshape(m1 // mdiv, mdiv, 32, Nr // 32, 32).permute(0, 1, 3, 2, 4))
            return res
        r = gemm_ref(a, b, a_mn=a_mn, b_mn=b_mn, alpha=alpha, bias=bias, act=act, glu=glu, rowscale=rowscale, mul=mul,
                     dmask=dmask, resid=resid, trans_out=trans_out, out_dtype=out_dtype)
        if out is not None:
            if accumulate:
                out.add_(r.to(out.dtype))
            else:
                out.copy_(r)
            return out
        return r
    lib = _lib.get()
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16, "tcgen05 GEMM takes bf16 operands"
    if a.stride(-1) != 1:
        a = a.contiguous()
    if b.stride(-1) != 1:
        b = b.contiguous()
    batch = 1
    if a.dim() == 3:
        batch = a.shape[0]
    if b.dim() == 3:
        batch = max(batch, b.shape[0])
    a3, b3 = _as3d(a), _as3d(b)
    if a_mn:
        K, M = a3.shape[1], a3.shape[2]
    else:
        M, K = a3.shape[1], a3.shape[2]
    if b_mn:
        Kb, N = b3.shape[1], b3.shape[2]
    else:
        N, Kb = b3.shape[1], b3.shape[2]
    assert K == Kb, "contraction extents differ: %d vs %d" % (K, Kb)
    peer_slab = 0
    if peer is not None:
        which, addrs = peer
        if which == "a":
            peer_slab, M = M, M * len(addrs)
        else:
            peer_slab, N = N, N * len(addrs)
    n_out = N // 2 if glu else N
    batched = a.dim() == 3 or b.dim() == 3
    oshape = (n_out, M) if trans_out else (M, n_out)
    if batched:
        oshape = (batch,) + oshape
    blocked = None
    if block_out is not None:
        shape, mdiv, sr2, sr1, sc1 = block_out
        assert M % 32 == 0 and n_out % 64 == 0 and (M // 32) % mdiv == 0 and out_dtype in (None, torch.bfloat16)
        blocked = torch.empty(shape, device=a.device, dtype=torch.bfloat16)
        assert blocked.numel() == M * n_out
        out = blocked.view(-1).as_strided((M, n_out), (8, 1))          # carries shape and dtype through the checks; the kernel ignores ldc
    if out is None:
        odt = out_dtype or torch.bfloat16
        out = torch.empty(oshape, device=a.device, dtype=odt)
    else:
        assert tuple(out.shape) == tuple(oshape), "out has shape %s, expected %s" % (tuple(out.shape), oshape)
        assert out.stride(-1) == 1
    if out.dtype == torch.bfloat16:
        assert not accumulate
        mode = OUT_BF16
    else:
        assert out.dtype == torch.float32
        mode = OUT_F32_ATOMIC if accumulate else OUT_F32
    g = _lib.GemmArgs()
    g.M, g.N, g.K = M, N, K
    g.splits = splits if accumulate else 1
    g.out_mode = mode
    g.trans_out = 1 if trans_out else 0
    g.act = _ACT[act]
    g.glu = 1 if glu else 0
    g.alpha = float(alpha)
    g.C = out.data_ptr()
    g.ldc = out.stride(-2)
    g.c_bstride = out.stride(0) if batched else 0
    if blocked is not None:
        g.cq, g.cq_mdiv, g.cq_sr2, g.cq_sr1, g.cq_sc1 = 1, int(block_out[1]), int(block_out[2]), int(block_out[3]), int(block_out[4])
    keep = [a, b, out]
    if bias is not None:
        bias = bias.to(torch.bfloat16).contiguous()
        assert bias.numel() == N
        g.bias = bias.data_ptr()
        keep.append(bias)
    if rowscale is not None:
        rowscale = rowscale.to(torch.float32).contiguous()
        g.rowscale = rowscale.data_ptr()
        g.rs_bstride = M if (batched and rowscale.dim() == 2) else 0
        keep.append(rowscale)
    if mul is not None:
        assert mul.dtype == torch.bfloat16 and mul.stride(-1) == 1
        g.mul = mul.data_ptr()
        g.ldmul = mul.stride(-2)
        g.mul_bstride = mul.stride(0) if (batched and mul.dim() == 3) else 0
    if dmask is not None:
        m, div, mod = dmask
        assert m.dtype == torch.bfloat16 and m.stride(-1) == 1 and m.shape[-1] == n_out
        g.dmask = m.data_ptr()
        g.lddm = m.stride(-2) if m.dim() >= 2 else 0
        g.dm_div, g.dm_mod = int(div), int(mod)
    else:
        g.dm_div, g.dm_mod = 1, 1
    if resid is not None:
        assert resid.dtype == torch.bfloat16 and resid.stride(-1) == 1
        g.resid = resid.data_ptr()
        g.ldres = resid.stride(-2)
        g.res_bstride = resid.stride(0) if (batched and resid.dim() == 3) else 0
    if peer is not None:
        import ctypes
        which, addrs = peer
        g.peer_slab = peer_slab
        arr = (ctypes.c_void_p * len(addrs))(*[int(x) for x in addrs])
        rc = lib.ffb_gemm_bf16_peer(_lib.ptr(a3), _lib.ptr(b3), 1 if a_mn else 0, 1 if b_mn else 0, a3.stride(1), b3.stride(1),
                                    a3.stride(0) if a.dim() == 3 else 0, b3.stride(0) if b.dim() == 3 else 0, batch, g,
                                    1 if which == "a" else 2, arr, len(addrs), _lib.stream_ptr())
        _lib.check(rc, "ffb_gemm_bf16_peer(M=%d,N=%d,K=%d,batch=%d,slab=%d)" % (M, N, K, batch, peer_slab))
        return blocked if blocked is not None else out
    rc = lib.ffb_gemm_bf16(_lib.ptr(a3), _lib.ptr(b3), 1 if a_mn else 0, 1 if b_mn else 0, a3.stride(1), b3.stride(1),
                           a3.stride(0) if a.dim() == 3 else 0, b3.stride(0) if b.dim() == 3 else 0, batch, bn, g,
                           _lib.stream_ptr())
    _lib.check(rc, "ffb_gemm_bf16(M=%d,N=%d,K=%d,batch=%d)" % (M, N, K, batch))
    return blocked if blocked is not None else out


def _wgrad_splits(tokens, n_out_tiles):
    """Split-K factor so that a weight-gradient GEMM (few output tiles, long contraction) fills the 148 SMs."""
    kb = (tokens + 63) // 64
    # one work item per SM (half of that for a single output tile): measured faster than two per SM at every shape of
    # the model - the fp32 reductions of the splits into the same tile contend in L2
    want = max(1, (74 if n_out_tiles == 1 else 148) // max(1, n_out_tiles))
    return max(1, min(kb, want))


class _Linear(torch.autograd.Function):
    """y = act(x @ W^T + b) on [tokens, c_in]; all three GEMMs on the tcgen05 kernel."""

    @staticmethod
    def forward(ctx, x, w, bias, act):
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm(x2, w, bias=bias, act=act)
        ctx.act = act
        ctx.has_bias = bias is not None
        ctx.save_for_backward(x2, w, y if act else None)
        ctx.bias_ref = bias if (bias is not None and grad_sink(bias) is not None) else None
        ctx.xshape = x.shape
        return y.reshape(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        from . import fused_ops
        x2, w, y = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if dy2.stride(-1) != 1 or dy2.stride(0) != dy2.shape[1]:
            dy2 = dy2.contiguous()
        if ctx.act:
            dy2 = fused_ops.act_backward(dy2, y, ctx.act)
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).reshape(ctx.xshape)
        if ctx.needs_input_grad[1] and not sink_weight_grad(w, dy2, x2):
            dw = weight_grad(dy2, x2, w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            if not (ctx.bias_ref is not None and sink_bias_grad(ctx.bias_ref, dy2)):
                db = fused_ops.colsum(dy2).to(w.dtype)
        return dx, dw, db, None


class _LinearT(torch.autograd.Function):
    """y_t [c_out, tokens] = (x @ W^T + b)^T: the GEMM epilogue stores the transpose, and both gradient GEMMs read the
    channel-major output gradient in place (as an MN-major / K-major operand), so nothing is ever transposed."""

    @staticmethod
    def forward(ctx, x2, w, bias):
        ctx.save_for_backward(x2, w)
        ctx.has_bias = bias is not None
        return gemm(x2, w, bias=bias, trans_out=True)

    @staticmethod
    def backward(ctx, dy_t):
        x2, w = ctx.saved_tensors
        dy_t = dy_t.contiguous()                                  # [c_out, tokens]
        dx = dw = db = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy_t, w, a_mn=True, b_mn=True)              # [tokens, c_in]: contraction over c_out, both operands stored [c_out, .]
        if ctx.needs_input_grad[1]:
            n_out, n_in = w.shape
            sink = grad_sink(w)
            tiles = ((n_out + 127) // 128) * ((n_in + 127) // 128)
            splits = _wgrad_splits(x2.shape[0], tiles)
            if sink is not None:                                  # contraction over tokens, added into the trainer's buffer
                _ParamGradStream.run(lambda: gemm(dy_t, x2, b_mn=True, out=sink, accumulate=True, splits=splits), dy_t, x2)
            else:
                acc = torch.zeros(n_out, n_in, device=w.device, dtype=torch.float32)
                gemm(dy_t, x2, b_mn=True, out=acc, accumulate=True, splits=splits)
                dw = acc.to(w.dtype)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            db = torch.sum(dy_t, dim=1, dtype=torch.float32).to(w.dtype)      # converts inside the reduction, no fp32 copy
        return dx, dw, db


class _LinearTMulti(torch.autograd.Function):
    """``linear_t`` with the weight given as several parameters stacked along the output dimension (the four GLU
    projections of the triangle multiplication).  Forward concatenates them; backward computes one input-gradient GEMM
    and writes each parameter's gradient straight into its fp32 sink (on the parameter-gradient stream) instead of
    producing the concatenated gradient and letting autograd split and accumulate it."""

    @staticmethod
    def forward(ctx, x2, n, *wb):
        ws, bs = wb[:n], wb[n:]
        w = torch.cat([t.detach() for t in ws], dim=0)
        b = torch.cat([t.detach() for t in bs], dim=0)
        ctx.save_for_backward(x2, w)
        ctx.ws, ctx.bs = ws, bs
        return gemm(x2, w, bias=b, trans_out=True)

    @staticmethod
    def backward(ctx, dy_t):
        x2, w = ctx.saved_tensors
        dy_t = dy_t.contiguous()                                  # [sum c_out, tokens]
        dx = gemm(dy_t, w, a_mn=True, b_mn=True) if ctx.needs_input_grad[0] else None
        n_in = w.shape[1]
        grads_w, grads_b = [], []
        rowsum = torch.sum(dy_t, dim=1, dtype=torch.float32)
        off = 0
        for wi, bi in zip(ctx.ws, ctx.bs):
            n_out = wi.shape[0]
            sl = dy_t[off:off + n_out]
            tiles = ((n_out + 127) // 128) * ((n_in + 127) // 128)
            splits = _wgrad_splits(x2.shape[0], tiles)
            sink = grad_sink(wi)
            if sink is not None:
                _ParamGradStream.run(lambda sl=sl, sink=sink, splits=splits: gemm(sl, x2, b_mn=True, out=sink, accumulate=True, splits=splits), sl, x2)
                grads_w.append(None)
            else:
                acc = torch.zeros(n_out, n_in, device=w.device, dtype=torch.float32)
                gemm(sl, x2, b_mn=True, out=acc, accumulate=True, splits=splits)
                grads_w.append(acc.to(wi.dtype))
            sb = grad_sink(bi)
            rs = rowsum[off:off + n_out]
            if sb is not None:
                _ParamGradStream.run(lambda sb=sb, rs=rs: sb.reshape(-1).add_(rs), rs)
                grads_b.append(None)
            else:
                grads_b.append(rs.to(bi.dtype))
            off += n_out
        return (dx, None) + tuple(grads_w) + tuple(grads_b)


def linear_t_multi(x2, weights, biases):
    """``linear_t(x2, cat(weights), cat(biases))`` whose backward feeds each parameter's gradient sink directly."""
    n_out = sum(w.shape[0] for w in weights)
    ok = (x2.is_cuda and x2.dtype == torch.bfloat16 and x2.dim() == 2 and x2.shape[1] % 8 == 0 and x2.shape[0] % 8 == 0 and n_out >= 64
          and weights[0].shape[1] >= 64 and x2.shape[0] >= 64 and all(w.dtype == torch.bfloat16 and w.shape[0] % 8 == 0 for w in weights)
          and torch.is_grad_enabled())
    if not ok:
        return linear_t(x2, torch.cat(list(weights), dim=0), torch.cat(list(biases), dim=0))
    return _LinearTMulti.apply(x2, len(weights), *weights, *biases)


NARROW_LINEAR_T = True      # channel-major projections with fewer than 64 outputs (pair-bias heads) on the tcgen05 kernel


def linear_t(x2, w, bias=None):
    """``(x2 @ w.T + bias).T`` as a contiguous ``[c_out, tokens]`` tensor."""
    ok = (x2.is_cuda and x2.dtype == torch.bfloat16 and x2.dim() == 2 and x2.shape[1] % 8 == 0 and x2.shape[0] % 8 == 0
          and (w.shape[0] >= 64 or NARROW_LINEAR_T) and w.shape[1] >= 64 and x2.shape[0] >= 64 and w.dtype == torch.bfloat16)
    if not ok:
        return torch.nn.functional.linear(x2, w, bias).t().contiguous()
    if torch.is_grad_enabled() and (x2.requires_grad or w.requires_grad or (bias is not None and bias.requires_grad)):
        return _LinearT.apply(x2, w, bias)
    return gemm(x2, w, bias=bias, trans_out=True)


GRAD_SINK_ATTR = "_ffb_grad32"     # set by the trainer on a parameter: fp32 view of its slice of the flat gradient buffer


def grad_sink(param):
    """The fp32 accumulation buffer of a parameter when a trainer has provided one (gradient kernels then add into it
    directly and the autograd function returns no gradient for the parameter), else None."""
    return getattr(param, GRAD_SINK_ATTR, None)


class _ParamGradStream:
    """Parameter gradients off the critical path of backward.

    The gradient of an activation is needed by the next backward node; the gradient of a weight or bias only by the
    optimiser.  While a trainer has set ``active`` (around ``loss.backward()``), the kernels that add a parameter gradient
    into its fp32 sink are enqueued on a side stream that waits for the main stream at the point of the call, so they run
    beside the input-gradient chain (inside a captured step: a parallel branch of the graph).  The operands are kept
    alive in ``keep`` until ``join()``, which makes the main stream wait for the side stream; the trainer joins after
    every checkpointed segment and after backward.  FASTFOLD_WGRAD_STREAM=0 turns the side stream off."""
    enabled = os.environ.get("FASTFOLD_WGRAD_STREAM", "1") != "0"
    active = False
    stream = None
    keep = []
    forked = False

    @classmethod
    def run(cls, fn, *operands):
        if not (cls.active and cls.enabled and operands[0].is_cuda):
            fn()
            return
        if cls.stream is None:
            cls.stream = torch.cuda.Stream()
        cls.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(cls.stream):
            fn()
        cls.keep.extend(operands)
        cls.forked = True

    @classmethod
    def join(cls):
        if cls.forked:
            torch.cuda.current_stream().wait_stream(cls.stream)
            cls.forked = False
        cls.keep.clear()


param_grad_stream = _ParamGradStream


def sink_weight_grad(w, dy2, x2):
    """Adds dy^T @ x into the parameter's fp32 sink with the split-K GEMM; True when it did."""
    sink = grad_sink(w)
    n_out, n_in = dy2.shape[1], x2.shape[1]
    if sink is None or not dy2.is_cuda:
        return False
    if n_out < 64 or n_in < 64 or n_out % 8 or n_in % 8:
        # narrow projections (32-wide outer-product factors): the MN-major tile is 64 wide, so the product is a library
        # call; it still leaves the critical path and lands in the fp32 buffer without an autograd accumulation
        _ParamGradStream.run(lambda: sink.add_(torch.matmul(dy2.t(), x2)), dy2, x2)
        return True
    tiles = ((n_out + 127) // 128) * ((n_in + 127) // 128)
    splits = _wgrad_splits(dy2.shape[0], tiles)
    _ParamGradStream.run(lambda: gemm(dy2, x2, a_mn=True, b_mn=True, out=sink, accumulate=True, splits=splits), dy2, x2)
    return True


def sink_bias_grad(bias, dy2):
    """Adds the column sums of ``dy2`` into the bias parameter's fp32 sink; True when it did."""
    sink = grad_sink(bias)
    if sink is None or not (dy2.is_cuda and dy2.dtype == torch.bfloat16 and dy2.shape[-1] % 2 == 0):
        return False
    from . import fused_ops
    _ParamGradStream.run(lambda: fused_ops.colsum(dy2, out=sink.reshape(-1)), dy2)
    return True


def weight_grad(dy2, x2, dtype=torch.bfloat16):
    """dW[c_out, c_in] = dy^T @ x, contraction over tokens, fp32 split-K accumulation."""
    n_out, n_in = dy2.shape[1], x2.shape[1]
    if not dy2.is_cuda:
        return (dy2.float().t() @ x2.float()).to(dtype)
    if n_out < 64 or n_in < 64 or n_out % 8 or n_in % 8:
        # narrow projections (pair-bias heads, 32-wide outer-product factors): the MN-major tile is 64 wide
        return torch.matmul(dy2.t(), x2).to(dtype)
    acc = torch.zeros(n_out, n_in, device=dy2.device, dtype=torch.float32)
    tiles = ((n_out + 127) // 128) * ((n_in + 127) // 128)
    gemm(dy2, x2, a_mn=True, b_mn=True, out=acc, accumulate=True, splits=_wgrad_splits(dy2.shape[0], tiles))
    return acc.to(dtype)


def linear(x, w, bias=None, act=None):
    """``act(x @ w.T + bias)`` over the last dimension of ``x``."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or x.shape[-1] % 8 or w.shape[0] % 8:
        y = torch.nn.functional.linear(x, w, bias)
        if _ACT[act] == ACT_RELU:
            y = torch.relu(y)
        elif _ACT[act] == ACT_SIGMOID:
            y = torch.sigmoid(y)
        return y
    if torch.is_grad_enabled() and (x.requires_grad or w.requires_grad or (bias is not None and bias.requires_grad)):
        return _Linear.apply(x, w, bias, act)
    x2 = x.reshape(-1, x.shape[-1])
    return gemm(x2, w, bias=bias, act=act).reshape(*x.shape[:-1], w.shape[0])


class _BmmNT(torch.autograd.Function):
    """out[b] = A[b] @ B[b]^T for [b, M, K] x [b, N, K]; gradients on the same kernel."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return gemm(a, b)

    @staticmethod
    def backward(ctx, dout):
        a, b = ctx.saved_tensors
        dout = dout.contiguous()
        da = db = None
        if ctx.needs_input_grad[0]:
            da = gemm(dout, b, b_mn=True)          # [b, M, N] x [b, N, K] (contraction N, B stored [N, K])
        if ctx.needs_input_grad[1]:
            db = gemm(dout, a, a_mn=True, b_mn=True)  # dout^T [N, M] x a [M, K], contraction over M
        return da, db


def bmm_nt(a, b):
    """Batched ``a @ b.transpose(-1, -2)`` (both operands contraction-contiguous)."""
    ok = (a.is_cuda and a.dtype == torch.bfloat16 and a.shape[-1] % 8 == 0 and a.shape[-2] % 8 == 0
          and b.shape[-2] % 8 == 0 and a.shape[-2] >= 64 and b.shape[-2] >= 64)
    if not ok:
        return torch.matmul(a, b.transpose(-1, -2))
    a = a.contiguous()
    b = b.contiguous()
    if torch.is_grad_enabled() and (a.requires_grad or b.requires_grad):
        return _BmmNT.apply(a, b)
    return gemm(a, b)
