"""Split-phase collectives: launch now, consume later.

Same surface as the reference's ``fastfold/distributed/comm_async.py``:
``gather_async`` / ``gather_async_opp`` (returning ``(tensor, work)``),
``All_to_All_Async`` / ``All_to_All_Async_Opp`` and the broadcast trio.  The
work handle travels with the tensor instead of through a module-global
(comm_async.py:150), so several all-to-alls may be in flight at once, and the
gather's backward is a reduce-scatter (see ``comm.py``).
"""
import torch
import torch.distributed as dist

from . import core
from .comm import _all_to_all, _reduce_scatter, divide


def get_rank():
    return core.get_dap_rank()


def get_world_size():
    return core.get_dap_size()


def broadcast_sync(src, tensor, host=False):
    if core.get_dap_size() == 1:
        return tensor if host else 0
    g = core.get_dap_group()
    root = core.mesh().dap_ranks[src]
    if not host:
        out = tensor[0] if isinstance(tensor, (list, tuple)) else tensor
        if out is None:
            raise ValueError("non-root ranks pass a receive buffer")
        dist.broadcast(out, src=root, group=g)
        return out
    dist.broadcast(tensor, src=root, group=g)
    return tensor


def broadcast_async(src, tensor, host=False):
    if core.get_dap_size() == 1:
        return tensor, None
    root = core.mesh().dap_ranks[src]
    work = dist.broadcast(tensor, src=root, group=core.get_dap_group(), async_op=True)
    return tensor, work


def broadcast_async_opp(tensor, work=None):
    if work is not None:
        work.wait()
    return tensor


class _Finished:
    """``work`` of a collective whose kernel already produced the final layout (one-kernel push collectives)."""


_FINISHED = _Finished()


def _gather_async(tensor, dim):
    P = core.get_dap_size()
    if P == 1:
        return tensor, None
    t = tensor.contiguous()
    from .comm import _heap_for, _unit_ok
    h = _heap_for(t)
    d = dim % t.dim()
    if h is not None and h.fits_push(t.numel() * t.element_size()) and _unit_ok(t, d, 1):
        return h.gather_dim(t, d), _FINISHED      # asynchronous on the stream; already concatenated along ``dim``
    if h is not None:
        return h.all_gather(None, t), None     # the kernels are asynchronous on the stream already
    out = torch.empty((P,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    work = dist.all_gather_into_tensor(out.view((-1,) + tuple(t.shape[1:])), t, group=core.get_dap_group(), async_op=True)
    return out, work


def _finish_gather(out, work, dim):
    if work is _FINISHED:
        return out
    if work is not None:
        work.wait()
    if core.get_dap_size() == 1:
        return out
    P = out.shape[0]
    dim = dim % (out.dim() - 1)
    body = out.movedim(0, dim)
    shape = list(out.shape[1:])
    shape[dim] *= P
    return body.reshape(shape)


class GatherAsyncOpp(torch.autograd.Function):
    """The layout step that completes an asynchronous gather along dim 2 in the reference
    (fastfold/distributed/comm_async.py:98-110): the P received slabs, stacked along dim 1 as ``[n, (x h), w, c]``, are
    laid side by side along dim 2 -> ``[n, h, (x w), c]``.  Backward is the exact inverse rearrangement (the reference
    resizes the gradient buffer in place instead).  ``gather_async_opp`` of this package does this step itself; the
    class is kept for programs that call it directly."""

    @staticmethod
    def forward(ctx, input):
        x = get_world_size()
        n, xh, w, c = input.shape
        ctx.x = x
        return input.reshape(n, x, xh // x, w, c).permute(0, 2, 1, 3, 4).reshape(n, xh // x, x * w, c)

    @staticmethod
    def backward(ctx, grad_output):
        x = ctx.x
        n, h, xw, c = grad_output.shape
        return grad_output.reshape(n, h, x, xw // x, c).permute(0, 2, 1, 3, 4).reshape(n, x * h, xw // x, c)


class GatherAsync(torch.autograd.Function):
    """Launch + wait fused in one autograd node; forward returns the gathered tensor.

    The split-phase pair below (``gather_async`` / ``gather_async_opp``) is what
    model code calls; with autograd enabled ``gather_async`` defers to this node
    at ``_opp`` time so that the backward is a single reduce-scatter.
    """

    @staticmethod
    def forward(ctx, x, dim):
        ctx.dim = dim
        out, work = _gather_async(x, dim)
        return _finish_gather(out, work, dim)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter(g.contiguous(), ctx.dim), None


class _Pending:
    """Handle returned as ``work`` when autograd must see the gather as one node."""

    def __init__(self, src, dim):
        self.src = src
        self.dim = dim


def gather_async(tensor, dim=-1):
    """Starts an all-gather of ``tensor`` along ``dim`` over the DAP group -> ``(buffer, work)``."""
    if core.get_dap_size() == 1:
        return tensor, None
    if torch.is_grad_enabled() and tensor.requires_grad:
        return tensor, _Pending(tensor, dim)
    return _gather_async(tensor, dim)


def gather_async_opp(tensor, work, dim=-1):
    """Completes ``gather_async``; returns the gathered tensor."""
    if core.get_dap_size() == 1:
        return tensor
    if isinstance(work, _Pending):
        return GatherAsync.apply(work.src, work.dim)
    return _finish_gather(tensor, work, dim)


class _A2AWork:
    def __init__(self, work, shape, in_dim, out_dim, keep):
        self.work, self.shape, self.in_dim, self.out_dim, self.keep = work, shape, in_dim, out_dim, keep


class _A2ASync(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, in_dim, out_dim):
        ctx.dims = (in_dim, out_dim)
        return _all_to_all(x, in_dim, out_dim)

    @staticmethod
    def backward(ctx, g):
        return _all_to_all(g.contiguous(), ctx.dims[1], ctx.dims[0]), None, None


class _AsyncHandle:
    def __init__(self, src, in_dim, out_dim):
        self.src, self.in_dim, self.out_dim = src, in_dim, out_dim


def all_to_all_async(x, in_dim, out_dim):
    """Starts an all-to-all (split ``in_dim``, concatenate along ``out_dim``) -> ``(buffer, work)``."""
    P = core.get_dap_size()
    if P == 1:
        return x, None
    if torch.is_grad_enabled() and x.requires_grad:
        return x, _AsyncHandle(x, in_dim, out_dim)
    in_d = in_dim % x.dim()
    size = divide(x.shape[in_d], P)
    shape = list(x.shape)
    from .comm import _heap_for as _hf, _unit_ok
    hp = _hf(x) if x.is_cuda else None
    if hp is not None and hp.fits_push(x.numel() * x.element_size() // P) and _unit_ok(x, in_d, P) and _unit_ok(x, out_dim % x.dim(), 1, in_d, P):
        return hp.all_to_all_dims(x, in_d, out_dim % x.dim()), _FINISHED
    send = x.reshape(shape[:in_d] + [P, size] + shape[in_d + 1:]).movedim(in_d, 0).contiguous()
    from .comm import _heap_for
    h = _heap_for(send)
    if h is not None:
        return h.all_to_all(None, send), _A2AWork(None, shape, in_d, out_dim % x.dim(), None)
    recv = torch.empty_like(send)
    work = dist.all_to_all_single(recv, send, group=core.get_dap_group(), async_op=True)
    return recv, _A2AWork(work, shape, in_d, out_dim % x.dim(), send)


def all_to_all_async_opp(buf, work, in_dim, out_dim):
    if core.get_dap_size() == 1 or work is None or work is _FINISHED:
        return buf
    if isinstance(work, _AsyncHandle):
        return _A2ASync.apply(work.src, work.in_dim, work.out_dim)
    if work.work is not None:
        work.work.wait()
    P = core.get_dap_size()
    size = work.shape[work.in_dim] // P
    recv = buf.movedim(0, work.out_dim)
    oshape = list(work.shape)
    oshape[work.in_dim] = size
    oshape[work.out_dim] = work.shape[work.out_dim] * P
    return recv.reshape(oshape)


class _ApplyShim:
    """``X.apply(...)`` call style of the reference for the two all-to-all halves."""

    def __init__(self, fn):
        self.apply = fn


All_to_All_Async = _ApplyShim(all_to_all_async)
All_to_All_Async_Opp = _ApplyShim(lambda buf, work, in_dim=-1, out_dim=-1: all_to_all_async_opp(buf, work, in_dim, out_dim))
