"""Synchronous DAP collectives with autograd (NCCL / Gloo through torch.distributed).

Same surface as the reference's ``fastfold/distributed/comm.py``: ``_reduce``,
``_split``, ``_gather``, the autograd pairs ``copy`` / ``scatter`` / ``reduce``
/ ``gather``, and the axis switches ``row_to_col`` / ``col_to_row`` on
``[1, A, B, c]`` tensors (dims 1 <-> 2).  Two differences, both on purpose:

* ``gather(..., reduce_grad=True)`` back-propagates with a *reduce-scatter*.
  The reference always slices the incoming gradient locally (comm.py:141-143),
  which is right only when every rank consumes the gathered tensor in the same
  replicated computation (the gather after the last block).  When each rank
  uses the gathered operand for its own shard of the output (pair bias,
  triangle-multiplication and outer-product operands) the gradient
  contributions of all ranks have to be summed.
* all-to-all uses ``all_to_all_single`` on one buffer instead of a list of
  chunks plus ``torch.cat``.

These are the baseline collectives; the fused P2P kernels in
``parallel/fused.py`` replace them on the hot path on GPUs.
"""
import torch
import torch.distributed as dist

from . import core


def divide(numerator, denominator):
    core.ensure_divisibility(numerator, denominator)
    return numerator // denominator


def _P():
    return core.get_dap_size()


def _heap_for(t):
    """Symmetric heap to use for this tensor, or None (CPU tensors, odd sizes, NCCL baseline selected)."""
    if not t.is_cuda:
        return None
    from . import symm
    h = symm.get_heap("dap")
    if h is None:
        return None
    nb = t.numel() * t.element_size()
    # messages larger than a ring slot (long sequences) go through NCCL, which is bandwidth-bound there anyway
    return h if (nb % (16 * h.world) == 0 and 0 < nb <= h.max_message()) else None


def _unit_ok(t, dim, parts, shrink_dim=None, shrink=1):
    """True when the contiguous run behind ``dim`` (of ``t`` with ``dim`` split in ``parts``, and ``shrink_dim`` divided by
    ``shrink``) is a whole number of 16-byte units - the granularity of the push collectives' placement."""
    shape = list(t.shape)
    if shrink_dim is not None:
        shape[shrink_dim] //= shrink
    run = shape[dim] // parts
    for d in shape[dim + 1:]:
        run *= d
    return (run * t.element_size()) % 16 == 0


def _reduce(tensor):
    if _P() == 1:
        return tensor
    dist.all_reduce(tensor, op=dist.ReduceOp.SUM, group=core.get_dap_group())
    return tensor


def _split(tensor, dim=-1):
    if _P() == 1:
        return tensor
    size = divide(tensor.shape[dim], _P())
    return tensor.narrow(dim, core.get_dap_rank() * size, size).contiguous()


def _gather(tensor, dim=-1):
    P = _P()
    if P == 1:
        return tensor
    dim = dim % tensor.dim()
    t = tensor.contiguous()
    h = _heap_for(t)
    if h is not None and h.fits_push(t.numel() * t.element_size()) and _unit_ok(t, dim, 1):
        return h.gather_dim(t, dim)          # one kernel, result already concatenated along ``dim``
    if h is not None:
        out = h.all_gather(None, t)
    else:
        out = torch.empty((P,) + tuple(t.shape), dtype=t.dtype, device=t.device)
        dist.all_gather_into_tensor(out.view((-1,) + tuple(t.shape[1:])), t, group=core.get_dap_group())
    if dim == 0:
        return out.reshape((P * t.shape[0],) + tuple(t.shape[1:]))
    # [P, d0, .., dim, ..] -> [d0, .., P*dim, ..]
    out = out.movedim(0, dim)
    shape = list(t.shape)
    shape[dim] *= P
    return out.reshape(shape)


def _reduce_scatter(tensor, dim):
    """Sum over the DAP group, keep this rank's slice along ``dim``."""
    P = _P()
    if P == 1:
        return tensor
    dim = dim % tensor.dim()
    size = divide(tensor.shape[dim], P)
    shape = list(tensor.shape)
    shape[dim] = size
    if tensor.is_cuda and tensor.dtype == torch.bfloat16:
        h = _heap_for(tensor)
        if h is not None and h.fits_push(tensor.numel() * tensor.element_size() // P) and (tensor.numel() // P * tensor.element_size()) % 16 == 0 \
                and _unit_ok(tensor, dim, P):
            # one kernel: slice q of every rank lands in rank q's slot and is summed there in fp32
            return h.reduce_scatter_dim(tensor, dim)
    # bring the P chunks to the front so that the collective works on one contiguous buffer
    t = tensor.reshape(shape[:dim] + [P, size] + shape[dim + 1:]).movedim(dim, 0).contiguous()
    h = _heap_for(t)
    if h is not None:
        # chunk q of every rank travels to rank q (NVLink traffic of a reduce-scatter), summed locally in fp32
        return h.all_to_all(None, t).float().sum(dim=0).to(tensor.dtype)
    out = torch.empty(shape, dtype=tensor.dtype, device=tensor.device)
    if dist.get_backend(core.get_dap_group()) == "gloo":
        dist.all_reduce(t, op=dist.ReduceOp.SUM, group=core.get_dap_group())
        out.copy_(t[core.get_dap_rank()])
    else:
        dist.reduce_scatter_tensor(out, t, op=dist.ReduceOp.SUM, group=core.get_dap_group())
    return out


def _all_to_all(tensor, in_dim, out_dim):
    """Splits ``in_dim`` over the ranks and concatenates what arrives along ``out_dim``."""
    P = _P()
    if P == 1:
        return tensor
    in_dim, out_dim = in_dim % tensor.dim(), out_dim % tensor.dim()
    size = divide(tensor.shape[in_dim], P)
    shape = list(tensor.shape)
    if tensor.is_cuda:
        h = _heap_for(tensor)
        if h is not None and h.fits_push(tensor.numel() * tensor.element_size() // P) and _unit_ok(tensor, in_dim, P) \
                and _unit_ok(tensor, out_dim, 1, in_dim, P):
            return h.all_to_all_dims(tensor, in_dim, out_dim)     # one kernel, no permuted copies on either side
    send = tensor.reshape(shape[:in_dim] + [P, size] + shape[in_dim + 1:]).movedim(in_dim, 0).contiguous()
    h = _heap_for(send)
    if h is not None:
        recv = h.all_to_all(None, send)
    else:
        recv = torch.empty_like(send)
        dist.all_to_all_single(recv, send, group=core.get_dap_group())
    # recv[p] = chunk from rank p, shaped like tensor with in_dim -> size
    recv = recv.movedim(0, out_dim)   # [.., P, out, ..] with P placed before out_dim's extent
    oshape = list(shape)
    oshape[in_dim] = size
    oshape[out_dim] = shape[out_dim] * P
    return recv.reshape(oshape)


class Copy(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return x

    @staticmethod
    def backward(ctx, g):
        return _reduce(g.contiguous())


class Scatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim):
        ctx.dim = dim
        return _split(x, dim)

    @staticmethod
    def backward(ctx, g):
        return _gather(g, ctx.dim), None


class Reduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x):
        return _reduce(x.clone())

    @staticmethod
    def backward(ctx, g):
        return g


class Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim, reduce_grad):
        ctx.dim = dim
        ctx.reduce_grad = reduce_grad
        return _gather(x, dim)

    @staticmethod
    def backward(ctx, g):
        if ctx.reduce_grad:
            return _reduce_scatter(g, ctx.dim), None, None
        return _split(g, ctx.dim), None, None


class All_to_All(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, in_dim, out_dim):
        ctx.dims = (in_dim, out_dim)
        return _all_to_all(x, in_dim, out_dim)

    @staticmethod
    def backward(ctx, g):
        return _all_to_all(g, ctx.dims[1], ctx.dims[0]), None, None


def copy(x):
    if torch.is_grad_enabled() and x.requires_grad and _P() > 1:
        return Copy.apply(x)
    return x


def scatter(x, dim=-1):
    if _P() == 1:
        return x
    if torch.is_grad_enabled() and x.requires_grad:
        return Scatter.apply(x, dim)
    return _split(x, dim)


def scatter_mask(x, dim=-1):
    """``scatter`` for a mask (no gradient, read-only): every block of a stack scatters the same tensor, so the shard
    is computed once per stack call (utils/memo.py)."""
    if _P() == 1:
        return x
    from ..utils import memo
    return memo.cached(("split", dim % x.dim()), (x,), lambda: _split(x, dim))


def reduce(x):
    if _P() == 1:
        return x
    if torch.is_grad_enabled() and x.requires_grad:
        return Reduce.apply(x)
    return _reduce(x.clone())


def gather(x, dim=-1, reduce_grad=False):
    if _P() == 1:
        return x
    if torch.is_grad_enabled() and x.requires_grad:
        return Gather.apply(x, dim, reduce_grad)
    return _gather(x, dim)


def col_to_row(x):
    """[1, A, B/P, c] -> [1, A/P, B, c]"""
    if _P() == 1:
        return x
    if torch.is_grad_enabled() and x.requires_grad:
        return All_to_All.apply(x, 1, 2)
    return _all_to_all(x, 1, 2)


def row_to_col(x):
    """[1, A/P, B, c] -> [1, A, B/P, c]"""
    if _P() == 1:
        return x
    if torch.is_grad_enabled() and x.requires_grad:
        return All_to_All.apply(x, 2, 1)
    return _all_to_all(x, 2, 1)
