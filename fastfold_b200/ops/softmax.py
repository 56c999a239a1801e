"""``fused_softmax(x, mask=None, bias=None)`` (csrc/softmax.cu).

Same call as the reference's ``fastfold.model.fastnn.kernel.fused_softmax``
(kernel/softmax.py:21-59): ``x [b1, b2, H, Q, K]``, ``mask [b1, b2, K]`` (zeros
mark masked keys, whose logits are replaced by -1e9), ``bias [b1, 1, H, Q, K]``
broadcast over ``b2``.  4-D inputs ``[b1, b2, H, K]`` (global attention) are
accepted too.  Unlike the reference's kernels the result is written out of
place, the mask row is located from ``(b1, b2)`` for any ``Q``, and the
gradient is exact for rows longer than 1024.
"""
import torch

from . import _lib


def softmax_ref(x, mask=None, bias=None):
    v = x.float()
    if bias is not None:
        v = v + bias.float()
    if mask is not None:
        m = mask
        while m.dim() < v.dim():
            m = m.unsqueeze(-2)
        v = torch.where(m == 0, torch.full_like(v, -1e9), v)
    return torch.softmax(v, dim=-1).to(x.dtype)


class _SoftmaxFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mask, bias):
        lib = _lib.get()
        squeeze = x.dim() == 4
        x5 = x.unsqueeze(-2) if squeeze else x
        B1, B2, H, Q, K = x5.shape
        xc = x5.contiguous()
        y = torch.empty_like(xc)
        mk = mask.to(x.dtype).contiguous() if mask is not None else None
        bs = None
        if bias is not None:
            bs = bias.to(x.dtype).expand(B1, 1, H, Q, K).contiguous()
        _lib.check(lib.ffb_softmax_fwd(_lib.ptr(xc), _lib.ptr(mk), _lib.ptr(bs), _lib.ptr(y), B1, B2, H, Q, K,
                                       _lib.dtype_code(x.dtype), _lib.stream_ptr()), "softmax_fwd")
        ctx.save_for_backward(y)
        ctx.has_bias = bias is not None
        ctx.bias_shape = tuple(bias.shape) if bias is not None else None
        ctx.squeeze = squeeze
        return y.squeeze(-2) if squeeze else y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib.get()
        (y,) = ctx.saved_tensors
        dyc = (dy.unsqueeze(-2) if ctx.squeeze else dy).contiguous()
        dx = torch.empty_like(y)
        K = y.shape[-1]
        _lib.check(lib.ffb_softmax_bwd(_lib.ptr(dyc), _lib.ptr(y), _lib.ptr(dx), y.numel() // K, K, _lib.dtype_code(y.dtype),
                                       _lib.stream_ptr()), "softmax_bwd")
        dbias = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            dbias = dx.sum(dim=1, keepdim=True)
            if tuple(dbias.shape) != ctx.bias_shape:
                dbias = dbias.sum_to_size(ctx.bias_shape)
        return (dx.squeeze(-2) if ctx.squeeze else dx), None, dbias


def fused_softmax(x, mask=None, bias=None):
    if not (x.is_cuda and x.dtype in _lib._DT and x.dim() in (4, 5)):
        v = x
        if bias is not None:
            v = v + bias
        if mask is not None:
            m = mask
            while m.dim() < v.dim():
                m = m.unsqueeze(-2)
            v = torch.where(m == 0, torch.full_like(v, -1e9), v)
        return torch.softmax(v, dim=-1)
    return _SoftmaxFn.apply(x, mask, bias)


# ---------------------------------------------------------------------------
# The reference's lower-level names (kernel/softmax.py:21-59, kernel/cuda_native/softmax.py:6-22,
# kernel/triton/softmax.py:153-215): its two back ends are one set of kernels here.
# ---------------------------------------------------------------------------
FusedSoftmaxFunc = _SoftmaxFn


def _softmax_forward_only(input_, mask_, bias_, rows=None, cols=None):
    """Masked, biased softmax without recording a graph; ``rows`` / ``cols`` are implied by the shape and only checked."""
    if cols is not None and cols != input_.shape[-1]:
        raise ValueError("cols = %d but the last dimension has %d entries" % (cols, input_.shape[-1]))
    if rows is not None and rows != input_.numel() // input_.shape[-1]:
        raise ValueError("rows = %d but the input has %d rows" % (rows, input_.numel() // input_.shape[-1]))
    with torch.no_grad():
        return fused_softmax(input_, mask_, bias_)


def _softmax_backward_only(grad_output, output, rows=None, cols=None):
    """``dx = y * (dy - sum(dy * y))`` over the last dimension (masked entries have y = 0, so their gradient is 0)."""
    K = output.shape[-1]
    if cols is not None and cols != K:
        raise ValueError("cols = %d but the last dimension has %d entries" % (cols, K))
    if rows is not None and rows != output.numel() // K:
        raise ValueError("rows = %d but the output has %d rows" % (rows, output.numel() // K))
    if output.is_cuda and output.dtype in _lib._DT:
        y, dy = output.contiguous(), grad_output.contiguous()
        dx = torch.empty_like(y)
        _lib.check(_lib.get().ffb_softmax_bwd(_lib.ptr(dy), _lib.ptr(y), _lib.ptr(dx), y.numel() // K, K, _lib.dtype_code(y.dtype),
                                              _lib.stream_ptr()), "softmax_bwd")
        return dx
    y, dy = output.float(), grad_output.float()
    return (y * (dy - (dy * y).sum(-1, keepdim=True))).to(output.dtype)


def softmax_cuda_kernel_wrapper(input_, mask_, bias_, rows, cols):
    return _softmax_forward_only(input_, mask_, bias_, rows, cols)


def softmax_grad_cuda_kernel_wrapper(grad_output, output, mask_, rows, cols):
    return _softmax_backward_only(grad_output, output, rows, cols)


def softmax_triton_kernel_wrapper(x, mask, bias, n_rows, n_cols):
    return _softmax_forward_only(x, mask, bias, n_rows, n_cols)


def softmax_grad_triton_kernel_wrapper(grad_output, output, n_rows, n_cols):
    return _softmax_backward_only(grad_output, output, n_rows, n_cols)
