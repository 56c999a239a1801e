"""LayerNorm over the last dimension (csrc/layernorm.cu), forward and backward.

``LayerNorm`` keeps the constructor and parameter names of the reference's
``fastfold.model.fastnn.kernel.LayerNorm`` (kernel/layer_norm.py:19-60):
``LayerNorm(normalized_shape, eps=1e-5)`` with ``weight`` / ``bias``.  The
reference splits inputs whose third-last dimension exceeds 4000 into chunks
(:37-50) to bound its workspace; this kernel needs no workspace proportional
to the input, so no chunking is necessary.
"""
import numbers

import torch
from torch import nn

from . import _lib


def layer_norm_ref(x, weight, bias, eps):
    return torch.nn.functional.layer_norm(x.float(), (x.shape[-1],), weight.float(), bias.float(), eps).to(x.dtype)


def _native_ok(x, weight):
    return x.is_cuda and x.dtype in _lib._DT and weight.dtype == x.dtype


class _LayerNormFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps):
        lib = _lib.get()
        xc = x.contiguous()
        C = xc.shape[-1]
        rows = xc.numel() // C
        y = torch.empty_like(xc)
        need_stats = torch.is_grad_enabled() or ctx.needs_input_grad[0] or ctx.needs_input_grad[1]
        mean = torch.empty(rows, device=x.device, dtype=torch.float32)
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        w = weight.contiguous()
        b = bias.contiguous()
        _lib.check(lib.ffb_layernorm_fwd(_lib.ptr(xc), _lib.ptr(w), _lib.ptr(b), _lib.ptr(y), _lib.ptr(mean), _lib.ptr(rstd),
                                         rows, C, float(eps), _lib.dtype_code(x.dtype), _lib.stream_ptr()), "layernorm_fwd")
        ctx.save_for_backward(xc, w, mean, rstd)
        ctx.params = (weight, bias)
        del need_stats
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib.get()
        xc, w, mean, rstd = ctx.saved_tensors
        dyc = dy.contiguous()
        C = xc.shape[-1]
        rows = xc.numel() // C
        dx = torch.empty_like(xc)
        nblocks = int(min(1184, max(1, (rows + 3) // 4)))   # 8 blocks per SM: enough warps in flight to hide the per-row reductions
        part = torch.empty(nblocks * 2 * C, device=xc.device, dtype=torch.float32)
        from .gemm import grad_sink
        sg, sb = grad_sink(ctx.params[0]), grad_sink(ctx.params[1])
        if sg is not None and sb is not None and xc.dtype == torch.bfloat16 and _lib.has("ffb_layernorm_bwd_acc"):
            # gamma / beta gradients go straight into the trainer's fp32 buffer
            _lib.check(lib.ffb_layernorm_bwd_acc(_lib.ptr(dyc), _lib.ptr(xc), _lib.ptr(w), _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(dx),
                                                 _lib.ptr(part), nblocks, _lib.ptr(sg), _lib.ptr(sb), rows, C, _lib.stream_ptr()),
                       "layernorm_bwd_acc")
            return dx, None, None, None
        dg = torch.empty_like(w)
        db = torch.empty_like(w)
        _lib.check(lib.ffb_layernorm_bwd(_lib.ptr(dyc), _lib.ptr(xc), _lib.ptr(w), _lib.ptr(mean), _lib.ptr(rstd), _lib.ptr(dx),
                                         _lib.ptr(part), nblocks, _lib.ptr(dg), _lib.ptr(db), rows, C,
                                         _lib.dtype_code(xc.dtype), _lib.stream_ptr()), "layernorm_bwd")
        return dx, dg, db, None


def layer_norm(x, weight, bias, eps=1e-5):
    if not _native_ok(x, weight):
        return torch.nn.functional.layer_norm(x, (x.shape[-1],), weight.to(x.dtype), bias.to(x.dtype), eps)
    return _LayerNormFn.apply(x, weight, bias, eps)


def _ln_t_supported(x_cm):
    return x_cm.is_cuda and x_cm.dtype == torch.bfloat16 and x_cm.shape[0] <= 256


def _ln_t_forward(x_cm, weight, bias, eps, want_stats):
    lib = _lib.get()
    C, rows = x_cm.shape
    x_cm = x_cm.contiguous()
    y = torch.empty(rows, C, device=x_cm.device, dtype=x_cm.dtype)
    mean = torch.empty(rows, device=x_cm.device, dtype=torch.float32) if want_stats else None
    rstd = torch.empty(rows, device=x_cm.device, dtype=torch.float32) if want_stats else None
    _lib.check(lib.ffb_layernorm_fwd_transposed(_lib.ptr(x_cm), _lib.ptr(weight.contiguous()), _lib.ptr(bias.contiguous()),
                                                _lib.ptr(y), _lib.ptr(mean), _lib.ptr(rstd), rows, C, float(eps), _lib.stream_ptr()),
               "layernorm_fwd_transposed")
    return y, x_cm, mean, rstd


class _LayerNormTFn(torch.autograd.Function):
    """LayerNorm over dim 0 of a channel-major tensor; the input gradient comes back channel-major as well."""

    @staticmethod
    def forward(ctx, x_cm, weight, bias, eps):
        y, x_c, mean, rstd = _ln_t_forward(x_cm, weight, bias, eps, True)
        ctx.save_for_backward(x_c, weight, mean, rstd)
        ctx.params = (weight, bias)
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _lib.get()
        x_cm, weight, mean, rstd = ctx.saved_tensors
        C, rows = x_cm.shape
        dy = dy.contiguous()
        dx = torch.empty_like(x_cm)
        part = torch.empty(((rows + 31) // 32) * 2 * C, device=dy.device, dtype=torch.float32)
        from .gemm import grad_sink
        sg, sb = grad_sink(ctx.params[0]), grad_sink(ctx.params[1])
        if sg is not None and sb is not None and weight.is_contiguous() and _lib.has("ffb_layernorm_bwd_transposed_acc"):
            # gamma / beta gradients go straight into the trainer's fp32 buffer
            _lib.check(lib.ffb_layernorm_bwd_transposed_acc(_lib.ptr(dy), _lib.ptr(x_cm), _lib.ptr(weight), _lib.ptr(mean), _lib.ptr(rstd),
                                                            _lib.ptr(dx), _lib.ptr(part), _lib.ptr(sg), _lib.ptr(sb), rows, C, _lib.stream_ptr()),
                       "layernorm_bwd_transposed_acc")
            return dx, None, None, None
        dg = torch.empty(C, device=dy.device, dtype=torch.float32)
        db = torch.empty(C, device=dy.device, dtype=torch.float32)
        _lib.check(lib.ffb_layernorm_bwd_transposed(_lib.ptr(dy), _lib.ptr(x_cm), _lib.ptr(weight.contiguous()), _lib.ptr(mean), _lib.ptr(rstd),
                                                    _lib.ptr(dx), _lib.ptr(part), _lib.ptr(dg), _lib.ptr(db), rows, C, _lib.stream_ptr()),
                   "layernorm_bwd_transposed")
        return dx, dg.to(weight.dtype), db.to(weight.dtype), None


def layer_norm_transposed(x_cm, weight, bias, eps=1e-5):
    """LayerNorm over dim 0 of ``x_cm [C, rows]`` returning ``[rows, C]``; differentiable (the gradient of ``x_cm`` is
    produced channel-major by its own kernel)."""
    if not _ln_t_supported(x_cm):
        return layer_norm(x_cm.t().contiguous(), weight, bias, eps)
    if torch.is_grad_enabled() and (x_cm.requires_grad or weight.requires_grad or bias.requires_grad):
        if _lib.has("ffb_layernorm_bwd_transposed"):
            return _LayerNormTFn.apply(x_cm, weight, bias, eps)
        return layer_norm(x_cm.t().contiguous(), weight, bias, eps)
    return _ln_t_forward(x_cm, weight, bias, eps, False)[0]


class LayerNorm(nn.Module):
    def __init__(self, normalized_shape, eps=1e-5):
        super().__init__()
        if isinstance(normalized_shape, numbers.Integral):
            normalized_shape = (normalized_shape,)
        self.normalized_shape = torch.Size(normalized_shape)
        assert len(self.normalized_shape) == 1, "LayerNorm normalises the last dimension"
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(*normalized_shape))
        self.bias = nn.Parameter(torch.zeros(*normalized_shape))

    def reset_parameters(self):
        nn.init.ones_(self.weight)
        nn.init.zeros_(self.bias)

    def forward(self, x):
        return layer_norm(x, self.weight, self.bias, self.eps)

    kernel_forward = forward       # the reference's forward chunks long inputs and calls this per chunk (kernel/layer_norm.py:36-60)

    def extra_repr(self):
        return "%s, eps=%g" % (tuple(self.normalized_shape), self.eps)


FusedLayerNorm = LayerNorm


class FusedLayerNormAffineFunction:
    """Call-compatible stand-in for the reference's CUDA-extension Function (kernel/cuda_native/layer_norm.py:8-38):
    ``.apply(input, weight, bias, normalized_shape, eps)``; differentiable in input, weight and bias."""

    @staticmethod
    def apply(input, weight, bias, normalized_shape, eps):
        assert tuple(normalized_shape) == (input.shape[-1],), "LayerNorm normalises the last dimension"
        return layer_norm(input, weight, bias, eps)


class LayerNormTritonFunc:
    """Call-compatible stand-in for the reference's Triton Function (kernel/triton/layer_norm.py:146-212), whose
    argument order differs: ``.apply(a_raw, normalized_shape, weight, bias, eps)``."""

    @staticmethod
    def apply(a_raw, normalized_shape, weight, bias, eps):
        return FusedLayerNormAffineFunction.apply(a_raw, weight, bias, normalized_shape, eps)
