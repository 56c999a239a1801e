"""Autograd wrappers of the fused communication kernels.

``a2a_layer_norm`` is the axis switch of a sharded activation (row-sharded <-> column-sharded) fused with the
LayerNorm - and, where the consumer wants it, the transpose - that follows it: the kernel reads each row once
from the owning peer over NVLink and writes the raw row (the residual stream) and the normalised row locally;
the re-sharded tensor never makes a separate trip through memory.  In the reference this is
``row_to_col`` / ``col_to_row`` (``dist.all_to_all`` + ``torch.cat``) followed by ``transpose`` and a LayerNorm
kernel (fastfold/model/fastnn/msa.py:145,91-92; triangle.py:245-250; ops.py:890-894).

Falls back to the unfused composition when there is no symmetric heap (one rank, CPU, NCCL baseline).
"""
import torch

from ..ops import layer_norm as _ln
from ..ops.layer_norm import _LayerNormFn
from . import comm, core


def _heap(x):
    if not (x.is_cuda and x.dtype == torch.bfloat16):
        return None
    from . import symm
    return symm.get_heap("dap")


class _A2ALayerNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gamma, beta, eps, mode, transpose_norm):
        h = _heap(x)
        P = h.world
        if mode == 0:                       # x [A/P, B, C] -> [A, B/P, C]
            A, B, C = x.shape[0] * P, x.shape[1], x.shape[2]
        else:                               # x [A, B/P, C] -> [A/P, B, C]
            A, B, C = x.shape[0], x.shape[1] * P, x.shape[2]
        raw, norm = h.a2a_layer_norm(None, x, mode, A, B, C, gamma.contiguous(), beta.contiguous(), eps, True, transpose_norm)
        ctx.save_for_backward(raw, gamma, beta)
        ctx.cfg = (eps, mode, transpose_norm)
        return raw, norm

    @staticmethod
    def backward(ctx, d_raw, d_norm):
        raw, gamma, beta = ctx.saved_tensors
        eps, mode, transpose_norm = ctx.cfg
        dx = d_raw
        dg = db = None
        if d_norm is not None:
            if transpose_norm:
                d_norm = d_norm.transpose(0, 1)
            with torch.enable_grad():
                r = raw.detach().requires_grad_(True)
                g = gamma.detach().requires_grad_(True)
                b = beta.detach().requires_grad_(True)
                y = _ln(r, g, b, eps)
            gr, dg, db = torch.autograd.grad(y, (r, g, b), d_norm.contiguous())
            dx = gr if dx is None else dx + gr
        # gradient of the axis switch is the opposite axis switch
        dx = dx.unsqueeze(0)
        dx = comm._all_to_all(dx.contiguous(), 1, 2) if mode == 0 else comm._all_to_all(dx.contiguous(), 2, 1)
        return dx.squeeze(0), dg, db, None, None, None


def a2a_layer_norm(x, ln, mode, transpose_norm=False):
    """``x`` is ``[1, a, b, C]``; returns ``(raw, norm)`` as ``[1, ., ., C]`` tensors in the switched sharding.

    mode 0: row-sharded -> column-sharded (``row_to_col``); mode 1: column-sharded -> row-sharded (``col_to_row``).
    ``norm`` is ``LayerNorm(raw)``; with ``transpose_norm`` it is laid out ``[1, b, a, C]``.
    """
    P = core.get_dap_size()
    h = _heap(x) if P > 1 else None
    if h is not None and x.numel() * x.element_size() > h.max_message():
        h = None
    if h is None or x.shape[-1] % 8 or ln.weight.dtype != x.dtype:
        raw = comm.row_to_col(x) if mode == 0 else comm.col_to_row(x)
        src = raw.transpose(-2, -3).contiguous() if transpose_norm else raw
        return raw, ln(src)
    x3 = x.squeeze(0)
    if torch.is_grad_enabled() and (x.requires_grad or ln.weight.requires_grad):
        raw, norm = _A2ALayerNorm.apply(x3, ln.weight, ln.bias, ln.eps, mode, transpose_norm)
    else:
        raw, norm = _A2ALayerNorm.forward(_NoCtx(), x3, ln.weight, ln.bias, ln.eps, mode, transpose_norm)
    return raw.unsqueeze(0), norm.unsqueeze(0)


class _NoCtx:
    def save_for_backward(self, *a):
        pass
