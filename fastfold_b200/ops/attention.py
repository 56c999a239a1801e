"""Attention core: ``softmax(scale * q k^T + bias, masked) v`` for the Evoformer's axial attentions.

``q, k, v`` are ``[b1, b2, H, n, d]``; ``mask`` is ``[b1, b2, n_k]`` with zeros at
masked keys; ``bias`` is ``[b1, 1, H, n_q, n_k]`` (the pair bias, shared by all
``b2`` rows).  ``attention_core`` returns ``[b1, b2, H, n, d]`` and is the one every
attention module calls; ``fused_attention_core`` wraps it in the reference's
contract (fastfold/model/fastnn/kernel/attention_core.py:34-53, forward-only
there and not wired into its model).
"""
import torch

from . import _lib
from .softmax import fused_softmax


def attention_core_ref(q, k, v, mask=None, bias=None, scale=None):
    d = q.shape[-1]
    scale = d ** -0.5 if scale is None else scale
    logits = torch.matmul(q.float() * scale, k.float().transpose(-1, -2))
    if bias is not None:
        logits = logits + bias.float()
    if mask is not None:
        logits = torch.where(mask[..., None, None, :] == 0, torch.full_like(logits, -1e9), logits)
    return torch.matmul(torch.softmax(logits, -1), v.float()).to(q.dtype)


def _composite(q, k, v, mask, bias, scale):
    logits = torch.matmul(q * scale, k.transpose(-1, -2))
    w = fused_softmax(logits, mask, bias)
    return torch.matmul(w, v)


def attention_core(q, k, v, mask=None, bias=None, scale=None, chunk=None):
    """Returns ``[b1, b2, H, n_q, d]``.  ``chunk`` bounds the number of ``b2`` rows processed at once."""
    d = q.shape[-1]
    scale = d ** -0.5 if scale is None else scale
    from . import flash
    if flash.supported(q, k, v, mask, bias):
        return flash.flash_attention(q, k, v, mask, bias, scale)
    B2 = q.shape[1]
    if chunk is None or chunk >= B2:
        return _composite(q, k, v, mask, bias, scale)
    outs = []
    for s in range(0, B2, chunk):
        e = min(B2, s + chunk)
        outs.append(_composite(q[:, s:e], k[:, s:e], v[:, s:e], None if mask is None else mask[:, s:e], bias, scale))
    return torch.cat(outs, dim=1)


def fused_attention_core(q, k, v, mask=None, bias=None):
    """The reference's call (fastfold/model/fastnn/kernel/attention_core.py:17-53): ``q`` un-scaled (the op applies
    ``1 / sqrt(d)``), result with the heads merged, ``[b1, b2, n, H * d]``.  Differentiable here."""
    o = attention_core(q, k, v, mask, bias)
    return o.transpose(-2, -3).reshape(*o.shape[:-3], o.shape[-2], o.shape[-3] * o.shape[-1])


class FusedAttenionCoreFunc:
    """Call-compatible stand-in for the reference's autograd Function of this (mis-spelt) name: ``.apply(q, k, v, mask, bias)``."""
    apply = staticmethod(fused_attention_core)


def attention_core_triton_kernel_wrapper(q, k, v, mask, bias):
    """Forward only, as the reference's Triton launcher (kernel/triton/attention_core.py:124-190): no graph is recorded."""
    with torch.no_grad():
        return fused_attention_core(q, k, v, mask, bias)
