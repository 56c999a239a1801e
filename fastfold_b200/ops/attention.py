"""Attention core: ``softmax(scale * q k^T + bias, masked) v`` for the Evoformer's axial attentions.

``q, k, v`` are ``[b1, b2, H, n, d]``; ``mask`` is ``[b1, b2, n_k]`` with zeros at
masked keys; ``bias`` is ``[b1, 1, H, n_q, n_k]`` (the pair bias, shared by all
``b2`` rows).  Same contract as the reference's ``fused_attention_core``
(fastfold/model/fastnn/kernel/attention_core.py:34-53), which is forward-only
and not wired into its model; here the op has a backward and is the one every
attention module calls.
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


def fused_attention_core(q, k, v, mask, bias):
    """Reference-compatible call: ``q`` is expected pre-scaled (as the reference's modules do)."""
    return attention_core(q, k, v, mask, bias, scale=1.0)
