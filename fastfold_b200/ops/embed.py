"""Fused pair update of the recycling embedder: ``LayerNorm(z_prev) + Linear(one_hot(distance bin))`` as a gather-add.

Kernel: csrc/embed.cu (inference, bf16 pair representation of 128 channels, fp32 coordinates); everything else goes
through ``recycle_pair_embed_ref``, the composite the reference uses (fastfold/model/fastnn/embedders.py:100-137).
"""
import torch

from . import _lib


def recycle_pair_embed_ref(z, x, sq_bins, inf, weight, bias, ln_weight, ln_bias, eps):
    upper = torch.cat([sq_bins[1:], sq_bins.new_tensor([inf])], dim=-1)
    d = torch.sum((x[..., :, None, :] - x[..., None, :, :]) ** 2, dim=-1, keepdims=True)
    one_hot = ((d > sq_bins) * (d < upper)).type(z.dtype)
    ln = torch.nn.functional.layer_norm(z, (z.shape[-1],), ln_weight, ln_bias, eps)
    return torch.nn.functional.linear(one_hot, weight, bias) + ln


def recycle_pair_embed_supported(z, x):
    return (z.is_cuda and z.dtype == torch.bfloat16 and x.dtype == torch.float32 and z.shape[-1] == 128 and not torch.is_grad_enabled()
            and z.numel() == z.shape[-2] * z.shape[-3] * 128 and x.numel() == z.shape[-2] * 3 and z.shape[-2] == z.shape[-3]
            and _lib.has("ffb_recycle_pair_embed"))


def recycle_pair_embed(z, x, sq_bins, inf, weight, bias, ln_weight, ln_bias, eps, out=None):
    """``z [.., N, N, 128]`` (previous pair representation), ``x [.., N, 3]`` (previous pseudo-beta positions),
    ``sq_bins [no_bins]`` squared lower bin edges -> ``LayerNorm(z) + weight[:, bin] + bias``; ``out`` may alias ``z``."""
    if not recycle_pair_embed_supported(z, x) or sq_bins.numel() > 64:
        r = recycle_pair_embed_ref(z, x, sq_bins, inf, weight, bias, ln_weight, ln_bias, eps)
        if out is not None:
            out.copy_(r)
            return out
        return r
    N = z.shape[-2]
    zc = z.contiguous()
    out = torch.empty_like(zc) if out is None else out
    assert out.is_contiguous() and out.shape == zc.shape and out.dtype == zc.dtype
    dt = zc.dtype
    _lib.check(_lib.get().ffb_recycle_pair_embed(
        _lib.ptr(zc), _lib.ptr(x.contiguous()), _lib.ptr(sq_bins.float().contiguous()), _lib.ptr(weight.to(dt).contiguous()),
        _lib.ptr(bias.to(dt).contiguous()), _lib.ptr(ln_weight.to(dt).contiguous()), _lib.ptr(ln_bias.to(dt).contiguous()), _lib.ptr(out),
        N, 0, N, 128, sq_bins.numel(), float(eps), float(inf), _lib.stream_ptr()), "recycle_pair_embed")
    return out
