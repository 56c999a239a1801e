"""Dispatch to the fused tcgen05 attention kernel (csrc/attention_tcgen05.cu) when it is built and the shape fits."""
import torch

from . import _lib


def supported(q, k, v, mask, bias):
    return False


def flash_attention(q, k, v, mask, bias, scale):
    raise NotImplementedError
