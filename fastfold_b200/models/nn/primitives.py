"""OpenFold-layout primitives: Linear with AlphaFold initialisers, LayerNorm, gated attention, global attention.

These pure-PyTorch modules define the ``state_dict`` layout that checkpoints and
``import_jax_weights_`` target (``linear_q/k/v/o/g`` ...), run on CPU in fp32,
and are the numerical oracle for the fast modules and the CUDA kernels.  Same
roles as fastfold/model/nn/primitives.py (Linear :102-167, Attention :291-419,
GlobalAttention :422-503, low-memory attention :506-565).
"""
import math
from typing import List, Optional, Tuple

import torch
import torch.nn as nn

from ...utils.tensor_utils import flatten_final_dims, permute_final_dims


def _prod(nums):
    out = 1
    for n in nums:
        out *= n
    return out


def _calculate_fan(shape, fan="fan_in"):
    fan_out, fan_in = shape
    if fan == "fan_in":
        return fan_in
    if fan == "fan_out":
        return fan_out
    if fan == "fan_avg":
        return (fan_in + fan_out) / 2
    raise ValueError("Invalid fan option")


def trunc_normal_init_(weights, scale=1.0, fan="fan_in"):
    f = _calculate_fan(weights.shape, fan)
    scale = scale / max(1, f)
    # std of a unit normal truncated to [-2, 2]
    std = math.sqrt(scale) / 0.87962566103423978
    with torch.no_grad():
        nn.init.trunc_normal_(weights, mean=0.0, std=std, a=-2.0 * std, b=2.0 * std)


def lecun_normal_init_(weights):
    trunc_normal_init_(weights, scale=1.0)


def he_normal_init_(weights):
    trunc_normal_init_(weights, scale=2.0)


def glorot_uniform_init_(weights):
    nn.init.xavier_uniform_(weights, gain=1)


def final_init_(weights):
    with torch.no_grad():
        weights.fill_(0.0)


def gating_init_(weights):
    with torch.no_grad():
        weights.fill_(0.0)


def normal_init_(weights):
    nn.init.kaiming_normal_(weights, nonlinearity="linear")


def ipa_point_weights_init_(weights):
    with torch.no_grad():
        weights.fill_(0.541324854612918)   # softplus^-1(1)


class Linear(nn.Linear):
    def __init__(self, in_dim, out_dim, bias=True, init="default", init_fn=None):
        super().__init__(in_dim, out_dim, bias=bias)
        if bias:
            with torch.no_grad():
                self.bias.fill_(0)
        if init_fn is not None:
            init_fn(self.weight, self.bias)
        elif init == "default":
            lecun_normal_init_(self.weight)
        elif init == "relu":
            he_normal_init_(self.weight)
        elif init == "glorot":
            glorot_uniform_init_(self.weight)
        elif init == "gating":
            gating_init_(self.weight)
            if bias:
                with torch.no_grad():
                    self.bias.fill_(1.0)
        elif init == "normal":
            normal_init_(self.weight)
        elif init == "final":
            final_init_(self.weight)
        else:
            raise ValueError("Invalid init string.")


class LayerNorm(nn.Module):
    def __init__(self, c_in, eps=1e-5):
        super().__init__()
        self.c_in = (c_in,)
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(c_in))
        self.bias = nn.Parameter(torch.zeros(c_in))

    def forward(self, x):
        return nn.functional.layer_norm(x, self.c_in, self.weight, self.bias, self.eps)


def softmax(t, dim=-1):
    return torch.nn.functional.softmax(t, dim=dim)


def _attention(query, key, value, biases):
    a = torch.matmul(query, permute_final_dims(key, (1, 0)))
    for b in biases:
        a = a + b
    a = softmax(a, -1)
    return torch.matmul(a, value)


def _lma(q, k, v, biases, q_chunk_size, kv_chunk_size):
    """Memory-efficient attention: online softmax over key/value chunks (Rabe & Staats)."""
    no_q, no_kv = q.shape[-3], k.shape[-3]
    o = q.new_zeros(q.shape)
    for q_s in range(0, no_q, q_chunk_size):
        q_chunk = q[..., q_s:q_s + q_chunk_size, :, :]
        large_bias_chunks = [b[..., q_s:q_s + q_chunk_size, :] for b in biases]
        maxes, weights, values = [], [], []
        for kv_s in range(0, no_kv, kv_chunk_size):
            k_chunk = k[..., kv_s:kv_s + kv_chunk_size, :, :]
            v_chunk = v[..., kv_s:kv_s + kv_chunk_size, :, :]
            small = [b[..., kv_s:kv_s + kv_chunk_size] for b in large_bias_chunks]
            a = torch.einsum("...qhd,...khd->...hqk", q_chunk, k_chunk)
            for b in small:
                a = a + b
            a = a.transpose(-2, -3)
            max_a = torch.max(a, dim=-1, keepdim=True)[0]
            exp_a = torch.exp(a - max_a)
            exp_v = torch.einsum("...vhf,...qhv->...qhf", v_chunk, exp_a)
            maxes.append(max_a.detach().squeeze(-1))
            weights.append(torch.sum(exp_a, dim=-1))
            values.append(exp_v)
        chunk_max = torch.stack(maxes, dim=-3)
        chunk_weights = torch.stack(weights, dim=-3)
        chunk_values = torch.stack(values, dim=-4)
        global_max = torch.max(chunk_max, dim=-3, keepdim=True)[0]
        max_diffs = torch.exp(chunk_max - global_max)
        chunk_values = chunk_values * max_diffs.unsqueeze(-1)
        chunk_weights = chunk_weights * max_diffs
        all_values = torch.sum(chunk_values, dim=-4)
        all_weights = torch.sum(chunk_weights.unsqueeze(-1), dim=-4)
        o[..., q_s:q_s + q_chunk_size, :, :] = all_values / all_weights
    return o


class Attention(nn.Module):
    """Standard multi-head attention with optional sigmoid gate: ``[*, Q, C_q] x [*, K, C_k] -> [*, Q, C_q]``."""

    def __init__(self, c_q, c_k, c_v, c_hidden, no_heads, gating=True):
        super().__init__()
        self.c_q, self.c_k, self.c_v, self.c_hidden, self.no_heads, self.gating = c_q, c_k, c_v, c_hidden, no_heads, gating
        self.linear_q = Linear(c_q, c_hidden * no_heads, bias=False, init="glorot")
        self.linear_k = Linear(c_k, c_hidden * no_heads, bias=False, init="glorot")
        self.linear_v = Linear(c_v, c_hidden * no_heads, bias=False, init="glorot")
        self.linear_o = Linear(c_hidden * no_heads, c_q, init="final")
        self.linear_g = Linear(c_q, c_hidden * no_heads, init="gating") if gating else None
        self.sigmoid = nn.Sigmoid()

    def _prep_qkv(self, q_x, kv_x):
        q, k, v = self.linear_q(q_x), self.linear_k(kv_x), self.linear_v(kv_x)
        q = q.view(q.shape[:-1] + (self.no_heads, -1)).transpose(-2, -3)
        k = k.view(k.shape[:-1] + (self.no_heads, -1)).transpose(-2, -3)
        v = v.view(v.shape[:-1] + (self.no_heads, -1)).transpose(-2, -3)
        q = q / math.sqrt(self.c_hidden)
        return q, k, v

    def _wrap_up(self, o, q_x):
        if self.linear_g is not None:
            g = self.sigmoid(self.linear_g(q_x))
            g = g.view(g.shape[:-1] + (self.no_heads, -1))
            o = o * g
        return self.linear_o(flatten_final_dims(o, 2))

    def forward(self, q_x, kv_x, biases=None, use_lma=False, q_chunk_size=None, kv_chunk_size=None):
        biases = [] if biases is None else biases
        q, k, v = self._prep_qkv(q_x, kv_x)
        if use_lma:
            biases = [b.expand(b.shape[:-2] + (q_x.shape[-2],) + (kv_x.shape[-2],)) for b in biases]
            o = _lma(q.transpose(-2, -3), k.transpose(-2, -3), v.transpose(-2, -3), biases, q_chunk_size, kv_chunk_size)
        else:
            o = _attention(q, k, v, biases).transpose(-2, -3)
        return self._wrap_up(o, q_x)


class GlobalAttention(nn.Module):
    def __init__(self, c_in, c_hidden, no_heads, inf, eps):
        super().__init__()
        self.c_in, self.c_hidden, self.no_heads, self.inf, self.eps = c_in, c_hidden, no_heads, inf, eps
        self.linear_q = Linear(c_in, c_hidden * no_heads, bias=False, init="glorot")
        self.linear_k = Linear(c_in, c_hidden, bias=False, init="glorot")
        self.linear_v = Linear(c_in, c_hidden, bias=False, init="glorot")
        self.linear_g = Linear(c_in, c_hidden * no_heads, init="gating")
        self.linear_o = Linear(c_hidden * no_heads, c_in, init="final")
        self.sigmoid = nn.Sigmoid()

    def forward(self, m, mask):
        q = torch.sum(m * mask.unsqueeze(-1), dim=-2) / (torch.sum(mask, dim=-1)[..., None] + self.eps)
        q = self.linear_q(q) * (self.c_hidden ** (-0.5))
        q = q.view(q.shape[:-1] + (self.no_heads, -1))
        k, v = self.linear_k(m), self.linear_v(m)
        a = torch.matmul(q, k.transpose(-1, -2))
        bias = (self.inf * (mask - 1))[..., :, None, :]
        a = softmax(a + bias)
        o = torch.matmul(a, v)
        g = self.sigmoid(self.linear_g(m))
        g = g.view(g.shape[:-1] + (self.no_heads, -1))
        o = o.unsqueeze(-3) * g
        o = o.reshape(o.shape[:-2] + (-1,))
        return self.linear_o(o)
