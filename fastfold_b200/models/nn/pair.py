"""OpenFold-layout pair-stack modules: outer product mean, transitions, triangle attention and multiplication.

Cf. fastfold/model/nn/outer_product_mean.py, pair_transition.py, triangular_attention.py and
triangular_multiplicative_update.py.
"""
from functools import partialmethod

import torch
import torch.nn as nn

from ...utils.tensor_utils import chunk_layer, permute_final_dims
from .primitives import Attention, LayerNorm, Linear


class OuterProductMean(nn.Module):
    def __init__(self, c_m, c_z, c_hidden, eps=1e-3):
        super().__init__()
        self.c_m, self.c_z, self.c_hidden, self.eps = c_m, c_z, c_hidden, eps
        self.layer_norm = nn.LayerNorm(c_m)
        self.linear_1 = Linear(c_m, c_hidden)
        self.linear_2 = Linear(c_m, c_hidden)
        self.linear_out = Linear(c_hidden ** 2, c_z, init="final")

    def _opm(self, a, b):
        outer = torch.einsum("...bac,...dae->...bdce", a, b)
        outer = outer.reshape(outer.shape[:-2] + (-1,))
        return self.linear_out(outer)

    def forward(self, m, mask=None, chunk_size=None):
        if mask is None:
            mask = m.new_ones(m.shape[:-1])
        m = self.layer_norm(m)
        mask = mask.unsqueeze(-1)
        a = self.linear_1(m) * mask
        b = self.linear_2(m) * mask
        a = a.transpose(-2, -3)
        b = b.transpose(-2, -3)
        if chunk_size is not None:
            outs = [self._opm(a[..., s:s + chunk_size, :, :], b) for s in range(0, a.shape[-3], chunk_size)]
            outer = torch.cat(outs, dim=-3)
        else:
            outer = self._opm(a, b)
        norm = torch.einsum("...abc,...adc->...bdc", mask, mask)
        return outer / (self.eps + norm)


class _Transition(nn.Module):
    def __init__(self, c, n):
        super().__init__()
        self.c, self.n = c, n
        self.layer_norm = LayerNorm(c)
        self.linear_1 = Linear(c, n * c, init="relu")
        self.relu = nn.ReLU()
        self.linear_2 = Linear(n * c, c, init="final")

    def _transition(self, x, mask):
        return self.linear_2(self.relu(self.linear_1(x))) * mask

    def forward(self, x, mask=None, chunk_size=None):
        if mask is None:
            mask = x.new_ones(x.shape[:-1])
        mask = mask.unsqueeze(-1)
        x = self.layer_norm(x)
        if chunk_size is not None:
            return chunk_layer(self._transition, {"x": x, "mask": mask}, chunk_size=chunk_size, no_batch_dims=len(x.shape[:-2]))
        return self._transition(x=x, mask=mask)


class PairTransition(_Transition):
    def __init__(self, c_z, n):
        super().__init__(c_z, n)

    def forward(self, z, mask=None, chunk_size=None):
        return super().forward(z, mask, chunk_size)


class MSATransition(_Transition):
    def __init__(self, c_m, n):
        super().__init__(c_m, n)

    def forward(self, m, mask=None, chunk_size=None):
        return super().forward(m, mask, chunk_size)


class TriangleAttention(nn.Module):
    def __init__(self, c_in, c_hidden, no_heads, starting, inf=1e9):
        super().__init__()
        self.c_in, self.c_hidden, self.no_heads, self.starting, self.inf = c_in, c_hidden, no_heads, starting, inf
        self.layer_norm = LayerNorm(c_in)
        self.linear = Linear(c_in, no_heads, bias=False, init="normal")
        self.mha = Attention(c_in, c_in, c_in, c_hidden, no_heads)

    def forward(self, x, mask=None, chunk_size=None):
        if mask is None:
            mask = x.new_ones(x.shape[:-1])
        if not self.starting:
            x = x.transpose(-2, -3)
            mask = mask.transpose(-1, -2)
        x = self.layer_norm(x)
        mask_bias = (self.inf * (mask - 1))[..., :, None, None, :]
        triangle_bias = permute_final_dims(self.linear(x), (2, 0, 1)).unsqueeze(-4)
        biases = [mask_bias, triangle_bias]
        if chunk_size is not None:
            x = chunk_layer(self.mha, {"q_x": x, "kv_x": x, "biases": biases}, chunk_size=chunk_size, no_batch_dims=len(x.shape[:-2]))
        else:
            x = self.mha(q_x=x, kv_x=x, biases=biases)
        if not self.starting:
            x = x.transpose(-2, -3)
        return x


class TriangleAttentionStartingNode(TriangleAttention):
    __init__ = partialmethod(TriangleAttention.__init__, starting=True)


class TriangleAttentionEndingNode(TriangleAttention):
    __init__ = partialmethod(TriangleAttention.__init__, starting=False)


_FUSED_TRI_MUL = False


def set_fused_triangle_multiplication(value=True):
    """Selects the fused-projection parameter layout (``linear_p`` / ``linear_g`` / ``linear_gate``) used by
    multimer v3 weights for modules constructed afterwards."""
    global _FUSED_TRI_MUL
    _FUSED_TRI_MUL = bool(value)


def is_fused_triangle_multiplication():
    return _FUSED_TRI_MUL


class TriangleMultiplicativeUpdate(nn.Module):
    def __init__(self, c_z, c_hidden, _outgoing=True):
        super().__init__()
        self.c_z, self.c_hidden, self._outgoing = c_z, c_hidden, _outgoing
        self.fused = _FUSED_TRI_MUL
        if self.fused:
            self.linear_p = Linear(c_z, 2 * c_hidden)
            self.linear_g = Linear(c_z, 2 * c_hidden, init="gating")
            self.linear_gate = Linear(c_z, c_z, init="gating")
        else:
            self.linear_a_p = Linear(c_z, c_hidden)
            self.linear_a_g = Linear(c_z, c_hidden, init="gating")
            self.linear_b_p = Linear(c_z, c_hidden)
            self.linear_b_g = Linear(c_z, c_hidden, init="gating")
            self.linear_g = Linear(c_z, c_z, init="gating")
        self.linear_z = Linear(c_hidden, c_z, init="final")
        self.layer_norm_in = LayerNorm(c_z)
        self.layer_norm_out = LayerNorm(c_hidden)
        self.sigmoid = nn.Sigmoid()

    def _combine(self, a, b):
        if self._outgoing:
            p = torch.matmul(permute_final_dims(a, (2, 0, 1)), permute_final_dims(b, (2, 1, 0)))
        else:
            p = torch.matmul(permute_final_dims(a, (2, 1, 0)), permute_final_dims(b, (2, 0, 1)))
        return permute_final_dims(p, (1, 2, 0))

    def forward(self, z, mask=None):
        if mask is None:
            mask = z.new_ones(z.shape[:-1])
        mask = mask.unsqueeze(-1)
        z = self.layer_norm_in(z)
        if self.fused:
            ab = self.linear_p(z) * mask * self.sigmoid(self.linear_g(z))
            a, b = ab.chunk(2, dim=-1)
            g = self.sigmoid(self.linear_gate(z))
        else:
            a = self.linear_a_p(z) * mask * self.sigmoid(self.linear_a_g(z))
            b = self.linear_b_p(z) * mask * self.sigmoid(self.linear_b_g(z))
            g = self.sigmoid(self.linear_g(z))
        x = self._combine(a, b)
        x = self.linear_z(self.layer_norm_out(x))
        return x * g


class TriangleMultiplicationOutgoing(TriangleMultiplicativeUpdate):
    __init__ = partialmethod(TriangleMultiplicativeUpdate.__init__, _outgoing=True)


class TriangleMultiplicationIncoming(TriangleMultiplicativeUpdate):
    __init__ = partialmethod(TriangleMultiplicativeUpdate.__init__, _outgoing=False)
