"""OpenFold-layout MSA attention modules (Algorithms 7, 8, 19); cf. fastfold/model/nn/msa.py."""
import torch
import torch.nn as nn

from ...utils.tensor_utils import chunk_layer, permute_final_dims
from .primitives import Attention, GlobalAttention, LayerNorm, Linear


class MSAAttention(nn.Module):
    def __init__(self, c_in, c_hidden, no_heads, pair_bias=False, c_z=None, inf=1e9):
        super().__init__()
        self.c_in, self.c_hidden, self.no_heads, self.pair_bias, self.c_z, self.inf = c_in, c_hidden, no_heads, pair_bias, c_z, inf
        self.layer_norm_m = LayerNorm(c_in)
        self.layer_norm_z = None
        self.linear_z = None
        if pair_bias:
            self.layer_norm_z = LayerNorm(c_z)
            self.linear_z = Linear(c_z, no_heads, bias=False, init="normal")
        self.mha = Attention(c_in, c_in, c_in, c_hidden, no_heads)

    def _chunk(self, m, biases, chunk_size):
        return chunk_layer(self.mha, {"q_x": m, "kv_x": m, "biases": biases}, chunk_size=chunk_size, no_batch_dims=len(m.shape[:-2]))

    def _prep_inputs(self, m, z, mask):
        m = self.layer_norm_m(m)
        n_seq, n_res = m.shape[-3:-1]
        if mask is None:
            mask = m.new_ones(m.shape[:-3] + (n_seq, n_res))
        mask_bias = (self.inf * (mask - 1))[..., :, None, None, :]
        if self.pair_bias and z is not None and self.layer_norm_z is not None:
            z = self.linear_z(self.layer_norm_z(z))
            z = permute_final_dims(z, (2, 0, 1)).unsqueeze(-4)
        return m, mask_bias, z

    def _chunked_rows(self, m, z, mask, rows_per_chunk, checkpoint):
        """Rows of the alignment attend independently: evaluate ``rows_per_chunk`` of them at a time, so that only their
        logits ``[rows, H, N, N]`` exist at once, each piece under activation checkpointing when ``checkpoint`` is set -
        the memory bound that makes the extra-MSA stack (thousands of rows) trainable
        (fastfold/model/nn/msa.py:117-161)."""
        m, mask_bias, z = self._prep_inputs(m, z, mask)

        def piece(m_c, mask_c, z_b):
            return self.mha(q_x=m_c, kv_x=m_c, biases=[mask_c] + ([z_b] if z_b is not None else []))

        outs = []
        for s in range(0, m.shape[-3], rows_per_chunk):
            m_c, mask_c = m[..., s:s + rows_per_chunk, :, :], mask_bias[..., s:s + rows_per_chunk, :, :, :]
            if checkpoint and torch.is_grad_enabled():
                from torch.utils.checkpoint import checkpoint as ckpt
                outs.append(ckpt(piece, m_c, mask_c, z, use_reentrant=False))
            else:
                outs.append(piece(m_c, mask_c, z))
        return torch.cat(outs, dim=-3)

    def forward(self, m, z=None, mask=None, chunk_size=None, _chunk_logits=None, _checkpoint_chunks=None):
        if _chunk_logits is not None:
            return self._chunked_rows(m, z, mask, _chunk_logits, bool(_checkpoint_chunks))
        m, mask_bias, z = self._prep_inputs(m, z, mask)
        biases = [mask_bias]
        if z is not None:
            biases.append(z)
        if chunk_size is not None:
            return self._chunk(m, biases, chunk_size)
        return self.mha(q_x=m, kv_x=m, biases=biases)


class MSARowAttentionWithPairBias(MSAAttention):
    def __init__(self, c_m, c_z, c_hidden, no_heads, inf=1e9):
        super().__init__(c_m, c_hidden, no_heads, pair_bias=True, c_z=c_z, inf=inf)


class MSAColumnAttention(nn.Module):
    def __init__(self, c_m, c_hidden, no_heads, inf=1e9):
        super().__init__()
        self._msa_att = MSAAttention(c_in=c_m, c_hidden=c_hidden, no_heads=no_heads, pair_bias=False, c_z=None, inf=inf)

    def forward(self, m, mask=None, chunk_size=None):
        m = m.transpose(-2, -3)
        if mask is not None:
            mask = mask.transpose(-1, -2)
        m = self._msa_att(m, mask=mask, chunk_size=chunk_size)
        return m.transpose(-2, -3)


class MSAColumnGlobalAttention(nn.Module):
    def __init__(self, c_in, c_hidden, no_heads, inf=1e9, eps=1e-10):
        super().__init__()
        self.layer_norm_m = nn.LayerNorm(c_in)
        self.global_attention = GlobalAttention(c_in=c_in, c_hidden=c_hidden, no_heads=no_heads, inf=inf, eps=eps)

    def forward(self, m, mask=None, chunk_size=None):
        if mask is None:
            mask = torch.ones(m.shape[:-1], dtype=m.dtype, device=m.device).detach()
        m = m.transpose(-2, -3)
        mask = mask.transpose(-1, -2)
        m = self.layer_norm_m(m)
        if chunk_size is not None:
            m = chunk_layer(self.global_attention, {"m": m, "mask": mask}, chunk_size=chunk_size, no_batch_dims=len(m.shape[:-2]))
        else:
            m = self.global_attention(m=m, mask=mask)
        return m.transpose(-2, -3)
