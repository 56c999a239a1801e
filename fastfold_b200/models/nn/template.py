"""Template pair stack and template pointwise attention (Algorithms 16, 17); cf. fastfold/model/nn/template.py."""
from functools import partial

import torch
import torch.nn as nn

from ...utils.checkpointing import checkpoint_blocks
from ...utils.tensor_utils import chunk_layer, permute_final_dims
from .dropout import DropoutColumnwise, DropoutRowwise
from .pair import (PairTransition, TriangleAttentionEndingNode, TriangleAttentionStartingNode, TriangleMultiplicationIncoming,
                   TriangleMultiplicationOutgoing)
from .primitives import Attention, LayerNorm


class TemplatePointwiseAttention(nn.Module):
    """Every pair position attends over the templates' embeddings at that position."""

    def __init__(self, c_t, c_z, c_hidden, no_heads, inf, **kwargs):
        super().__init__()
        self.c_t, self.c_z, self.c_hidden, self.no_heads, self.inf = c_t, c_z, c_hidden, no_heads, inf
        self.mha = Attention(c_z, c_t, c_t, c_hidden, no_heads, gating=False)

    def forward(self, t, z, template_mask=None, chunk_size=None):
        if template_mask is None:
            template_mask = t.new_ones(t.shape[:-3])
        bias = self.inf * (template_mask[..., None, None, None, None, :] - 1)
        z = z.unsqueeze(-2)                       # [*, N, N, 1, C_z]
        t = permute_final_dims(t, (1, 2, 0, 3))   # [*, N, N, N_templ, C_t]
        biases = [bias]
        if chunk_size is not None:
            z = chunk_layer(self.mha, {"q_x": z, "kv_x": t, "biases": biases}, chunk_size=chunk_size, no_batch_dims=len(z.shape[:-2]))
        else:
            z = self.mha(q_x=z, kv_x=t, biases=biases)
        return z.squeeze(-2)


class TemplatePairStackBlock(nn.Module):
    def __init__(self, c_t, c_hidden_tri_att, c_hidden_tri_mul, no_heads, pair_transition_n, dropout_rate, inf, tri_mul_first=False, **kwargs):
        super().__init__()
        self.tri_mul_first = tri_mul_first
        self.dropout_row = DropoutRowwise(dropout_rate)
        self.dropout_col = DropoutColumnwise(dropout_rate)
        self.tri_att_start = TriangleAttentionStartingNode(c_t, c_hidden_tri_att, no_heads, inf=inf)
        self.tri_att_end = TriangleAttentionEndingNode(c_t, c_hidden_tri_att, no_heads, inf=inf)
        self.tri_mul_out = TriangleMultiplicationOutgoing(c_t, c_hidden_tri_mul)
        self.tri_mul_in = TriangleMultiplicationIncoming(c_t, c_hidden_tri_mul)
        self.pair_transition = PairTransition(c_t, pair_transition_n)

    def _att(self, s, mask, chunk_size):
        s = s + self.dropout_row(self.tri_att_start(s, chunk_size=chunk_size, mask=mask))
        return s + self.dropout_col(self.tri_att_end(s, chunk_size=chunk_size, mask=mask))

    def _mul(self, s, mask):
        s = s + self.dropout_row(self.tri_mul_out(s, mask=mask))
        return s + self.dropout_row(self.tri_mul_in(s, mask=mask))

    def forward(self, z, mask, chunk_size=None, _mask_trans=True):
        outs = []
        for s, m in zip([t.unsqueeze(-4) for t in torch.unbind(z, dim=-4)], [t.unsqueeze(-3) for t in torch.unbind(mask, dim=-3)]):
            if self.tri_mul_first:
                s = self._att(self._mul(s, m), m, chunk_size)
            else:
                s = self._mul(self._att(s, m, chunk_size), m)
            s = s + self.pair_transition(s, mask=m if _mask_trans else None, chunk_size=chunk_size)
            outs.append(s)
        return torch.cat(outs, dim=-4)


class TemplatePairStack(nn.Module):
    def __init__(self, c_t, c_hidden_tri_att, c_hidden_tri_mul, no_blocks, no_heads, pair_transition_n, dropout_rate, blocks_per_ckpt,
                 inf=1e9, tri_mul_first=False, **kwargs):
        super().__init__()
        self.blocks_per_ckpt = blocks_per_ckpt
        self.blocks = nn.ModuleList([
            TemplatePairStackBlock(c_t, c_hidden_tri_att, c_hidden_tri_mul, no_heads, pair_transition_n, dropout_rate, inf, tri_mul_first)
            for _ in range(no_blocks)
        ])
        self.layer_norm = LayerNorm(c_t)

    def forward(self, t, mask, chunk_size=None, _mask_trans=True):
        if mask.shape[-3] == 1:
            expand_idx = list(mask.shape)
            expand_idx[-3] = t.shape[-4]
            mask = mask.expand(*expand_idx)
        (t,) = checkpoint_blocks([partial(b, mask=mask, chunk_size=chunk_size, _mask_trans=_mask_trans) for b in self.blocks], args=(t,),
                                 blocks_per_ckpt=self.blocks_per_ckpt if self.training else None)
        return self.layer_norm(t)
