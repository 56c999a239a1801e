"""Fast (DAP-aware) template pair stack and template pointwise attention.

Each template's pair embedding ``[1, N, N, c_t]`` is row-sharded over the DAP group and goes through the same fast
triangle modules as the Evoformer pair stack, in the template stack's order: attention (starting, ending node),
multiplication (outgoing, incoming), transition - or multiplication first for the multimer model - with an axis switch
(all-to-all) between row- and column-sharded modules.  Same role as fastfold/model/fastnn/template.py
(TemplatePointwiseAttention :33-182, TemplatePairBlock :185-297, TemplatePairStack :300-434).
"""
from functools import partial

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops as K
from ...parallel import core
from ...parallel.comm import col_to_row, gather, row_to_col, scatter
from ...utils.checkpointing import checkpoint_blocks
from ..nn.template import TemplatePointwiseAttention as _PointwiseAttention
from .evoformer import draw_block_dropout, pad_amount
from .ops import (AsyncChunkTriangleMultiplicationIncoming, AsyncChunkTriangleMultiplicationOutgoing, ChunkTransition,
                  ChunkTriangleAttentionEndingNode, ChunkTriangleAttentionStartingNode)


class TemplatePointwiseAttention(_PointwiseAttention):
    """Attention of every pair position over the templates; chunked over pair rows when ``chunk_size`` is given.
    ``inplace`` adds the result into ``z[0]`` chunk by chunk."""

    def inplace(self, t, z, template_mask=None, chunk_size=None):
        n = z[0].shape[-3]
        step = n if chunk_size is None else max(1, chunk_size)
        for i in range(0, n, step):
            upd = super().forward(t[..., i:i + step, :, :], z[0][..., i:i + step, :, :], template_mask=template_mask, chunk_size=None)
            z[0][..., i:i + step, :, :] += upd
        return z


class TemplatePairBlock(nn.Module):
    def __init__(self, c_t, c_hidden_tri_att, c_hidden_tri_mul, no_heads, pair_transition_n, dropout_rate, inf, first_block, last_block,
                 tri_mul_first=False, **kwargs):
        super().__init__()
        self.first_block, self.last_block, self.tri_mul_first = first_block, last_block, tri_mul_first
        self.c_t, self.n_head, self.p_drop = c_t, no_heads, dropout_rate
        self.TriangleAttentionStartingNode = ChunkTriangleAttentionStartingNode(c_t, p_drop=dropout_rate, c=c_hidden_tri_att, n_head=no_heads)
        self.TriangleAttentionEndingNode = ChunkTriangleAttentionEndingNode(c_t, p_drop=dropout_rate, c=c_hidden_tri_att, n_head=no_heads)
        self.TriangleMultiplicationOutgoing = AsyncChunkTriangleMultiplicationOutgoing(c_t, p_drop=dropout_rate, c=c_hidden_tri_mul)
        self.TriangleMultiplicationIncoming = AsyncChunkTriangleMultiplicationIncoming(c_t, p_drop=dropout_rate, c=c_hidden_tri_mul)
        self.PairTransition = ChunkTransition(d=c_t, n=pair_transition_n)

    def _attention(self, z, mask_row, mask_col, d):
        z = self.TriangleAttentionStartingNode(z, mask_row, d.get("tri_att_start"))
        z = row_to_col(z)
        z = self.TriangleAttentionEndingNode(z, mask_col, d.get("tri_att_end"))
        return col_to_row(z)

    def _multiplication(self, z, mask_row, mask_col, d):
        z = self.TriangleMultiplicationOutgoing(z, mask_row, d.get("tri_mul_out"))
        z = row_to_col(z)
        dm = d.get("tri_mul_in")
        if dm is not None:
            dm = scatter(dm, dim=2)
        z = self.TriangleMultiplicationIncoming(z, mask_col, dm)
        return col_to_row(z)

    def inplace(self, z, mask, chunk_size=None, _mask_trans=True, _drop=None):
        """``z`` is a one-element list whose tensor is updated through the in-place residual epilogues."""
        from . import ops as fops
        with fops.inplace_scope():
            z[0] = self.forward(z[0], mask, chunk_size, _mask_trans, _drop)
        return z

    def forward(self, z, mask, chunk_size=None, _mask_trans=True, _drop=None):
        """``z [*, N_templ, N, N, c_t]`` (full on the first block, row shards afterwards), ``mask [*, N_templ, N, N]``.
        ``_drop``: one dict of axis-shared dropout masks per template (``draw_block_dropout``), drawn by the stack outside
        its activation-checkpoint boundary so that the recomputation in backward sees the masks of the first pass."""
        P = core.get_dap_size()
        n = mask.shape[-1]
        pad = pad_amount(n, P)
        if self.first_block:
            z = F.pad(z, (0, 0, 0, pad, 0, pad))
            z = scatter(z, dim=-3)
        mask = F.pad(mask, (0, pad, 0, pad))
        outs = []
        for i in range(z.shape[-4]):
            s = z[..., i, :, :, :].reshape((1,) + z.shape[-3:])
            m = mask[..., i, :, :].reshape((1,) + mask.shape[-2:])
            m_row, m_col = scatter(m, dim=1), scatter(m, dim=2)
            d = {}
            if self.training and self.p_drop > 0:
                d = _drop[i] if _drop is not None else draw_block_dropout(n + pad, 0, self.c_t, s.device, s.dtype, p_pair=self.p_drop, n_res=n)
            if self.tri_mul_first:
                s = self._attention(self._multiplication(s, m_row, m_col, d), m_row, m_col, d)
            else:
                s = self._multiplication(self._attention(s, m_row, m_col, d), m_row, m_col, d)
            s = self.PairTransition(s)
            outs.append(s)
        z = torch.stack([o[0] for o in outs], dim=0).reshape(z.shape)
        if self.last_block:
            z = gather(z, dim=-3)
            if pad:
                z = z[..., :n, :n, :]
        return z


class TemplatePairStack(nn.Module):
    def __init__(self, c_t, c_hidden_tri_att, c_hidden_tri_mul, no_blocks, no_heads, pair_transition_n, dropout_rate, blocks_per_ckpt, inf=1e9,
                 tri_mul_first=False, **kwargs):
        super().__init__()
        self.blocks_per_ckpt = blocks_per_ckpt
        self.blocks = nn.ModuleList([
            TemplatePairBlock(c_t, c_hidden_tri_att, c_hidden_tri_mul, no_heads, pair_transition_n, dropout_rate, inf, first_block=(i == 0),
                              last_block=(i == no_blocks - 1), tri_mul_first=tri_mul_first) for i in range(no_blocks)])
        self.layer_norm = K.LayerNorm(c_t)

    def forward(self, t, mask, chunk_size=None, _mask_trans=True):
        if mask.shape[-3] == 1:
            expand_idx = list(mask.shape)
            expand_idx[-3] = t.shape[-4]
            mask = mask.expand(*expand_idx)
        fns = []
        n = mask.shape[-1]
        n_pad = n + pad_amount(n, core.get_dap_size())
        for b in self.blocks:
            drop = None
            if self.training and b.p_drop > 0:
                # masks are inputs of the checkpointed function, not random draws inside it (no RNG state is saved)
                drop = [draw_block_dropout(n_pad, 0, b.c_t, t.device, t.dtype, p_pair=b.p_drop, n_res=n) for _ in range(t.shape[-4])]
            fns.append(partial(b, mask=mask, chunk_size=chunk_size, _mask_trans=_mask_trans, _drop=drop))
        (t,) = checkpoint_blocks(fns, args=(t,), blocks_per_ckpt=self.blocks_per_ckpt if self.training else None)
        return self.layer_norm(t)

    def inplace(self, t, mask, chunk_size=None, _mask_trans=True):
        t[0] = self.forward(t[0], mask, chunk_size=chunk_size, _mask_trans=_mask_trans)
        return t
