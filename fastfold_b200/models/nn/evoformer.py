"""OpenFold-layout Evoformer and extra-MSA stacks (Algorithms 6 and 18); cf. fastfold/model/nn/evoformer.py."""
from functools import partial

import torch
import torch.nn as nn

from ...utils.checkpointing import checkpoint_blocks
from .dropout import DropoutColumnwise, DropoutRowwise
from .msa import MSAColumnAttention, MSAColumnGlobalAttention, MSARowAttentionWithPairBias
from .pair import (MSATransition, OuterProductMean, PairTransition, TriangleAttentionEndingNode, TriangleAttentionStartingNode,
                   TriangleMultiplicationIncoming, TriangleMultiplicationOutgoing)
from .primitives import Linear


class EvoformerBlockCore(nn.Module):
    def __init__(self, c_m, c_z, c_hidden_opm, c_hidden_mul, c_hidden_pair_att, no_heads_msa, no_heads_pair, transition_n,
                 pair_dropout, inf, eps, _is_extra_msa_stack=False, is_multimer=False):
        super().__init__()
        self.is_multimer = is_multimer
        self.msa_transition = MSATransition(c_m=c_m, n=transition_n)
        self.outer_product_mean = OuterProductMean(c_m, c_z, c_hidden_opm)
        self.tri_mul_out = TriangleMultiplicationOutgoing(c_z, c_hidden_mul)
        self.tri_mul_in = TriangleMultiplicationIncoming(c_z, c_hidden_mul)
        self.tri_att_start = TriangleAttentionStartingNode(c_z, c_hidden_pair_att, no_heads_pair, inf=inf)
        self.tri_att_end = TriangleAttentionEndingNode(c_z, c_hidden_pair_att, no_heads_pair, inf=inf)
        self.pair_transition = PairTransition(c_z, transition_n)
        self.ps_dropout_row_layer = DropoutRowwise(pair_dropout)
        self.ps_dropout_col_layer = DropoutColumnwise(pair_dropout)

    def forward(self, m, z, msa_mask, pair_mask, chunk_size=None, _mask_trans=True):
        msa_trans_mask = msa_mask if _mask_trans else None
        pair_trans_mask = pair_mask if _mask_trans else None
        m = m + self.msa_transition(m, mask=msa_trans_mask, chunk_size=chunk_size)
        z = z + self.outer_product_mean(m, mask=msa_mask, chunk_size=chunk_size)
        z = z + self.ps_dropout_row_layer(self.tri_mul_out(z, mask=pair_mask))
        z = z + self.ps_dropout_row_layer(self.tri_mul_in(z, mask=pair_mask))
        z = z + self.ps_dropout_row_layer(self.tri_att_start(z, mask=pair_mask, chunk_size=chunk_size))
        z = z + self.ps_dropout_col_layer(self.tri_att_end(z, mask=pair_mask, chunk_size=chunk_size))
        z = z + self.pair_transition(z, mask=pair_trans_mask, chunk_size=chunk_size)
        return m, z


class EvoformerBlock(nn.Module):
    def __init__(self, c_m, c_z, c_hidden_msa_att, c_hidden_opm, c_hidden_mul, c_hidden_pair_att, no_heads_msa, no_heads_pair,
                 transition_n, msa_dropout, pair_dropout, inf, eps, is_multimer=False):
        super().__init__()
        self.msa_att_row = MSARowAttentionWithPairBias(c_m=c_m, c_z=c_z, c_hidden=c_hidden_msa_att, no_heads=no_heads_msa, inf=inf)
        self.msa_att_col = MSAColumnAttention(c_m, c_hidden_msa_att, no_heads_msa, inf=inf)
        self.msa_dropout_layer = DropoutRowwise(msa_dropout)
        self.core = EvoformerBlockCore(c_m, c_z, c_hidden_opm, c_hidden_mul, c_hidden_pair_att, no_heads_msa, no_heads_pair,
                                       transition_n, pair_dropout, inf, eps, is_multimer=is_multimer)
        self.is_multimer = is_multimer

    def forward(self, m, z, msa_mask, pair_mask, chunk_size=None, _mask_trans=True):
        if self.is_multimer:
            z = z + self.core.outer_product_mean(m, mask=msa_mask, chunk_size=chunk_size)
        m = m + self.msa_dropout_layer(self.msa_att_row(m, z=z, mask=msa_mask, chunk_size=chunk_size))
        m = m + self.msa_att_col(m, mask=msa_mask, chunk_size=chunk_size)
        if self.is_multimer:
            m = m + self.core.msa_transition(m, mask=msa_mask if _mask_trans else None, chunk_size=chunk_size)
            c = self.core
            z = z + c.ps_dropout_row_layer(c.tri_mul_out(z, mask=pair_mask))
            z = z + c.ps_dropout_row_layer(c.tri_mul_in(z, mask=pair_mask))
            z = z + c.ps_dropout_row_layer(c.tri_att_start(z, mask=pair_mask, chunk_size=chunk_size))
            z = z + c.ps_dropout_col_layer(c.tri_att_end(z, mask=pair_mask, chunk_size=chunk_size))
            z = z + c.pair_transition(z, mask=pair_mask if _mask_trans else None, chunk_size=chunk_size)
            return m, z
        return self.core(m, z, msa_mask=msa_mask, pair_mask=pair_mask, chunk_size=chunk_size, _mask_trans=_mask_trans)


class ExtraMSABlock(nn.Module):
    def __init__(self, c_m, c_z, c_hidden_msa_att, c_hidden_opm, c_hidden_mul, c_hidden_pair_att, no_heads_msa, no_heads_pair,
                 transition_n, msa_dropout, pair_dropout, inf, eps, ckpt, is_multimer=False):
        super().__init__()
        self.ckpt = ckpt
        self.msa_att_row = MSARowAttentionWithPairBias(c_m=c_m, c_z=c_z, c_hidden=c_hidden_msa_att, no_heads=no_heads_msa, inf=inf)
        self.msa_att_col = MSAColumnGlobalAttention(c_in=c_m, c_hidden=c_hidden_msa_att, no_heads=no_heads_msa, inf=inf, eps=eps)
        self.msa_dropout_layer = DropoutRowwise(msa_dropout)
        self.core = EvoformerBlockCore(c_m, c_z, c_hidden_opm, c_hidden_mul, c_hidden_pair_att, no_heads_msa, no_heads_pair,
                                       transition_n, pair_dropout, inf, eps, is_multimer=is_multimer)
        self.is_multimer = is_multimer

    def forward(self, m, z, msa_mask, pair_mask, chunk_size=None, _chunk_logits=1024, _mask_trans=True):
        if self.is_multimer:
            z = z + self.core.outer_product_mean(m, mask=msa_mask, chunk_size=chunk_size)
        # with gradients the row attention runs ``_chunk_logits`` rows at a time (checkpointed when the block is): the
        # logits of all N_extra rows at once are what makes this stack run out of memory in training
        grad = torch.is_grad_enabled()
        m = m + self.msa_dropout_layer(self.msa_att_row(m.clone(), z=z.clone(), mask=msa_mask, chunk_size=chunk_size,
                                                        _chunk_logits=_chunk_logits if grad else None,
                                                        _checkpoint_chunks=self.ckpt if grad else False))
        m = m + self.msa_att_col(m, mask=msa_mask, chunk_size=chunk_size)
        if self.is_multimer:
            c = self.core
            m = m + c.msa_transition(m, mask=msa_mask if _mask_trans else None, chunk_size=chunk_size)
            z = z + c.ps_dropout_row_layer(c.tri_mul_out(z, mask=pair_mask))
            z = z + c.ps_dropout_row_layer(c.tri_mul_in(z, mask=pair_mask))
            z = z + c.ps_dropout_row_layer(c.tri_att_start(z, mask=pair_mask, chunk_size=chunk_size))
            z = z + c.ps_dropout_col_layer(c.tri_att_end(z, mask=pair_mask, chunk_size=chunk_size))
            z = z + c.pair_transition(z, mask=pair_mask if _mask_trans else None, chunk_size=chunk_size)
            return m, z
        return self.core(m, z, msa_mask=msa_mask, pair_mask=pair_mask, chunk_size=chunk_size, _mask_trans=_mask_trans)


class EvoformerStack(nn.Module):
    def __init__(self, c_m, c_z, c_hidden_msa_att, c_hidden_opm, c_hidden_mul, c_hidden_pair_att, c_s, no_heads_msa, no_heads_pair,
                 no_blocks, transition_n, msa_dropout, pair_dropout, blocks_per_ckpt, inf, eps, clear_cache_between_blocks=False,
                 is_multimer=False, **kwargs):
        super().__init__()
        self.blocks_per_ckpt = blocks_per_ckpt
        self.clear_cache_between_blocks = clear_cache_between_blocks
        self.blocks = nn.ModuleList([
            EvoformerBlock(c_m, c_z, c_hidden_msa_att, c_hidden_opm, c_hidden_mul, c_hidden_pair_att, no_heads_msa, no_heads_pair,
                           transition_n, msa_dropout, pair_dropout, inf, eps, is_multimer=is_multimer) for _ in range(no_blocks)
        ])
        self.linear = Linear(c_m, c_s)

    def forward(self, m, z, msa_mask, pair_mask, chunk_size=None, _mask_trans=True):
        blocks = [partial(b, msa_mask=msa_mask, pair_mask=pair_mask, chunk_size=chunk_size, _mask_trans=_mask_trans) for b in self.blocks]
        m, z = checkpoint_blocks(blocks, args=(m, z), blocks_per_ckpt=self.blocks_per_ckpt if self.training else None)
        s = self.linear(m[..., 0, :, :])
        return m, z, s


class ExtraMSAStack(nn.Module):
    def __init__(self, c_m, c_z, c_hidden_msa_att, c_hidden_opm, c_hidden_mul, c_hidden_pair_att, no_heads_msa, no_heads_pair,
                 no_blocks, transition_n, msa_dropout, pair_dropout, inf, eps, ckpt=False, clear_cache_between_blocks=False,
                 is_multimer=False, **kwargs):
        super().__init__()
        self.clear_cache_between_blocks = clear_cache_between_blocks
        self.ckpt = ckpt
        self.blocks = nn.ModuleList([
            ExtraMSABlock(c_m, c_z, c_hidden_msa_att, c_hidden_opm, c_hidden_mul, c_hidden_pair_att, no_heads_msa, no_heads_pair,
                          transition_n, msa_dropout, pair_dropout, inf, eps, ckpt=ckpt, is_multimer=is_multimer) for _ in range(no_blocks)
        ])

    def forward(self, m, z, chunk_size=None, msa_mask=None, pair_mask=None, _mask_trans=True):
        blocks = [partial(b, msa_mask=msa_mask, pair_mask=pair_mask, chunk_size=chunk_size, _mask_trans=_mask_trans) for b in self.blocks]
        m, z = checkpoint_blocks(blocks, args=(m, z), blocks_per_ckpt=1 if (self.ckpt and self.training) else None)
        return z
