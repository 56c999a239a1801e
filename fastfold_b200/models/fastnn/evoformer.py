"""Evoformer block and stack under Dynamic Axial Parallelism.

Public contract of the reference's ``fastfold.model.fastnn.Evoformer`` /
``EvoformerStack`` (fastnn/evoformer.py:17-332): inputs without a batch
dimension, the first block pads / scatters, the last block gathers / un-pads,
``chunk_size`` and ``_mask_trans`` are accepted and ignored (chunking is set by
``set_chunk_size``), ``.inplace`` takes one-element lists.

Dropout masks are shared along one axis of the activation.  A block draws all
of its masks in one call at its start (or receives them through ``_drop``);
the stack draws them outside the activation-checkpoint boundary, so the
recomputation in backward sees the very same masks without saving or
restoring RNG state, and all DAP ranks - seeded alike - draw identical masks.
"""
from functools import partial

import torch
import torch.nn as nn
import torch.nn.functional as F

from ...parallel import core
from ...parallel.comm import gather, scatter, col_to_row
from ...parallel.comm_async import all_to_all_async, all_to_all_async_opp
from ...utils import memo
from ...utils.checkpointing import checkpoint_blocks
from .msa import MSACore
from .ops import Linear, OutProductMean
from .triangle import PairCore, pad_amount
from . import ops as fops


def draw_block_dropout(n_res_padded, c_m, c_z, device, dtype, p_msa=0.15, p_pair=0.25, generator=None, n_res=None):
    """All five axis-shared dropout masks of one block, from a single random draw.

    The draw has the un-padded length ``n_res`` (rows added to make the length divisible by the DAP size get a
    pass-through mask), so the random stream - and therefore the result - does not depend on the DAP size.
    """
    n_res = n_res_padded if n_res is None else n_res
    r = torch.rand(n_res, c_m + 4 * c_z, device=device, generator=generator)
    if n_res_padded > n_res:
        r = torch.cat([r, r.new_ones(n_res_padded - n_res, r.shape[1])], dim=0)
    keep_m = (r[:, :c_m] >= p_msa).to(dtype) / (1.0 - p_msa)
    keep_z = (r[:, c_m:] >= p_pair).to(dtype) / (1.0 - p_pair)
    kz = keep_z.reshape(n_res_padded, 4, c_z)
    return {
        "msa_row": keep_m.reshape(1, 1, n_res_padded, c_m),
        "tri_mul_out": kz[:, 0].reshape(1, 1, n_res_padded, c_z).contiguous(),
        "tri_mul_in": kz[:, 1].reshape(1, 1, n_res_padded, c_z).contiguous(),
        "tri_att_start": kz[:, 2].reshape(1, 1, n_res_padded, c_z).contiguous(),
        "tri_att_end": kz[:, 3].reshape(1, n_res_padded, 1, c_z).contiguous(),
    }


class Evoformer(nn.Module):
    def __init__(self, c_m=256, c_z=128, first_block=True, last_block=True, is_multimer=False):
        super().__init__()
        self.first_block, self.last_block = first_block, last_block
        self.c_m, self.c_z = c_m, c_z
        self.msa = MSACore(c_m, c_z, p_drop=0.15)
        self.communication = OutProductMean(n_feat=c_m, n_feat_out=c_z, n_feat_proj=32)
        self.pair = PairCore(d_pair=c_z)
        self.is_multimer = is_multimer
        # True: the last block returns the pair tensor as this rank's row shard [N/P, N, c] instead of gathering it on
        # every rank (long sequences: structure module, heads and recycling then work on the shard)
        self.keep_pair_sharded = False

    def forward(self, m, z, msa_mask, pair_mask, chunk_size=None, _mask_trans=True, _drop=None, _memo=None):
        with memo.use(_memo):
            return self._forward(m, z, msa_mask, pair_mask, chunk_size, _mask_trans, _drop)

    def _forward(self, m, z, msa_mask, pair_mask, chunk_size=None, _mask_trans=True, _drop=None):
        P = core.get_dap_size()
        seq_length = pair_mask.size(-1)
        pad = pad_amount(seq_length, P)
        if self.first_block:
            m = F.pad(m.unsqueeze(0), (0, 0, 0, pad))
            m = scatter(m, dim=2) if self.is_multimer else scatter(m, dim=1)
            if P > 1 and pad == 0 and z.shape[0] * P == seq_length:
                z = z.unsqueeze(0)                      # the caller keeps the pair tensor row-sharded between the stacks
            else:
                z = F.pad(z.unsqueeze(0), (0, 0, 0, pad, 0, pad))
                z = scatter(z, dim=1)
        msa_mask = memo.cached(("pad_msa", pad), (msa_mask,), lambda: F.pad(msa_mask.unsqueeze(0), (0, pad)))
        pair_mask = memo.cached(("pad_pair", pad), (pair_mask,), lambda: F.pad(pair_mask.unsqueeze(0), (0, pad, 0, pad)))
        if _drop is None and self.training:
            _drop = draw_block_dropout(seq_length + pad, self.c_m, self.c_z, m.device, m.dtype, n_res=seq_length)
        d_msa = None if _drop is None else _drop.get("msa_row")
        if not self.is_multimer:
            m = self.msa(m, z, msa_mask, d_msa)
            z = self.communication(m, msa_mask, z)
            m, work = all_to_all_async(m, 1, 2)
            z = self.pair(z, pair_mask, _drop)
            m = all_to_all_async_opp(m, work, 1, 2)
        else:
            z = self.communication(m, msa_mask, z)
            z_ori = z.clone() if fops.INPLACE else z          # the MSA stack below reads the pair tensor of BEFORE the pair stack
            m, work = all_to_all_async(m, 1, 2)
            z = self.pair(z, pair_mask, _drop)
            m = all_to_all_async_opp(m, work, 1, 2)
            m = self.msa(m, z_ori, msa_mask, d_msa)
        if self.last_block:
            m = m.squeeze(0)
            z = z.squeeze(0)
            m = gather(m, dim=1) if self.is_multimer else gather(m, dim=0)
            m = m[:, :seq_length, :]
            if not (self.keep_pair_sharded and P > 1 and pad == 0):
                z = gather(z, dim=0)
                z = z[:seq_length, :seq_length, :]
        return m, z

    def inplace(self, m, z, msa_mask, pair_mask, chunk_size=None, _mask_trans=True, _drop=None):
        with fops.inplace_scope():
            m[0], z[0] = self.forward(m[0], z[0], msa_mask, pair_mask, chunk_size, _mask_trans, _drop)
        return m, z


def run_blocks(blocks, m, z, msa_mask, pair_mask, chunk_size, _mask_trans, training, blocks_per_ckpt, c_m, c_z,
               clear_cache_between_blocks=False):
    """Runs a list of (extra-)Evoformer blocks with optional activation checkpointing."""
    P = core.get_dap_size()
    n_pad = pair_mask.size(-1) + pad_amount(pair_mask.size(-1), P)
    fns = []
    mm = memo.Memo()        # mask-derived tensors are computed once for all blocks and both passes (utils/memo.py)
    for b in blocks:
        drop = draw_block_dropout(n_pad, c_m, c_z, m.device, m.dtype, n_res=pair_mask.size(-1)) if training else None
        fns.append(partial(b, msa_mask=msa_mask, pair_mask=pair_mask, chunk_size=chunk_size, _mask_trans=_mask_trans, _drop=drop, _memo=mm))
    return checkpoint_blocks(fns, args=(m, z), blocks_per_ckpt=blocks_per_ckpt)


class EvoformerStack(nn.Module):
    """Algorithm 6: ``no_blocks`` Evoformer blocks and the projection of the first MSA row to the single representation."""

    def __init__(self, c_m, c_z, c_s, no_blocks, blocks_per_ckpt, clear_cache_between_blocks=False, is_multimer=False, **kwargs):
        super().__init__()
        self.blocks_per_ckpt = blocks_per_ckpt
        self.clear_cache_between_blocks = clear_cache_between_blocks
        self.c_m, self.c_z = c_m, c_z
        self.blocks = nn.ModuleList([
            Evoformer(c_m=c_m, c_z=c_z, first_block=(i == 0), last_block=(i == no_blocks - 1), is_multimer=is_multimer)
            for i in range(no_blocks)
        ])
        self.linear = Linear(c_m, c_s)

    def forward(self, m, z, msa_mask, pair_mask, chunk_size=None, _mask_trans=True):
        m, z = run_blocks(self.blocks, m, z, msa_mask, pair_mask, chunk_size, _mask_trans, self.training,
                          self.blocks_per_ckpt if self.training else None, self.c_m, self.c_z)
        s = self.linear(m[..., 0, :, :])
        return m, z, s

    def inplace(self, m, z, msa_mask, pair_mask, chunk_size=None, _mask_trans=True):
        with fops.inplace_scope():
            m[0], z[0], s = self.forward(m[0], z[0], msa_mask, pair_mask, chunk_size, _mask_trans)
        return m, z, s
