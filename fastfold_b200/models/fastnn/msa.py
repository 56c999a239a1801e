"""MSA half of the Evoformer / extra-MSA blocks (names as in fastfold/model/fastnn/msa.py)."""
import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops as K
from ...parallel import core
from ...parallel.comm import gather, scatter, scatter_mask, row_to_col, col_to_row
from ...parallel.comm_async import all_to_all_async, all_to_all_async_opp
from ...parallel.fused import a2a_layer_norm
from ...utils import memo
from ...utils.checkpointing import checkpoint_blocks
from .ops import (ChunkMSARowAttentionWithPairBias, ChunkMSAColumnGlobalAttention, ChunkTransition, GlobalAttention,
                  OutProductMean, SelfAttention, Transition, _fusable)
from .triangle import PairCore, pad_amount
from . import ops as fops


class MSARowAttentionWithPairBias(ChunkMSARowAttentionWithPairBias):
    """Row-wise gated self attention with pair bias (Algorithm 7); ``M_raw [1, S/P, N, c_m]``."""

    def __init__(self, d_node, d_pair, c=32, n_head=8, p_drop=0.15):
        super().__init__(d_node=d_node, d_pair=d_pair, c=c, n_head=n_head, p_drop=p_drop)


class MSAColumnAttention(nn.Module):
    """Column-wise gated self attention (Algorithm 8); ``M_raw [1, S, N/P, c_m]``."""

    def __init__(self, d_node, c=32, n_head=8):
        super().__init__()
        self.d_node, self.c, self.n_head = d_node, c, n_head
        self.layernormM = K.LayerNorm(d_node)
        self.attention = SelfAttention(qkv_dim=d_node, c=c, n_head=n_head, out_dim=d_node, gating=True)

    def strided_for(self, n_seq, like):
        """GPU path without transposed copies: the attention kernels walk the sequence axis (dim 1) through their row /
        batch strides.  ``n_seq``: length of that axis."""
        from ...ops import flash
        from . import ops as fops
        if fops.CHUNK_SIZE is not None:
            return False
        if not (like.is_cuda and like.dtype == torch.bfloat16 and self.c == flash.HEAD_DIM and n_seq % 8 == 0):
            return False
        return True

    def forward(self, M_raw, M_mask, M_norm_t=None, strided=None):
        """``M_norm_t``: ``layernormM`` of the input when the caller already has it - transposed ``[1, N/P, S, c]`` unless
        ``strided`` (then in the layout of ``M_raw``); ``strided=None`` decides here."""
        if strided is None:
            strided = M_norm_t is None and self.strided_for(M_raw.shape[1], M_raw)
        if strided:
            M = self.layernormM(M_raw) if M_norm_t is None else M_norm_t
            out, _ = self.attention(M, memo.cached("mask_t", (M_mask,), lambda: M_mask.transpose(-1, -2).contiguous()), transposed=True)
            return M_raw.add_(out) if fops.INPLACE else M_raw + out
        M = self.layernormM(M_raw.transpose(-2, -3).contiguous()) if M_norm_t is None else M_norm_t
        out, _ = self.attention(M, memo.cached("mask_t", (M_mask,), lambda: M_mask.transpose(-1, -2).contiguous()))
        return M_raw.add_(out.transpose(-2, -3)) if fops.INPLACE else M_raw + out.transpose(-2, -3)


class MSAColumnGlobalAttention(ChunkMSAColumnGlobalAttention):
    pass


class MSACore(nn.Module):
    def __init__(self, d_node, d_pair, p_drop=0.15):
        super().__init__()
        self.MSARowAttentionWithPairBias = MSARowAttentionWithPairBias(d_node=d_node, d_pair=d_pair, p_drop=p_drop)
        self.MSAColumnAttention = MSAColumnAttention(d_node=d_node)
        self.MSATransition = Transition(d=d_node)

    def forward(self, node, pair, node_mask, dropmask=None):
        node_mask_row = scatter_mask(node_mask, dim=1)
        node = self.MSARowAttentionWithPairBias(node, pair, node_mask_row, dropmask)
        # row -> column switch fused with the transpose + LayerNorm of the column attention
        strided = self.MSAColumnAttention.strided_for(node.shape[1] * core.get_dap_size(), node)     # full sequence count after the switch
        node, node_nt = a2a_layer_norm(node, self.MSAColumnAttention.layernormM, 0, transpose_norm=not strided)
        node_mask_col = scatter_mask(node_mask, dim=2)
        node = self.MSAColumnAttention(node, node_mask_col, M_norm_t=node_nt, strided=strided)
        node = self.MSATransition(node)
        return node


class ExtraMSACore(nn.Module):
    def __init__(self, d_node, d_pair, p_drop=0.15):
        super().__init__()
        self.MSARowAttentionWithPairBias = ChunkMSARowAttentionWithPairBias(d_node=d_node, d_pair=d_pair, p_drop=p_drop, c=8)
        self.MSAColumnAttention = ChunkMSAColumnGlobalAttention(d_node=d_node, c=8)
        self.MSATransition = ChunkTransition(d=d_node)

    def forward(self, node, pair, node_mask, dropmask=None):
        node_mask_row = scatter_mask(node_mask, dim=1)
        node = self.MSARowAttentionWithPairBias(node, pair, node_mask_row, dropmask)
        node = row_to_col(node)
        node_mask_col = scatter_mask(node_mask, dim=2)
        node = self.MSAColumnAttention(node, node_mask_col)
        node = self.MSATransition(node)
        return node

    def inplace(self, node, pair, node_mask, dropmask=None):
        with fops.inplace_scope():
            node[0] = self.forward(node[0], pair[0] if isinstance(pair, list) else pair, node_mask, dropmask)
        return node


class ExtraMSABlock(nn.Module):
    """One extra-MSA block under DAP; pads both the sequence-count and the residue axis to the DAP size."""

    def __init__(self, c_m, c_z, first_block, last_block, is_multimer=False):
        super().__init__()
        self.first_block, self.last_block = first_block, last_block
        self.msa_stack = ExtraMSACore(c_m, c_z, p_drop=0.15)
        self.communication = OutProductMean(n_feat=c_m, n_feat_out=c_z, n_feat_proj=32)
        self.pair_stack = PairCore(d_pair=c_z)
        self.is_multimer = is_multimer
        self.keep_pair_sharded = False                  # see ``Evoformer.keep_pair_sharded``

    def forward(self, m, z, msa_mask, pair_mask, chunk_size=None, _mask_trans=True, _drop=None, _memo=None):
        with memo.use(_memo):
            return self._forward(m, z, msa_mask, pair_mask, chunk_size, _mask_trans, _drop)

    def _forward(self, m, z, msa_mask, pair_mask, chunk_size=None, _mask_trans=True, _drop=None):
        P = core.get_dap_size()
        cnt_pad = pad_amount(msa_mask.size(-2), P)
        len_pad = pad_amount(pair_mask.size(-1), P)
        if self.first_block:
            m = F.pad(m.unsqueeze(0), (0, 0, 0, len_pad, 0, cnt_pad))
            m = scatter(m, dim=1) if not self.is_multimer else scatter(m, dim=2)
            if P > 1 and len_pad == 0 and z.shape[0] * P == pair_mask.size(-1):
                z = z.unsqueeze(0)                      # already this rank's row shard
            else:
                z = F.pad(z.unsqueeze(0), (0, 0, 0, len_pad, 0, len_pad))
                z = scatter(z, dim=1)
        msa_mask = memo.cached(("pad_msa", len_pad, cnt_pad), (msa_mask,), lambda: F.pad(msa_mask.unsqueeze(0), (0, len_pad, 0, cnt_pad)))
        pair_mask = memo.cached(("pad_pair", len_pad), (pair_mask,), lambda: F.pad(pair_mask.unsqueeze(0), (0, len_pad, 0, len_pad)))
        d_msa = None if _drop is None else _drop.get("msa_row")
        if not self.is_multimer:
            m = self.msa_stack(m, z, msa_mask, d_msa)
            z = self.communication(m, msa_mask, z)
            m, work = all_to_all_async(m, 1, 2)
            z = self.pair_stack(z, pair_mask, _drop)
            m = all_to_all_async_opp(m, work, 1, 2)
        else:
            z = self.communication(m, msa_mask, z)
            z_ori = z.clone() if fops.INPLACE else z          # the MSA stack below reads the pair tensor of BEFORE the pair stack
            m, work = all_to_all_async(m, 1, 2)
            z = self.pair_stack(z, pair_mask, _drop)
            m = all_to_all_async_opp(m, work, 1, 2)
            m = self.msa_stack(m, z_ori, msa_mask, d_msa)
        if self.last_block:
            m = gather(m, dim=1) if not self.is_multimer else gather(m, dim=2)
            m = m[:, :m.shape[1] - cnt_pad, :m.shape[2] - len_pad, :].squeeze(0)
            if self.keep_pair_sharded and P > 1 and len_pad == 0:
                z = z.squeeze(0)
            else:
                z = gather(z, dim=1)
                z = z[:, :z.shape[1] - len_pad, :z.shape[2] - len_pad, :].squeeze(0)
        return m, z

    def inplace(self, m, z, msa_mask, pair_mask, chunk_size=None, _mask_trans=True, _drop=None):
        with fops.inplace_scope():
            m[0], z[0] = self.forward(m[0], z[0], msa_mask, pair_mask, chunk_size, _mask_trans, _drop)
        return m, z


class ExtraMSAStack(nn.Module):
    """Algorithm 18; returns the updated pair representation only."""

    def __init__(self, c_m, c_z, no_blocks, clear_cache_between_blocks=False, is_multimer=False, blocks_per_ckpt=None, **kwargs):
        super().__init__()
        self.clear_cache_between_blocks = clear_cache_between_blocks
        self.blocks_per_ckpt = blocks_per_ckpt
        self.blocks = nn.ModuleList([
            ExtraMSABlock(c_m=c_m, c_z=c_z, first_block=(i == 0), last_block=(i == no_blocks - 1), is_multimer=is_multimer)
            for i in range(no_blocks)
        ])

    def forward(self, m, z, chunk_size=None, msa_mask=None, pair_mask=None, _mask_trans=True):
        from .evoformer import run_blocks
        m, z = run_blocks(self.blocks, m, z, msa_mask, pair_mask, chunk_size, _mask_trans, self.training,
                          self.blocks_per_ckpt if self.training else None, c_m=m.shape[-1], c_z=z.shape[-1])
        return z

    def inplace(self, m, z, chunk_size=None, msa_mask=None, pair_mask=None, _mask_trans=True):
        with fops.inplace_scope():
            z[0] = self.forward(m[0], z[0], chunk_size, msa_mask, pair_mask, _mask_trans)
        m[0] = None
        return z
