"""Pair half of the Evoformer block (names as in fastfold/model/fastnn/triangle.py)."""
import torch.nn as nn

from ...parallel.comm import scatter, scatter_mask, row_to_col, col_to_row
from ...parallel.fused import a2a_layer_norm
from ...utils.tensor_utils import permute_final_dims  # noqa: F401
from .ops import (AsyncChunkTriangleMultiplicationOutgoing, AsyncChunkTriangleMultiplicationIncoming,
                  ChunkTriangleAttentionStartingNode, ChunkTriangleAttentionEndingNode, ChunkTransition)


def pad_amount(n, P):
    """Rows/columns to add so that ``n`` divides by the DAP size (0 when it already does).

    The reference always pads by at least one (fastfold/model/fastnn/evoformer.py:42-43) because it
    strips the padding with ``[:-pad]``; padded positions are masked, so the outputs are the same.
    """
    return (-n) % P


class TriangleMultiplicationOutgoing(AsyncChunkTriangleMultiplicationOutgoing):
    pass


class TriangleMultiplicationIncoming(AsyncChunkTriangleMultiplicationIncoming):
    pass


class TriangleAttentionStartingNode(ChunkTriangleAttentionStartingNode):
    pass


class TriangleAttentionEndingNode(ChunkTriangleAttentionEndingNode):
    pass


class PairCore(nn.Module):
    """tri-mul out -> a2a -> tri-mul in -> a2a -> tri-att start -> a2a -> tri-att end -> transition -> a2a."""

    def __init__(self, d_pair, p_drop=0.25):
        super().__init__()
        self.d_pair = d_pair
        self.n_head = 4
        self.hidden_c = int(d_pair / self.n_head)
        self.TriangleMultiplicationOutgoing = AsyncChunkTriangleMultiplicationOutgoing(d_pair, p_drop=p_drop, c=d_pair)
        self.TriangleMultiplicationIncoming = AsyncChunkTriangleMultiplicationIncoming(d_pair, p_drop=p_drop, c=d_pair)
        self.TriangleAttentionStartingNode = ChunkTriangleAttentionStartingNode(d_pair, p_drop=p_drop, c=self.hidden_c, n_head=self.n_head)
        self.TriangleAttentionEndingNode = ChunkTriangleAttentionEndingNode(d_pair, p_drop=p_drop, c=self.hidden_c, n_head=self.n_head)
        self.PairTransition = ChunkTransition(d=d_pair)

    def forward(self, pair, pair_mask, _drop=None):
        d = _drop or {}
        pair_mask_row = scatter_mask(pair_mask, dim=1)
        pair_mask_col = scatter_mask(pair_mask, dim=2)
        # each axis switch is fused with the LayerNorm (and transpose) of the module that consumes its result
        pair = self.TriangleMultiplicationOutgoing(pair, pair_mask_row, d.get("tri_mul_out"))
        pair, pn = a2a_layer_norm(pair, self.TriangleMultiplicationIncoming.layernorm1, 0)
        dm = d.get("tri_mul_in")
        if dm is not None:
            dm = scatter(dm, dim=2)
        pair = self.TriangleMultiplicationIncoming(pair, pair_mask_col, dm, Z_norm=pn)
        pair, pn = a2a_layer_norm(pair, self.TriangleAttentionStartingNode.layernorm1, 1)
        pair = self.TriangleAttentionStartingNode(pair, pair_mask_row, d.get("tri_att_start"), Z_norm=pn)
        # the ending node attends along the first pair axis, which is complete after the switch to column shards
        strided = self.TriangleAttentionEndingNode.strided_for(pair.shape[2], pair)
        pair, pn = a2a_layer_norm(pair, self.TriangleAttentionEndingNode.layernorm1, 0, transpose_norm=not strided)
        pair = self.TriangleAttentionEndingNode(pair, pair_mask_col, d.get("tri_att_end"), Z_norm=pn, strided=strided)
        pair = self.PairTransition(pair)
        pair = col_to_row(pair)
        return pair

    def inplace(self, pair, pair_mask, _drop=None):
        from . import ops as fops
        with fops.inplace_scope():
            pair[0] = self.forward(pair[0], pair_mask, _drop)
        return pair
