"""Building blocks of the fast (DAP-aware) trunk.

Module and parameter names follow the reference's ``fastfold/model/fastnn/ops.py``
so that its pickled models and ``inject_fastnn`` name map stay valid
(``to_qkv``, ``gating_linear``, ``gating_bias``, ``o_linear``, ``out_bias``,
``left_right_projection``, ``left_right_gate``, ``output_gate``,
``output_projection``, ``output_bias``, ``layernorm1/2``, ``linear_b`` ...).
The implementation is new: each forward is a short chain of fused kernels
(``fastfold_b200.ops``), with a fully fused no-grad variant (GEMM epilogues
carry bias, gate, mask, dropout and residual) used for inference and for the
first pass of activation checkpointing, and a variant that saves what the
hand-written backward kernels need when gradients are required.

``set_chunk_size`` keeps the reference's meaning (ops.py:31-42, 98, 164, 326):
attention in groups of ``C`` rows, transitions in ``48*C`` rows, outer product
in ``C`` columns, triangle multiplication slab by slab.  Results do not depend
on it; it only bounds transient memory.
"""
import math
import os

import torch
import torch.nn as nn
import torch.nn.functional as F

from ... import ops as K
from ...ops import flash
from ...ops.attention import attention_core
from ...parallel import comm, core
from ...parallel.comm import gather, scatter, scatter_mask
from ...utils import memo
from ...utils.tensor_utils import permute_final_dims  # noqa: F401  (public name of this module in the reference)
from ...parallel.comm_async import (gather_async, gather_async_opp, broadcast_async, broadcast_async_opp)
from .initializer import glorot_uniform_af

CHUNK_SIZE = None
DEBUG = False
# True while an ``.inplace`` entry point runs (inference only): residual-carrying GEMM epilogues then write their result
# tile over the residual tile they just read (same warp, same tile: read before write), so a module's output replaces
# its input in the same storage and no second copy of the MSA / pair tensor exists at any time.
INPLACE = False


class inplace_scope:
    """``with inplace_scope():`` - modules called inside overwrite their residual input (see ``INPLACE``)."""

    def __enter__(self):
        global INPLACE
        self.prev, INPLACE = INPLACE, (not torch.is_grad_enabled())
        return self

    def __exit__(self, *exc):
        global INPLACE
        INPLACE = self.prev
        return False


def _res_out(resid2d):
    """``out=`` argument of a residual GEMM: the residual's own storage in in-place mode, else a fresh tensor."""
    return resid2d if (INPLACE and resid2d.is_contiguous()) else None


def set_chunk_size(chunk_size):
    global CHUNK_SIZE
    CHUNK_SIZE = chunk_size


def get_chunk_size():
    return CHUNK_SIZE


def _fusable(x):
    """True when the no-grad, fully fused bf16 CUDA path applies."""
    return x.is_cuda and x.dtype == torch.bfloat16 and not torch.is_grad_enabled()


def _mask_idx(x, mask):
    from ...ops.fused_ops import _mask_index
    m2, div, mod = _mask_index(x, mask)
    return (m2.contiguous(), div, mod)


def _apply_dropout(mask, p, training):
    """Reference call style: a tensor of ones goes in, dropout is applied to it (ops.py:405, msa.py:70)."""
    if mask is None or not training:
        return None
    return mask


def make_dropout_mask(shape, p, device, dtype, generator=None):
    """Bernoulli keep-mask scaled by 1/(1-p)."""
    keep = torch.rand(shape, device=device, generator=generator) >= p
    return keep.to(dtype) / (1.0 - p)


class DropoutRowwise(nn.Module):
    def __init__(self, p):
        super().__init__()
        self.p = p

    def forward(self, x):
        return x * F.dropout(torch.ones_like(x[:, 0:1, :, :]), p=self.p, training=self.training)


class DropoutColumnwise(nn.Module):
    def __init__(self, p):
        super().__init__()
        self.p = p

    def forward(self, x):
        return x * F.dropout(torch.ones_like(x[:, :, 0:1, :]), p=self.p, training=self.training)


class Linear(nn.Linear):
    """nn.Linear with AlphaFold initialisers, evaluated by the tcgen05 GEMM on CUDA bf16 tensors."""

    def __init__(self, feature_in, feature_out, initializer="linear", use_bias=True, bias_init=0.0):
        super().__init__(feature_in, feature_out, bias=use_bias)
        self.use_bias = use_bias
        if initializer == "linear":
            glorot_uniform_af(self.weight, gain=1.0)
        elif initializer == "relu":
            glorot_uniform_af(self.weight, gain=2.0)
        elif initializer in ("zeros", "zero"):
            nn.init.zeros_(self.weight)
        if self.use_bias:
            with torch.no_grad():
                self.bias.fill_(bias_init)

    def forward(self, x, act=None):
        return K.linear(x, self.weight, self.bias, act)


# ---------------------------------------------------------------------------
# Transition
# ---------------------------------------------------------------------------
class Transition(nn.Module):
    def __init__(self, d, n=4):
        super().__init__()
        self.norm = K.LayerNorm(d)
        self.linear1 = Linear(d, n * d, initializer="relu")
        self.linear2 = Linear(n * d, d, initializer="zeros")

    def _one(self, src):
        x = self.norm(src)
        h = self.linear1(x, act="relu")
        if _fusable(src):
            s2 = src.reshape(-1, src.shape[-1])
            out = K.gemm(h.reshape(-1, h.shape[-1]), self.linear2.weight, bias=self.linear2.bias, resid=s2, out=_res_out(s2))
            return out.reshape(src.shape)
        return src + self.linear2(h)

    def forward(self, src):
        if CHUNK_SIZE is None:
            return self._one(src)
        step = CHUNK_SIZE * 48
        out = src if INPLACE else torch.empty_like(src)
        for ax in range(0, src.shape[1], step):
            part = src[:, ax:ax + step]
            res = self._one(part)
            if res.data_ptr() != part.data_ptr():
                out[:, ax:ax + step] = res
        return out

    def inplace(self, src):
        with inplace_scope():
            src[0] = self.forward(src[0])
        return src


ChunkTransition = Transition


# ---------------------------------------------------------------------------
# Outer product mean
# ---------------------------------------------------------------------------
# all-gather fused into the outer-product GEMM's load stage (no-grad pass under DAP); FASTFOLD_OPM_FUSED_GATHER=0 selects
# the publish + pull all-gather instead
_OPM_FUSED_GATHER = os.environ.get("FASTFOLD_OPM_FUSED_GATHER", "1") != "0"


class OutProductMean(nn.Module):
    def __init__(self, n_feat=64, n_feat_out=128, n_feat_proj=32):
        super().__init__()
        self.layernormM = K.LayerNorm(n_feat)
        self.linear_a = Linear(n_feat, n_feat_proj)
        self.linear_b = Linear(n_feat, n_feat_proj)
        self.o_linear = Linear(n_feat_proj * n_feat_proj, n_feat_out, initializer="zero", use_bias=True)
        self.n_feat_proj = n_feat_proj

    def _outer(self, left, right_all, inv_norm, Z_raw):
        """left [1,S,ni,d], right_all [1,S,N,e] -> Z_raw + o_linear(outer) * inv_norm."""
        S, ni, d = left.shape[1], left.shape[2], left.shape[3]
        N, e = right_all.shape[2], right_all.shape[3]
        l2 = left.reshape(S, ni * d)
        r2 = right_all.reshape(S, N * e)
        if (Z_raw.is_cuda and Z_raw.dtype == torch.bfloat16 and d == 32 and e == 32 and N % 32 == 0 and ni * d >= 64
                and self.o_linear.bias is not None):
            # the product [(i d), (j e)] leaves the GEMM epilogue already laid out as [i, j, d, e], the operand layout of
            # the output projection; its gradient comes back the other way through the same block-permuting store
            if torch.is_grad_enabled() and any(t.requires_grad for t in (l2, r2, Z_raw, self.o_linear.weight)):
                out = _OpmCore.apply(l2, r2, self.o_linear.weight, self.o_linear.bias, inv_norm.reshape(-1), Z_raw.reshape(ni * N, -1))
            else:
                out = _opm_forward(l2, r2, self.o_linear.weight, self.o_linear.bias, inv_norm.reshape(-1), Z_raw.reshape(ni * N, -1))[0]
            return out.reshape(Z_raw.shape)
        if left.is_cuda and left.dtype == torch.bfloat16 and (ni * d) % 8 == 0 and (N * e) % 64 == 0 and ni * d >= 64:
            o = K.gemm(l2, r2, a_mn=True, b_mn=True) if not torch.is_grad_enabled() else _bmm_tn(l2, r2)
        else:
            o = torch.matmul(l2.t(), r2)
        o = o.reshape(ni, d, N, e).permute(0, 2, 1, 3).reshape(1, ni, N, d * e)
        return Z_raw + self.o_linear(o) * inv_norm.to(o.dtype)

    def _fused_gather(self, M, M_mask, M_mask_col, Z_raw, src):
        """No-grad pass under DAP on the GPU: the masked right projection is written straight into a symmetric-heap
        slot and the outer-product GEMM reads every rank's slab of it tile by tile with TMA over NVLink (B operand,
        MN-major, gathered along N) - the all-gather and its gathered copy disappear.  Returns None when the shapes do
        not fit (slab extent a whole number of 128-wide tiles)."""
        P = core.get_dap_size()
        if P == 1 or torch.is_grad_enabled() or CHUNK_SIZE is not None or not (M.is_cuda and M.dtype == torch.bfloat16):
            return None
        S, ni, e = M.shape[1], M.shape[2], self.n_feat_proj
        if e != 32 or (ni * e) % 128 or self.o_linear.bias is None:
            return None
        from ...parallel import symm
        heap = symm.get_heap("dap")
        if heap is None or S * ni * e * 2 > heap.max_message():
            return None
        slot = heap.next_ring_slot(S * ni * e * 2)
        heap.slot_fence(slot, pre=True)
        r_local = heap.view(slot, (1, S, ni, e), M.dtype)
        mask_col_a = memo.cached(("opm_mask_col_as", M.dtype), (src,), lambda: M_mask_col.to(M.dtype))
        torch.mul(self.linear_b(M), mask_col_a, out=r_local)
        heap.slot_fence(slot, pre=False)
        left_act = self.linear_a(M) * mask_col_a
        inv_norm = memo.cached("opm_inv_norm", (src,), lambda: 1.0 / (torch.einsum("bsid,bsjd->bijd", M_mask_col.float(), M_mask.float()) + 1e-3))
        inv_norm = inv_norm.reshape(-1)
        N = ni * P
        l2 = left_act.reshape(S, ni * e)
        heap.consume_fence(slot, pre=True)
        o4 = K.gemm(l2, r_local.reshape(S, ni * e), a_mn=True, b_mn=True, block_out=((ni * N, 1024), 1, N * 1024, 0, 1024),
                    peer=("b", heap.peer_addresses(slot, 0)))
        heap.consume_fence(slot, pre=False)
        z2 = Z_raw.reshape(ni * N, -1)
        out = K.gemm(o4, self.o_linear.weight, bias=self.o_linear.bias, rowscale=inv_norm, resid=z2, out=_res_out(z2))
        return out.reshape(Z_raw.shape)

    def forward(self, M, M_mask, Z_raw):
        M = self.layernormM(M)
        src = M_mask                                     # the tensors below depend on the mask only: once per stack call
        M_mask = memo.cached("opm_mask", (src,), lambda: src.unsqueeze(-1))
        M_mask_col = memo.cached("opm_mask_col", (src,), lambda: scatter_mask(M_mask, dim=2))
        if _OPM_FUSED_GATHER:
            out = self._fused_gather(M, M_mask, M_mask_col, Z_raw, src)
            if out is not None:
                return out
        mask_col_a = memo.cached(("opm_mask_col_as", M.dtype), (src,), lambda: M_mask_col.to(M.dtype))
        right_act = self.linear_b(M)
        # mask before the gather: identical result, and the gathered operand is ready to use
        right_act = right_act * mask_col_a
        right_act_all, work = gather_async(right_act, dim=2)
        left_act = self.linear_a(M) * mask_col_a
        inv_norm = memo.cached("opm_inv_norm", (src,), lambda: 1.0 / (torch.einsum("bsid,bsjd->bijd", M_mask_col.float(), M_mask.float()) + 1e-3))
        right_act_all = gather_async_opp(right_act_all, work, dim=2)
        if CHUNK_SIZE is None:
            return self._outer(left_act, right_act_all, inv_norm, Z_raw)
        out = Z_raw if INPLACE else torch.empty_like(Z_raw)
        for ax in range(0, left_act.shape[2], CHUNK_SIZE):
            zpart = Z_raw[:, ax:ax + CHUNK_SIZE]
            res = self._outer(left_act[:, :, ax:ax + CHUNK_SIZE].contiguous(), right_act_all, inv_norm[:, ax:ax + CHUNK_SIZE], zpart)
            if res.data_ptr() != zpart.data_ptr():
                out[:, ax:ax + CHUNK_SIZE] = res
        return out

    def inplace(self, M, M_mask, Z_raw):
        with inplace_scope():
            Z_raw[0] = self.forward(M, M_mask, Z_raw[0])
        return Z_raw


def _opm_forward(l2, r2, w, bias, inv_norm, z2):
    """o4 [i, j, d, e] = sum_s l2[s, (i d)] r2[s, (j e)];  out = z2 + inv_norm * (o4 W^T + bias)."""
    S = l2.shape[0]
    ni, N = l2.shape[1] // 32, r2.shape[1] // 32
    o4 = K.gemm(l2, r2, a_mn=True, b_mn=True, block_out=((ni * N, 1024), 1, N * 1024, 0, 1024))
    out = K.gemm(o4, w, bias=bias, rowscale=inv_norm, resid=z2, out=_res_out(z2) if not torch.is_grad_enabled() else None)
    return out, o4


class _OpmCore(torch.autograd.Function):
    """Outer product + output projection + normalisation + residual of the outer-product-mean module, with a hand-written
    backward: five tcgen05 GEMMs and no permuted copy in either direction."""

    @staticmethod
    def forward(ctx, l2, r2, w, bias, inv_norm, z2):
        out, o4 = _opm_forward(l2, r2, w, bias, inv_norm, z2)
        ctx.save_for_backward(l2, r2, w, inv_norm, o4)
        ctx.bias_param = bias
        return out

    @staticmethod
    def backward(ctx, dout):
        l2, r2, w, inv_norm, o4 = ctx.saved_tensors
        ni, N = l2.shape[1] // 32, r2.shape[1] // 32
        dout = dout.contiguous()
        dys = dout * inv_norm.to(dout.dtype).unsqueeze(-1)                 # gradient of (o4 W^T + bias)
        dw = db = dl = dr = None
        from ...ops.gemm import sink_bias_grad, sink_weight_grad
        if ctx.needs_input_grad[2] and not sink_weight_grad(w, dys, o4):
            dw = K.weight_grad(dys, o4).to(w.dtype)
        if ctx.needs_input_grad[3] and not (ctx.bias_param is not None and sink_bias_grad(ctx.bias_param, dys)):
            db = K.colsum(dys).to(w.dtype)
        if ctx.needs_input_grad[0] or ctx.needs_input_grad[1]:
            # d o4 = dys W, stored as the matrix [(i d), (j e)] that the two operand gradients contract with
            do = K.gemm(dys, w, b_mn=True, block_out=((ni * 32, N * 32), N // 32, N * 1024, 1024, 32 * N))
            if ctx.needs_input_grad[0]:
                dl = K.gemm(r2, do)                      # [S, (i d)] = r2 [S, (j e)] x do^T
            if ctx.needs_input_grad[1]:
                dr = K.gemm(l2, do, b_mn=True)           # [S, (j e)] = l2 [S, (i d)] x do
        return dl, dr, dw, db, None, dout if ctx.needs_input_grad[5] else None


# ---------------------------------------------------------------------------
# Gated self attention
# ---------------------------------------------------------------------------
class SelfAttention(nn.Module):
    """Multi-head gated self attention on ``[b1, b2, n, c]`` (attention along ``n``)."""

    def __init__(self, qkv_dim, c, n_head, out_dim, gating=True, last_bias_fuse=False):
        super().__init__()
        self.qkv_dim, self.c, self.n_head, self.out_dim = qkv_dim, c, n_head, out_dim
        self.gating = gating
        self.last_bias_fuse = last_bias_fuse
        self.scaling = self.c ** (-0.5)
        self.to_qkv = Linear(qkv_dim, 3 * n_head * c, initializer="linear", use_bias=False)
        if gating:
            self.gating_bias = nn.Parameter(torch.ones((n_head * c,)))
            self.gating_linear = Linear(qkv_dim, n_head * c, initializer="zero", use_bias=False)
        self.o_linear = Linear(n_head * c, out_dim, initializer="zero", use_bias=(not last_bias_fuse))

    def _bias(self, nonbatched_bias, transposed=False):
        if nonbatched_bias is None:
            return None
        if isinstance(nonbatched_bias[-1], int) and nonbatched_bias[-1] == -1:
            return nonbatched_bias[0]          # already ``[b, h, q, k]`` (``pair_bias_hqk``)
        if transposed:      # projected from the un-transposed pair tensor [k, q_local, h]: gather the query axis
            b = gather_async_opp(*nonbatched_bias, dim=2)
            return b.permute(0, 3, 2, 1).contiguous()      # 'b k q h -> b h q k'
        b = gather_async_opp(*nonbatched_bias, dim=1)
        return b.permute(0, 3, 1, 2).contiguous()          # 'b q k h -> b h q k'

    def _padded_heads(self):
        """Weights of the same layer with every head widened to the fused attention kernel's 32 channels by zero rows /
        columns (the extra-MSA stack has 8-channel heads): zero q / k channels leave the logits unchanged, zero v
        channels give zero outputs that the zero columns of the output projection ignore.  Inference only; cached."""
        H, d, D = self.n_head, self.c, flash.HEAD_DIM
        # Cached in eval mode only: an optimiser that updates the parameters through raw pointers (the flat fused Adam)
        # changes neither ``_version`` nor ``data_ptr``, so in training the widened copies are rebuilt on every call.
        key = (self.to_qkv.weight.data_ptr(), self.to_qkv.weight._version, self.o_linear.weight._version,
               self.gating_linear.weight._version if self.gating else 0)
        if self.training or getattr(self, "_pad_cache", None) is None or self._pad_cache[0] != key:
            def rows(w, groups):                      # [groups * H * d, ...] -> [groups * H * D, ...]
                w = w.detach().reshape(groups, H, d, *w.shape[1:])
                out = w.new_zeros(groups, H, D, *w.shape[3:])
                out[:, :, :d] = w
                return out.reshape(groups * H * D, *w.shape[3:])
            wq = rows(self.to_qkv.weight, 3)
            wg = rows(self.gating_linear.weight, 1) if self.gating else None
            bg = rows(self.gating_bias, 1) if self.gating else None
            wo = rows(self.o_linear.weight.detach().t().contiguous(), 1).t().contiguous()
            if self.training:
                # never kept: the parameters may change without a version bump, and tensors built while a CUDA graph is
                # being captured live in the graph's memory pool, whose contents later eager code must not rely on
                self._pad_cache = None
                return wq, wg, bg, wo
            self._pad_cache = (key, wq, wg, bg, wo)
        return self._pad_cache[1:]

    def _padded_heads_differentiable(self):
        """The widened weights of ``_padded_heads`` built with differentiable ops (training): gradients flow back to the
        narrow parameters through the padding, the zero rows / columns receive none."""
        H, d, D = self.n_head, self.c, flash.HEAD_DIM
        wq = F.pad(self.to_qkv.weight.reshape(3, H, d, -1), (0, 0, 0, D - d)).reshape(3 * H * D, -1)
        wg = bg = None
        if self.gating:
            wg = F.pad(self.gating_linear.weight.reshape(H, d, -1), (0, 0, 0, D - d)).reshape(H * D, -1)
            bg = F.pad(self.gating_bias.reshape(H, d), (0, D - d)).reshape(H * D)
        wo = F.pad(self.o_linear.weight.reshape(-1, H, d), (0, D - d)).reshape(-1, H * D)
        return wq, wg, bg, wo

    def _one_padded_train(self, x, mask, bias):
        """Training on the GPU with heads narrower than the fused kernel's 32 channels (extra-MSA row attention: 8,
        template triangle attention: 16): the same zero-padding as in inference, built differentiably, so that forward and
        backward run on the fused attention kernels instead of a composite that materialises the logits."""
        H, D = self.n_head, flash.HEAD_DIM
        b1, b2, n, _ = x.shape
        wq, wg, bg, wo = self._padded_heads_differentiable()
        qkv = K.linear(x, wq).reshape(b1, b2, n, 3, H, D)
        bias5 = None if bias is None else bias.unsqueeze(1)
        if not flash.packed_supported(qkv, mask, bias5):
            return None
        o = flash.flash_attention_packed(qkv, mask, bias5, self.scaling)
        if self.gating:
            o = K.bias_sigmod_ele(K.linear(x, wg), bg, o)
        return K.linear(o, wo, self.o_linear.bias), False

    def _one_padded(self, x, mask, bias, tail):
        """No-grad GPU path for heads narrower than the fused kernel's: see ``_padded_heads``."""
        H, D = self.n_head, flash.HEAD_DIM
        wq, wg, bg, wo = self._padded_heads()
        b1, b2, n, _ = x.shape
        x2 = x.reshape(-1, x.shape[-1])
        qkv = K.gemm(x2, wq).reshape(b1, b2, n, 3, H, D)
        bias5 = None if bias is None else bias.unsqueeze(1)
        if not flash.packed_supported(qkv, mask, bias5):
            return None
        o = flash.flash_attention_packed(qkv, mask, bias5, self.scaling).reshape(-1, H * D)
        if self.gating:
            o = K.gemm(x2, wg, bias=bg, act="sigmoid", mul=o)
        if tail is not None:
            out_bias, dmask, resid = tail
            r2 = resid.reshape(-1, resid.shape[-1])
            out = K.gemm(o, wo, bias=out_bias if out_bias is not None else self.o_linear.bias, dmask=dmask, resid=r2, out=_res_out(r2))
            return out.reshape(resid.shape), True
        out = K.gemm(o, wo, bias=self.o_linear.bias)
        return out.reshape(b1, b2, n, -1), False

    def _one(self, x, mask, bias, tail, transposed=False):
        """``transposed``: ``x [b1, n, b2, c]`` and the attention runs along dim 1 (``mask [b1, b2, n]``)."""
        H, d = self.n_head, self.c
        if d < flash.HEAD_DIM and not transposed and _fusable(x) and x.shape[-2] % 8 == 0:
            res = self._one_padded(x, mask, bias, tail)
            if res is not None:
                return res
        if (d < flash.HEAD_DIM and not transposed and torch.is_grad_enabled() and x.is_cuda and x.dtype == torch.bfloat16
                and x.shape[-2] % 8 == 0 and flash.HEAD_DIM % d == 0):
            res = self._one_padded_train(x, mask, bias)
            if res is not None:
                return res
        bias5 = None if bias is None else bias.unsqueeze(1)
        if transposed:
            b1, n, b2, _ = x.shape
            qkv = self.to_qkv(x).reshape(b1, n, b2, 3, H, d)
            if not flash.packed_supported(qkv, mask, bias5, transposed=True):
                out, _ = self._one(x.transpose(1, 2).contiguous(), mask, bias, None)
                return out.transpose(1, 2).contiguous(), False
            o = flash.flash_attention_packed(qkv, mask, bias5, self.scaling, transposed=True)      # [b1, n, b2, H*d]
            b2, n = n, b2        # below only the flattened row count b2 * n matters
        else:
            b1, b2, n, _ = x.shape
            qkv = self.to_qkv(x).reshape(b1, b2, n, 3, H, d)
        if transposed:
            pass
        elif flash.packed_supported(qkv, mask, bias5):
            o = flash.flash_attention_packed(qkv, mask, bias5, self.scaling)           # [b1, b2, n, H*d]
        else:
            q, k, v = (qkv[:, :, :, i].permute(0, 1, 3, 2, 4) for i in range(3))
            o = attention_core(q, k, v, mask, bias5, self.scaling)
            o = o.permute(0, 1, 3, 2, 4).reshape(b1, b2, n, H * d)
        fused = _fusable(x)
        if self.gating:
            if fused:
                o = K.gemm(x.reshape(-1, x.shape[-1]), self.gating_linear.weight, bias=self.gating_bias, act="sigmoid",
                           mul=o.reshape(-1, H * d)).reshape(b1, b2, n, H * d)
            else:
                o = K.bias_sigmod_ele(self.gating_linear(x), self.gating_bias, o)
        if tail is not None and fused:
            out_bias, dmask, resid = tail
            r2 = resid.reshape(-1, resid.shape[-1])
            out = K.gemm(o.reshape(-1, H * d), self.o_linear.weight, bias=out_bias if out_bias is not None else self.o_linear.bias,
                         dmask=dmask, resid=r2, out=_res_out(r2))
            return out.reshape(resid.shape), True
        return self.o_linear(o), False

    def forward(self, in_data, mask, nonbatched_bias=None, tail=None, transposed=False):
        """``tail=(out_bias, (mask2d, div, mod) or None, residual)`` lets the output projection absorb the
        bias / dropout / residual that follow it; the second return value says whether it did.
        ``transposed``: attend along dim 1 of ``in_data`` instead of dim 2 (no chunking in that mode)."""
        bias = self._bias(nonbatched_bias, transposed)
        if transposed or CHUNK_SIZE is None or CHUNK_SIZE >= in_data.shape[1]:
            return self._one(in_data, mask, bias, tail, transposed)
        outs = []
        for ax in range(0, in_data.shape[1], CHUNK_SIZE):
            o, _ = self._one(in_data[:, ax:ax + CHUNK_SIZE], mask[:, ax:ax + CHUNK_SIZE], bias, None)
            outs.append(o)
        return torch.cat(outs, dim=1), False


def pair_bias_hqk(Zn, weight):
    """Pair bias of a row-sharded normalised pair tensor ``Zn [1, A/P, N, c]`` for attention over its second axis:
    ``[1, H, A, N]`` with ``bias[h, q, k] = Zn[q, k] . weight[h]``.

    On the GPU the projection GEMM stores its result channel-major (``[H, (q k)]``, transposed epilogue), so one rank's
    slab of the bias is contiguous per head and the all-gather places the slabs straight into ``[H, q, k]`` order - the
    layout the attention kernel's bias tiles are read from.  No ``'b q k h -> b h q k'`` copy exists, at any DAP size;
    the gradient of the gathered bias comes back through the matching reduce-scatter.  Returns None when the shapes do
    not fit that path (the caller then projects channel-last and permutes)."""
    A, N, H = Zn.shape[1], Zn.shape[2], weight.shape[0]
    if not (Zn.is_cuda and Zn.dtype == torch.bfloat16 and weight.dtype == torch.bfloat16 and (A * N) % 8 == 0 and A * N >= 64
            and Zn.shape[-1] % 8 == 0 and Zn.shape[-1] >= 64 and K.gemm_mod.NARROW_LINEAR_T):
        return None
    b_t = K.linear_t(Zn.reshape(A * N, Zn.shape[-1]), weight)            # [H, (q_local k)]
    return gather(b_t.view(1, H, A, N), dim=2, reduce_grad=True)


class GlobalAttention(nn.Module):
    """Column-wise global attention of the extra-MSA stack: one mean-pooled query per column."""

    def __init__(self, qkv_dim, c, n_head, out_dim):
        super().__init__()
        self.qkv_dim, self.c, self.n_head, self.out_dim = qkv_dim, c, n_head, out_dim
        self.scaling = self.c ** (-0.5)
        self.eps = 1e-10
        self.inf = 1e9
        self.to_q = Linear(qkv_dim, c * n_head, use_bias=False)
        self.to_kv = Linear(qkv_dim, 2 * c, initializer="linear", use_bias=False)
        self.gating_bias = nn.Parameter(torch.ones((n_head * c,)))
        self.gating_linear = Linear(qkv_dim, n_head * c, initializer="zero", use_bias=False)
        self.o_linear = Linear(n_head * c, out_dim, initializer="zero")

    def _one(self, m, mask):
        mk = mask.to(m.dtype)
        q = torch.sum(m * mk.unsqueeze(-1), dim=-2) / (torch.sum(mk, dim=-1)[..., None] + self.eps)
        q = self.to_q(q * self.scaling)
        q = q.view(q.shape[:-1] + (self.n_head, -1))                     # [b1, b2, H, c]
        kv = self.to_kv(m)                                               # [b1, b2, S, 2c]
        if K.fused_ops.global_attention_supported(q, kv, m):
            # inference: softmax, both small products and the gate in one kernel (one pass over kv and the gate tensor)
            gate = self.gating_linear(m)
            o = K.global_attention_core(q.reshape(-1, self.n_head, self.c), kv.reshape(-1, kv.shape[-2], 2 * self.c),
                                        mk.reshape(-1, mk.shape[-1]), gate.reshape(-1, gate.shape[-2], gate.shape[-1]), self.gating_bias)
            return self.o_linear(o.view(gate.shape))
        k, v = kv.chunk(2, dim=-1)
        logits = torch.matmul(q, k.transpose(-1, -2))                    # [b1, b2, H, S]
        weights = K.fused_softmax(logits, mk)
        o = torch.matmul(weights, v)                                     # [b1, b2, H, c]
        o = o.reshape(o.shape[:-2] + (self.n_head * self.c,))
        gate = self.gating_linear(m)
        o = K.bias_sigmod_ele(gate, self.gating_bias, o.unsqueeze(-2).expand_as(gate).contiguous())
        return self.o_linear(o)

    def forward(self, m, mask):
        if CHUNK_SIZE is None:
            return self._one(m, mask)
        outs = [self._one(m[:, ax:ax + CHUNK_SIZE], mask[:, ax:ax + CHUNK_SIZE]) for ax in range(0, m.shape[1], CHUNK_SIZE)]
        return torch.cat(outs, dim=1)


# ---------------------------------------------------------------------------
# Triangle multiplication
# ---------------------------------------------------------------------------
def _dense_fits(z, factor=8, share=0.25):
    """True when ``factor`` times the bytes of ``z`` are at most ``share`` of the device's memory."""
    if not z.is_cuda:
        return True
    total = torch.cuda.get_device_properties(z.device).total_memory
    return factor * z.numel() * z.element_size() <= share * total


class _TriangleMultiplication(nn.Module):
    """Shared body of the outgoing / incoming triangular multiplicative update.

    outgoing (z row-sharded  [1, N/P, N, c]): ab[i, j] = sum_k a[i, k] * b[j, k]; the right operand is
        all-gathered along rows.
    incoming (z column-sharded [1, N, N/P, c]): ab[i, j] = sum_k a[k, i] * b[k, j]; the left operand is
        all-gathered along columns.
    The per-channel contraction runs as one batched tcgen05 GEMM over channel-major operands
    (K-major for outgoing, MN-major for incoming).
    """
    outgoing = True

    def __init__(self, d_pair, p_drop, c=128):
        super().__init__()
        self.d_pair, self.c, self.p_drop = d_pair, c, p_drop
        self.layernorm1 = K.LayerNorm(d_pair)
        self.left_right_projection = Linear(d_pair, 2 * c)
        self.left_right_gate = Linear(d_pair, 2 * c, initializer="zeros", bias_init=1.0)
        self.output_gate = Linear(d_pair, d_pair, initializer="zeros", bias_init=1.0)
        self.layernorm2 = K.LayerNorm(c)
        self.output_projection = Linear(d_pair, d_pair, initializer="zeros", use_bias=False)
        self.output_bias = nn.Parameter(torch.zeros((d_pair,)))
        self._glu_cache = None

    # -- helpers ------------------------------------------------------------
    def _glu_weights(self):
        """Projection and gate weights interleaved row-wise so that the GEMM epilogue sees (value, gate) pairs."""
        wp, wg = self.left_right_projection.weight, self.left_right_gate.weight
        # Cached in eval mode only (see ``SelfAttention._padded_heads``): under the flat fused Adam the parameters change
        # without a version bump, and a CUDA graph must capture the rebuild so that replays see the current weights.
        key = (wp._version, wg._version, wp.data_ptr(), wg.data_ptr(), wp.dtype,
               self.left_right_projection.bias._version, self.left_right_gate.bias._version)
        if self.training or self._glu_cache is None or self._glu_cache[0] != key:
            w = torch.stack([wp.detach(), wg.detach()], dim=1).reshape(-1, wp.shape[1]).contiguous()
            b = torch.stack([self.left_right_projection.bias.detach(), self.left_right_gate.bias.detach()], dim=1).reshape(-1).contiguous()
            if self.training:
                self._glu_cache = None          # see ``SelfAttention._padded_heads``
                return w, b
            self._glu_cache = (key, w, b)
        return self._glu_cache[1], self._glu_cache[2]

    def _contract(self, left, right):
        """left/right: [1, A, B, c] channel-last -> ab [1, i, j, c]."""
        c = left.shape[-1]
        if self.outgoing:
            lt = left[0].permute(2, 0, 1).contiguous()       # [c, i, k]
            rt = right[0].permute(2, 0, 1).contiguous()      # [c, j, k]
            p = K.bmm_nt(lt, rt)                             # [c, i, j]
        else:
            lt = left[0].permute(2, 0, 1).contiguous()       # [c, k, i]
            rt = right[0].permute(2, 0, 1).contiguous()      # [c, k, j]
            p = _bmm_tn(lt, rt)                              # [c, i, j]
        return p.permute(1, 2, 0).unsqueeze(0)

    def _fused_nograd(self, Z_raw, Z_mask, dropmask, Z_norm=None):
        """Inference / checkpoint first pass: 7 kernels, no transposed copies."""
        c = self.c
        A, B = Z_raw.shape[1], Z_raw.shape[2]
        Z = self.layernorm1(Z_raw) if Z_norm is None else Z_norm
        z2 = Z.reshape(A * B, -1)
        w, b = self._glu_weights()
        P = core.get_dap_size()
        heap = None
        if P > 1:
            from ...parallel import symm
            heap = symm.get_heap("dap")
            # the gathered operand's slab extent must be a whole number of 128-wide tiles
            if heap is not None and ((A if self.outgoing else B) % 128 or (2 * c * A * B * 2) % 16 or 2 * c * A * B * 2 > heap.max_message()):
                heap = None
        if heap is not None:
            # All-gather fused into the contraction GEMM: the projection GEMM writes its (channel-major) result
            # straight into a symmetric-heap slot; the contraction then reads every rank's slab of the gathered
            # operand tile by tile through TMA over NVLink - no gathered copy exists anywhere.
            slot = heap.next_ring_slot(2 * c * A * B * 2)
            heap.slot_fence(slot, pre=True)
            lr_t = K.gemm(z2, w, bias=b, glu=True, rowscale=Z_mask.reshape(-1), trans_out=True, out=heap.view(slot, (2 * c, A * B), Z.dtype))
            heap.slot_fence(slot, pre=False)
        else:
            lr_t = K.gemm(z2, w, bias=b, glu=True, rowscale=Z_mask.reshape(-1), trans_out=True)      # [2c, A*B]
        left_t = lr_t[:c].reshape(c, A, B)
        right_t = lr_t[c:].reshape(c, A, B)
        g = K.gemm(z2, self.output_gate.weight, bias=self.output_gate.bias, act="sigmoid")
        if heap is not None:
            heap.consume_fence(slot, pre=True)
            if self.outgoing:      # right operand [c, j, k] gathered along j (the GEMM's N extent)
                p = K.gemm(left_t, right_t, peer=("b", heap.peer_addresses(slot, c * A * B * 2)))
            else:                  # left operand [c, k, i] gathered along i (the GEMM's M extent)
                p = K.gemm(left_t, right_t, a_mn=True, b_mn=True, peer=("a", heap.peer_addresses(slot, 0)))
            heap.consume_fence(slot, pre=False)
        elif self.outgoing:
            if P > 1:
                right_t = comm._gather(right_t.contiguous(), dim=1)                             # [c, N, k]
            p = K.gemm(left_t, right_t)                                                        # [c, i, j]
        else:
            if P > 1:
                left_t = comm._gather(left_t.contiguous(), dim=2)                               # [c, k, N]
            p = K.gemm(left_t, right_t, a_mn=True, b_mn=True)                                  # [c, i, j]
        n_i, n_j = p.shape[1], p.shape[2]
        ab = K.layer_norm_transposed(p.reshape(c, n_i * n_j), self.layernorm2.weight, self.layernorm2.bias, self.layernorm2.eps)
        zr2 = Z_raw.reshape(A * B, -1)
        out = K.gemm(ab, self.output_projection.weight, bias=self.output_bias, mul=g,
                     dmask=None if dropmask is None else _mask_idx(Z_raw, dropmask), resid=zr2, out=_res_out(zr2))
        return out.reshape(Z_raw.shape)

    def _chunked(self, Z_raw, Z_mask):
        """Slab-by-slab evaluation for long sequences: the gathered operand is never materialised.

        Every rank in turn broadcasts its projected slab (double-buffered, asynchronous); the receiver
        contracts it with its own operand and fills the matching block of output columns (outgoing) or
        rows (incoming).  Same result as the dense path; cf. the reference's broadcast pipeline
        (ops.py:414-498, 543-630), which additionally re-projects the slab for every output chunk.
        """
        c = self.c
        P, rank = core.get_dap_size(), core.get_dap_rank()
        Z = self.layernorm1(Z_raw)
        proj = K.glu_mask(self.left_right_projection(Z), self.left_right_gate(Z), Z_mask)
        left, right = proj[..., :c], proj[..., c:]
        g = self.output_gate(Z, act="sigmoid")
        del Z
        mine = (right if self.outgoing else left)[0].permute(2, 0, 1).contiguous()       # channel-major slab
        other = (left if self.outgoing else right)[0].permute(2, 0, 1).contiguous()
        out = torch.empty_like(Z_raw)
        bufs = [torch.empty_like(mine), torch.empty_like(mine)]
        pending = None
        for r in range(P + 1):
            nxt = None
            if r < P:
                buf = mine if r == rank else bufs[r % 2]
                nxt = (r, *broadcast_async(r, buf)) if P > 1 else (r, mine, None)
            if pending is not None:
                pr, slab, work = pending
                slab = broadcast_async_opp(slab, work)
                if self.outgoing:
                    p = K.gemm(other, slab)                                   # [c, i, j_r]
                    w = p.shape[2]
                    ab = K.layer_norm(p.permute(1, 2, 0).contiguous(), self.layernorm2.weight, self.layernorm2.bias, self.layernorm2.eps)
                    sl = (slice(None), slice(None), slice(pr * w, (pr + 1) * w))
                else:
                    p = K.gemm(slab, other, a_mn=True, b_mn=True)             # [c, i_r, j]
                    w = p.shape[1]
                    ab = K.layer_norm(p.permute(1, 2, 0).contiguous(), self.layernorm2.weight, self.layernorm2.bias, self.layernorm2.eps)
                    sl = (slice(None), slice(pr * w, (pr + 1) * w), slice(None))
                ab = self.output_projection(ab).unsqueeze(0)
                out[sl] = Z_raw[sl] + g[sl] * (ab + self.output_bias)
            pending = nxt
        return out

    def forward(self, Z_raw, Z_mask, dropmask=None, Z_norm=None):
        """``Z_norm``: ``layernorm1(Z_raw)`` when the caller already has it (fused all-to-all + LayerNorm)."""
        training = self.training
        if dropmask is None and training and self.p_drop > 0:
            dropmask = F.dropout(torch.ones_like(Z_raw[:, 0:1, :, :]), p=self.p_drop, training=True)
        if not training:
            dropmask = None
        can_fuse = _fusable(Z_raw) and (Z_raw.shape[1] * Z_raw.shape[2]) % 8 == 0 and Z_raw.shape[1] % 8 == 0 and Z_raw.shape[2] % 8 == 0
        if CHUNK_SIZE is not None and not torch.is_grad_enabled():
            # The slab pipeline bounds memory (its temporaries are one rank's slab) but pays permuted copies of both
            # operands; the dense no-grad path has none and needs about eight times the local pair tensor, so it is
            # taken whenever that is a small part of the GPU's memory.
            if not (can_fuse and _dense_fits(Z_raw)):
                return self._chunked(Z_raw, Z_mask)
        if can_fuse:
            return self._fused_nograd(Z_raw, Z_mask, dropmask, Z_norm)
        c = self.c
        Z = self.layernorm1(Z_raw) if Z_norm is None else Z_norm
        if (Z_raw.is_cuda and Z_raw.dtype == torch.bfloat16 and (Z_raw.shape[1] * Z_raw.shape[2]) % 8 == 0 and Z_raw.shape[1] % 8 == 0
                and Z_raw.shape[2] % 8 == 0 and c <= 256 and c % 8 == 0):
            return self._channel_major_train(Z_raw, Z, Z_mask, dropmask, training)
        proj = K.glu_mask(self.left_right_projection(Z), self.left_right_gate(Z), Z_mask)
        left, right = proj[..., :c], proj[..., c:]
        if self.outgoing:
            right, work = gather_async(right.contiguous(), dim=1)
            g = self.output_gate(Z, act="sigmoid")
            right = gather_async_opp(right, work, dim=1)
        else:
            left, work = gather_async(left.contiguous(), dim=2)
            g = self.output_gate(Z, act="sigmoid")
            left = gather_async_opp(left, work, dim=2)
        ab = self._contract(left, right)
        ab = self.output_projection(self.layernorm2(ab.contiguous()))
        return K.bias_ele_dropout_residual(ab, self.output_bias, g, dropmask, Z_raw, prob=0.0, training=training)

    def _channel_major_train(self, Z_raw, Z, Z_mask, dropmask, training):
        """Differentiable GPU path: the projections leave their GEMM channel-major, the gate, the contraction and the
        second LayerNorm's input stay channel-major, and every backward kernel reads / writes that layout too, so the
        step has no permuted copy in either direction."""
        c = self.c
        A, B = Z_raw.shape[1], Z_raw.shape[2]
        z2 = Z.reshape(A * B, -1)
        # [4c, tokens]: values, then gates; each projection's gradient goes straight to its own buffer
        pre_t = K.linear_t_multi(z2, (self.left_right_projection.weight, self.left_right_gate.weight),
                                 (self.left_right_projection.bias, self.left_right_gate.bias))
        left_t, right_t = K.glu_mask_t(pre_t, Z_mask.reshape(-1), split=c)                               # 2 x [c, A*B]
        left_t = left_t.reshape(c, A, B)
        right_t = right_t.reshape(c, A, B)
        g = self.output_gate(Z, act="sigmoid")
        if self.outgoing:
            right_t = gather(right_t, dim=1, reduce_grad=True)          # [c, j (all), k]
            p = K.bmm_nt(left_t, right_t)                               # [c, i, j]
        else:
            left_t = gather(left_t, dim=2, reduce_grad=True)            # [c, k, i (all)]
            p = _bmm_tn(left_t, right_t)                                # [c, i, j]
        n_i, n_j = p.shape[1], p.shape[2]
        ab = K.layer_norm_transposed(p.reshape(c, n_i * n_j), self.layernorm2.weight, self.layernorm2.bias, self.layernorm2.eps)
        ab = self.output_projection(ab).reshape(Z_raw.shape)
        return K.bias_ele_dropout_residual(ab, self.output_bias, g, dropmask, Z_raw, prob=0.0, training=training)

    def inplace(self, Z_raw, Z_mask, dropmask=None):
        with inplace_scope():
            Z_raw[0] = self.forward(Z_raw[0], Z_mask, dropmask)
        return Z_raw


class _BmmTN(torch.autograd.Function):
    """out[b] = A[b]^T @ B[b] for A [b, K, M], B [b, K, N] (both contraction-strided)."""

    @staticmethod
    def forward(ctx, a, b):
        ctx.save_for_backward(a, b)
        return K.gemm(a, b, a_mn=True, b_mn=True)

    @staticmethod
    def backward(ctx, dout):
        a, b = ctx.saved_tensors
        dout = dout.contiguous()
        da = db = None
        if ctx.needs_input_grad[0]:
            da = K.gemm(b, dout)                  # [K, M] = b [K, N] x dout [M, N]^T
        if ctx.needs_input_grad[1]:
            db = K.gemm(a, dout, b_mn=True)       # [K, N] = a [K, M] x dout [M, N]
        return da, db


def _bmm_tn(a, b):
    ok = (a.is_cuda and a.dtype == torch.bfloat16 and a.shape[-1] % 8 == 0 and b.shape[-1] % 8 == 0 and a.shape[-2] % 8 == 0
          and a.shape[-1] >= 64 and b.shape[-1] >= 64)
    if not ok:
        return torch.matmul(a.transpose(-1, -2), b)
    if torch.is_grad_enabled() and (a.requires_grad or b.requires_grad):
        return _BmmTN.apply(a, b)
    return K.gemm(a, b, a_mn=True, b_mn=True)


class AsyncChunkTriangleMultiplicationOutgoing(_TriangleMultiplication):
    outgoing = True


class AsyncChunkTriangleMultiplicationIncoming(_TriangleMultiplication):
    outgoing = False


# ---------------------------------------------------------------------------
# Triangle attention
# ---------------------------------------------------------------------------
class _TriangleAttention(nn.Module):
    starting = True

    def __init__(self, d_pair, p_drop, c=32, n_head=4):
        super().__init__()
        self.d_pair, self.c, self.n_head, self.p_drop = d_pair, c, n_head, p_drop
        self.layernorm1 = K.LayerNorm(d_pair)
        self.linear_b = Linear(d_pair, n_head, initializer="linear", use_bias=False)
        self.attention = SelfAttention(qkv_dim=d_pair, c=c, n_head=n_head, out_dim=d_pair, gating=True, last_bias_fuse=True)
        self.out_bias = nn.Parameter(torch.zeros((d_pair,)))

    def forward(self, Z_raw, Z_mask, dropmask=None, Z_norm=None, strided=None):
        """``Z_norm``: the normalised input when the caller already has it from the fused all-to-all + LayerNorm; for the
        ending node the caller also says through ``strided`` which layout that is (``self.strided_for`` decides:
        True = same layout as ``Z_raw``, False = transposed)."""
        training = self.training
        if self.starting:
            mask = Z_mask
            if dropmask is None and training and self.p_drop > 0:
                dropmask = F.dropout(torch.ones_like(Z_raw[:, 0:1, :, :]), p=self.p_drop, training=True)
        else:
            mask = memo.cached("mask_t", (Z_mask,), lambda: Z_mask.transpose(-1, -2).contiguous())
            if dropmask is None and training and self.p_drop > 0:
                dropmask = F.dropout(torch.ones_like(Z_raw[:, :, 0:1, :]), p=self.p_drop, training=True)
        if not training:
            dropmask = None
        if strided is None:
            strided = self.strided(Z_raw)
        if Z_norm is not None:
            Z = Z_norm
        else:
            Z = self.layernorm1(Z_raw if (self.starting or strided) else Z_raw.transpose(-2, -3).contiguous())
        b = pair_bias_hqk(Z, self.linear_b.weight) if not strided else None
        if b is not None:
            work = -1
        else:
            b = self.linear_b(Z)
            b, work = gather_async(b, dim=2 if strided else 1)
        tail = None
        if (self.starting or strided) and _fusable(Z_raw):
            tail = (self.out_bias, None if dropmask is None else _mask_idx(Z_raw, dropmask), Z_raw)
        out, done = self.attention(Z, mask, (b, work), tail=tail, transposed=strided)
        if done:
            return out
        if strided:
            return K.bias_dropout_add(out, self.out_bias, dropmask, Z_raw, prob=0.0, training=training)
        if not self.starting:
            out = out.transpose(-2, -3)
        return K.bias_dropout_add(out.contiguous(), self.out_bias, dropmask, Z_raw, prob=0.0, training=training)

    def strided(self, Z_raw):
        """Ending node on the GPU: the attention kernels walk the first pair axis through their row / batch strides, so
        neither the input nor the output is transposed (``Z_norm``, when given, is then in the un-transposed layout)."""
        return self.strided_for(Z_raw.shape[1], Z_raw)

    def strided_for(self, n_attn, like):
        """``n_attn``: length of the axis the ending node attends along (the full first pair axis)."""
        if self.starting or CHUNK_SIZE is not None:
            return False
        if not (like.is_cuda and like.dtype == torch.bfloat16 and self.c == flash.HEAD_DIM and n_attn % 8 == 0):
            return False
        return True

    def inplace(self, Z_raw, Z_mask, dropmask=None):
        with inplace_scope():
            Z_raw[0] = self.forward(Z_raw[0], Z_mask, dropmask)
        return Z_raw


class ChunkTriangleAttentionStartingNode(_TriangleAttention):
    starting = True


class ChunkTriangleAttentionEndingNode(_TriangleAttention):
    starting = False


# ---------------------------------------------------------------------------
# MSA attentions
# ---------------------------------------------------------------------------
class ChunkMSARowAttentionWithPairBias(nn.Module):
    def __init__(self, d_node, d_pair, c=32, n_head=8, p_drop=0.15):
        super().__init__()
        self.d_node, self.d_pair, self.c, self.n_head, self.p_drop = d_node, d_pair, c, n_head, p_drop
        self.layernormM = K.LayerNorm(d_node)
        self.layernormZ = K.LayerNorm(d_pair)
        self.linear_b_weights = nn.Parameter(torch.nn.init.normal_(torch.zeros([n_head, d_pair]), std=1.0 / math.sqrt(d_pair)))
        self.attention = SelfAttention(qkv_dim=d_node, c=c, n_head=n_head, out_dim=d_node, gating=True, last_bias_fuse=True)
        self.out_bias = nn.Parameter(torch.zeros((d_node,)))

    def forward(self, M_raw, Z, M_mask, dropmask=None):
        training = self.training
        if dropmask is None and training and self.p_drop > 0:
            dropmask = F.dropout(torch.ones_like(M_raw[:, 0:1, :, :]), p=self.p_drop, training=True)
        if not training:
            dropmask = None
        M = self.layernormM(M_raw)
        Zn = self.layernormZ(Z)
        b = pair_bias_hqk(Zn, self.linear_b_weights)
        if b is not None:
            work = -1
        else:
            b = K.linear(Zn, self.linear_b_weights)
            b, work = gather_async(b, dim=1)
        tail = None
        if _fusable(M_raw):
            tail = (self.out_bias, None if dropmask is None else _mask_idx(M_raw, dropmask), M_raw)
        out, done = self.attention(M, M_mask, (b, work), tail=tail)
        if done:
            return out
        return K.bias_dropout_add(out, self.out_bias, dropmask, M_raw, prob=0.0, training=training)

    def inplace(self, M_raw, Z, M_mask, dropmask=None):
        with inplace_scope():
            M_raw[0] = self.forward(M_raw[0], Z, M_mask, dropmask)
        return M_raw


class ChunkMSAColumnGlobalAttention(nn.Module):
    def __init__(self, d_node, c=8, n_head=8):
        super().__init__()
        self.d_node, self.c, self.n_head = d_node, c, n_head
        self.layernormM = K.LayerNorm(d_node)
        self.global_attention = GlobalAttention(qkv_dim=d_node, c=c, n_head=n_head, out_dim=d_node)

    def forward(self, M_raw, M_mask):
        M = self.layernormM(M_raw.transpose(-2, -3).contiguous())
        M = self.global_attention(M, M_mask.transpose(-1, -2).contiguous())
        if INPLACE:
            return M_raw.add_(M.transpose(-2, -3))
        return M_raw + M.transpose(-2, -3)

    def inplace(self, M_raw, M_mask):
        with inplace_scope():
            M_raw[0] = self.forward(M_raw[0], M_mask)
        return M_raw


def __getattr__(name):
    # fastfold/model/fastnn/ops.py:1238-1420 defines the lean input / recycling embedders in this module; here they live
    # in embedders.py (which builds on models.nn.embedders) and are reachable under the old names.
    if name in ("InputEmbedder", "RecyclingEmbedder"):
        from . import embedders
        return getattr(embedders, name)
    raise AttributeError("module %r has no attribute %r" % (__name__, name))
