"""Memory-lean embedders for long sequences (roles of fastfold/model/fastnn/embedders.py and the embedder classes of
fastnn/ops.py:1046-1334).

Same parameters as the ``models.nn`` embedders (``inject_embedder`` moves the weights with ``load_state_dict``); what
changes is the evaluation order: pair-shaped intermediates ([N, N, bins] one-hots, per-template 88-channel features)
are produced a block of rows at a time and consumed immediately, and per-template pair embeddings can wait in host
memory while the others are computed (``chunk_size`` 1..4, as in the reference).
"""
from functools import partial

import torch
import torch.nn as nn

from ...utils.feats import build_template_angle_feat, build_template_pair_feat
from ...utils.tensor_utils import const_like, tensor_tree_map
from ..nn import embedders as ref

ROW_BLOCK = 256


class InputEmbedder(ref.InputEmbedder):
    def forward(self, tf, ri, msa, rows=None):
        """``rows=(r0, r1)``: build only those rows of the pair embedding (a DAP rank's shard)."""
        tf_emb_i = self.linear_tf_z_i(tf)
        tf_emb_j = self.linear_tf_z_j(tf)
        n = tf.shape[-2]
        if rows is not None:
            r0, r1 = rows
            rii = ri.long()
            table = self.linear_relpos.weight.t()
            pair_emb = tf_emb_i.new_empty(tf.shape[:-2] + (r1 - r0, n, self.c_z))
            for i in range(r0, r1, ROW_BLOCK):
                e = min(i + ROW_BLOCK, r1)
                idx = torch.clamp(rii[..., i:e, None] - rii[..., None, :], -self.relpos_k, self.relpos_k) + self.relpos_k
                rel = torch.nn.functional.embedding(idx, table) + self.linear_relpos.bias
                pair_emb[..., i - r0:e - r0, :, :] = rel + tf_emb_i[..., i:e, None, :] + tf_emb_j[..., None, :, :]
            n_clust = msa.shape[-3]
            tf_m = self.linear_tf_m(tf).unsqueeze(-3).expand(((-1,) * len(tf.shape[:-2]) + (n_clust, -1, -1)))
            return self.linear_msa_m(msa) + tf_m, pair_emb
        pair_emb = tf_emb_i.new_empty(tf.shape[:-2] + (n, n, self.c_z))
        # one_hot(nearest bin of i - j) times the weight is a row lookup: bin = clip(i - j, -k, k) + k, computed on the
        # integer residue indices (in bf16 the indices themselves stop being exact beyond 256)
        rii = ri.long()
        table = self.linear_relpos.weight.t()                                   # [2k + 1, c_z]
        for i in range(0, n, ROW_BLOCK):
            idx = torch.clamp(rii[..., i:i + ROW_BLOCK, None] - rii[..., None, :], -self.relpos_k, self.relpos_k) + self.relpos_k
            rel = torch.nn.functional.embedding(idx, table) + self.linear_relpos.bias
            pair_emb[..., i:i + ROW_BLOCK, :, :] = rel + tf_emb_i[..., i:i + ROW_BLOCK, None, :] + tf_emb_j[..., None, :, :]
        n_clust = msa.shape[-3]
        tf_m = self.linear_tf_m(tf).unsqueeze(-3).expand(((-1,) * len(tf.shape[:-2]) + (n_clust, -1, -1)))
        return self.linear_msa_m(msa) + tf_m, pair_emb


class RecyclingEmbedder(ref.RecyclingEmbedder):
    def forward(self, m, z, x, row0=0):
        """``z`` may be a row shard ``[n_local, N, c]`` of the pair tensor whose first row is residue ``row0``."""
        bins = torch.linspace(self.min_bin, self.max_bin, self.no_bins, dtype=x.dtype, device=x.device, requires_grad=False)
        squared_bins = bins ** 2
        upper = torch.cat([squared_bins[1:], const_like(squared_bins, [self.inf], "inf_%r" % (self.inf,))], dim=-1)
        m_update = self.layer_norm_m(m)
        from ...ops import embed as kembed
        if z.shape[-3] != x.shape[-2]:
            nl = z.shape[-3]
            z_update = torch.empty_like(z)
            for i in range(0, nl, ROW_BLOCK):
                e = min(i + ROW_BLOCK, nl)
                d = torch.sum((x[..., row0 + i:row0 + e, None, :] - x[..., None, :, :]) ** 2, dim=-1, keepdims=True)
                d = ((d > squared_bins) * (d < upper)).type(z.dtype)
                z_update[..., i:e, :, :] = self.linear(d) + self.layer_norm_z(z[..., i:e, :, :])
            return m_update, z_update
        if kembed.recycle_pair_embed_supported(z, x):
            # one pass: distance bin, weight-column gather, LayerNorm and add (no one-hot tensor, no GEMM with K = no_bins)
            ln = self.layer_norm_z
            return m_update, kembed.recycle_pair_embed(z, x, squared_bins, self.inf, self.linear.weight, self.linear.bias,
                                                       ln.weight, ln.bias, ln.eps)
        n = z.shape[-3]
        z_update = torch.empty_like(z)
        for i in range(0, n, ROW_BLOCK):
            d = torch.sum((x[..., i:i + ROW_BLOCK, None, :] - x[..., None, :, :]) ** 2, dim=-1, keepdims=True)
            d = ((d > squared_bins) * (d < upper)).type(z.dtype)
            z_update[..., i:i + ROW_BLOCK, :, :] = self.linear(d) + self.layer_norm_z(z[..., i:i + ROW_BLOCK, :, :])
        return m_update, z_update


class ExtraMSAEmbedder(ref.ExtraMSAEmbedder):
    pass


class TemplateAngleEmbedder(ref.TemplateAngleEmbedder):
    pass


class TemplatePairEmbedder(ref.TemplatePairEmbedder):
    pass


class TemplateEmbedder(ref.TemplateEmbedder):
    """One template at a time through feature construction, pair embedding and the pair stack; the finished
    ``[N, N, c_t]`` embeddings wait on the host when ``chunk_size`` is 1..4 (fastnn/embedders.py:139-254)."""

    def forward(self, batch, z, pair_mask, templ_dim, chunk_size, _mask_trans=True, inplace=False):
        n_templ = batch["template_aatype"].shape[templ_dim]
        offload = chunk_size is not None and 1 <= chunk_size <= 4 and z.is_cuda
        angles, pairs = [], []
        for i in range(n_templ):
            idx = const_like(batch["template_aatype"], i, "templ_idx_%d" % i)
            single = tensor_tree_map(lambda t: torch.index_select(t, templ_dim, idx), batch)
            if self.config.embed_angles:
                angles.append(self.template_angle_embedder(build_template_angle_feat(single)))
            t = build_template_pair_feat(single, use_unit_vector=self.config.use_unit_vector, inf=self.config.inf, eps=self.config.eps,
                                         **self.config.distogram).to(z.dtype)
            t = self.template_pair_embedder(t)
            t = self.template_pair_stack(t, pair_mask.unsqueeze(-3).to(dtype=z.dtype), chunk_size=chunk_size, _mask_trans=_mask_trans)
            pairs.append(t.cpu() if offload else t)
            del t, single
        t = torch.cat([p.to(z.device) for p in pairs], dim=templ_dim)
        del pairs
        t = self.template_pointwise_att(t, z, template_mask=batch["template_mask"].to(dtype=z.dtype), chunk_size=chunk_size)
        t = t * (torch.sum(batch["template_mask"]) > 0)
        ret = {"template_pair_embedding": t}
        if self.config.embed_angles:
            ret["template_angle_embedding"] = torch.cat(angles, dim=templ_dim)
        return ret


def inject_embedder(model):
    """Swaps the input / recycling / extra-MSA / template embedders for the lean versions (same weights)."""
    def swap(name, cls, *args, **kwargs):
        old = getattr(model, name)
        new = cls(*args, **kwargs)
        p = next(old.parameters())
        new = new.to(device=p.device, dtype=p.dtype)
        new.load_state_dict(old.state_dict())
        new.train(old.training)
        setattr(model, name, new)
    c = model.config
    if not model.globals.get("is_multimer", False):
        swap("input_embedder", InputEmbedder, **c["input_embedder"])
        if c.template.enabled and isinstance(model.template_embedder, ref.TemplateEmbedder):
            old = model.template_embedder
            new = TemplateEmbedder(c.template)
            new.template_angle_embedder = old.template_angle_embedder
            new.template_pair_embedder = old.template_pair_embedder
            new.template_pair_stack = old.template_pair_stack
            new.template_pointwise_att = old.template_pointwise_att
            new.train(old.training)
            model.template_embedder = new
    else:
        from . import embedders_multimer as mm
        swap("input_embedder", mm.InputEmbedderMultimer, **c["input_embedder"])
        if c.template.enabled and hasattr(model.template_embedder, "template_single_embedder"):
            old = model.template_embedder
            new = mm.TemplateEmbedderMultimer.__new__(mm.TemplateEmbedderMultimer)
            nn.Module.__init__(new)
            new.config = old.config
            pe = mm.TemplatePairEmbedderMultimer.__new__(mm.TemplatePairEmbedderMultimer)
            nn.Module.__init__(pe)
            pe._modules.update(old.template_pair_embedder._modules)           # same parameter objects, lean forward
            new.template_pair_embedder = pe
            new.template_single_embedder = old.template_single_embedder
            new.template_pair_stack = old.template_pair_stack
            new.linear_t = old.linear_t
            new.train(old.training)
            model.template_embedder = new
    swap("recycling_embedder", RecyclingEmbedder, **c["recycling_embedder"])
    return model
