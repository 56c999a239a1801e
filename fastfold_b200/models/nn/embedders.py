"""Input, recycling, template and extra-MSA embedders in the OpenFold parameter layout.

Same roles as fastfold/model/nn/embedders.py (InputEmbedder, RecyclingEmbedder, Template{Angle,Pair}Embedder,
ExtraMSAEmbedder) and the template embedder wrapper of fastfold/model/nn/template.py.
"""
from functools import partial

import torch
import torch.nn as nn

from ...utils.feats import build_template_angle_feat, build_template_pair_feat
from ...utils.tensor_utils import const_like, dict_multimap, one_hot, tensor_tree_map
from .primitives import LayerNorm, Linear
from .template import TemplatePairStack, TemplatePointwiseAttention


class InputEmbedder(nn.Module):
    """Algorithm 3 + relative position encoding (Algorithm 4)."""

    def __init__(self, tf_dim, msa_dim, c_z, c_m, relpos_k, **kwargs):
        super().__init__()
        self.tf_dim, self.msa_dim, self.c_z, self.c_m, self.relpos_k = tf_dim, msa_dim, c_z, c_m, relpos_k
        self.linear_tf_z_i = Linear(tf_dim, c_z)
        self.linear_tf_z_j = Linear(tf_dim, c_z)
        self.linear_tf_m = Linear(tf_dim, c_m)
        self.linear_msa_m = Linear(msa_dim, c_m)
        self.no_bins = 2 * relpos_k + 1
        self.linear_relpos = Linear(self.no_bins, c_z)

    def relpos(self, ri):
        d = ri[..., None] - ri[..., None, :]
        boundaries = torch.arange(start=-self.relpos_k, end=self.relpos_k + 1, device=d.device)
        oh = one_hot(d, boundaries).type(ri.dtype)
        return self.linear_relpos(oh)

    def forward(self, tf, ri, msa):
        tf_emb_i = self.linear_tf_z_i(tf)
        tf_emb_j = self.linear_tf_z_j(tf)
        pair_emb = self.relpos(ri.type(tf_emb_i.dtype)) + tf_emb_i[..., None, :] + tf_emb_j[..., None, :, :]
        n_clust = msa.shape[-3]
        tf_m = self.linear_tf_m(tf).unsqueeze(-3).expand(((-1,) * len(tf.shape[:-2]) + (n_clust, -1, -1)))
        return self.linear_msa_m(msa) + tf_m, pair_emb


class RecyclingEmbedder(nn.Module):
    """Algorithm 32: LayerNorm of the recycled first MSA row and pair representation + distogram of recycled CB positions."""

    def __init__(self, c_m, c_z, min_bin, max_bin, no_bins, inf=1e8, **kwargs):
        super().__init__()
        self.c_m, self.c_z, self.min_bin, self.max_bin, self.no_bins, self.inf = c_m, c_z, min_bin, max_bin, no_bins, inf
        self.linear = Linear(no_bins, c_z)
        self.layer_norm_m = LayerNorm(c_m)
        self.layer_norm_z = LayerNorm(c_z)

    def forward(self, m, z, x):
        bins = torch.linspace(self.min_bin, self.max_bin, self.no_bins, dtype=x.dtype, device=x.device, requires_grad=False)
        m_update = self.layer_norm_m(m)
        squared_bins = bins ** 2
        upper = torch.cat([squared_bins[1:], const_like(squared_bins, [self.inf], "inf_%r" % (self.inf,))], dim=-1)
        d = torch.sum((x[..., None, :] - x[..., None, :, :]) ** 2, dim=-1, keepdims=True)
        d = ((d > squared_bins) * (d < upper)).type(x.dtype)
        z_update = self.linear(d.to(z.dtype)) + self.layer_norm_z(z)
        return m_update, z_update


class TemplateAngleEmbedder(nn.Module):
    def __init__(self, c_in, c_out, **kwargs):
        super().__init__()
        self.linear_1 = Linear(c_in, c_out, init="relu")
        self.relu = nn.ReLU()
        self.linear_2 = Linear(c_out, c_out, init="relu")

    def forward(self, x):
        return self.linear_2(self.relu(self.linear_1(x)))


class TemplatePairEmbedder(nn.Module):
    def __init__(self, c_in, c_out, **kwargs):
        super().__init__()
        self.linear = Linear(c_in, c_out, init="relu")

    def forward(self, x):
        return self.linear(x)


class ExtraMSAEmbedder(nn.Module):
    def __init__(self, c_in, c_out, **kwargs):
        super().__init__()
        self.linear = Linear(c_in, c_out)

    def forward(self, x):
        return self.linear(x)


class TemplateEmbedder(nn.Module):
    """Embeds every template's pair features through the template pair stack and attends over templates (Algorithm 2,
    lines 7-13); also returns the template angle embedding that is appended to the MSA."""

    def __init__(self, config):
        super().__init__()
        self.config = config
        self.template_angle_embedder = TemplateAngleEmbedder(**config["template_angle_embedder"])
        self.template_pair_embedder = TemplatePairEmbedder(**config["template_pair_embedder"])
        self.template_pair_stack = TemplatePairStack(**config["template_pair_stack"])
        self.template_pointwise_att = TemplatePointwiseAttention(**config["template_pointwise_attention"])

    def forward(self, batch, z, pair_mask, templ_dim, chunk_size, _mask_trans=True, inplace=False):
        template_embeds = []
        n_templ = batch["template_aatype"].shape[templ_dim]
        for i in range(n_templ):
            idx = const_like(batch["template_aatype"], i, "templ_idx_%d" % i)
            single = tensor_tree_map(lambda t: torch.index_select(t, templ_dim, idx), batch)
            emb = {}
            if self.config.embed_angles:
                emb["angle"] = self.template_angle_embedder(build_template_angle_feat(single))
            t = build_template_pair_feat(single, use_unit_vector=self.config.use_unit_vector, inf=self.config.inf, eps=self.config.eps,
                                         **self.config.distogram).to(z.dtype)
            emb["pair"] = self.template_pair_embedder(t)
            template_embeds.append(emb)
        template_embeds = dict_multimap(partial(torch.cat, dim=templ_dim), template_embeds)
        t = self.template_pair_stack(template_embeds["pair"], pair_mask.unsqueeze(-3).to(dtype=z.dtype), chunk_size=chunk_size,
                                     _mask_trans=_mask_trans)
        t = self.template_pointwise_att(t, z, template_mask=batch["template_mask"].to(dtype=z.dtype), chunk_size=chunk_size)
        t = t * (torch.sum(batch["template_mask"]) > 0)
        ret = {}
        if self.config.embed_angles:
            ret["template_angle_embedding"] = template_embeds["angle"]
        ret["template_pair_embedding"] = t
        return ret
