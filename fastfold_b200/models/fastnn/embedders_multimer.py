"""Lean embedders of the multimer model (roles of fastfold/model/fastnn/embedders_multimer.py:18-387).

Same parameters as ``models.nn.embedders_multimer`` (``inject_embedder`` moves the weights over), different evaluation:

* ``InputEmbedderMultimer``: the chain-aware relative-position term is a sum of three table lookups (rows of the
  ``linear_relpos`` weight selected by the integer bin indices) instead of a one-hot tensor of ``N x N x 73`` entries
  pushed through a linear layer - no ``[N, N, bins]`` tensor exists.
* ``TemplatePairEmbedderMultimer``: the rank-one terms (residue-type rows / columns, masks) are added as broadcasts and the
  unit-vector / mask channels through one stacked ``[N, N, 5] x [5, c]`` product instead of five 1-channel linears.
* ``TemplateEmbedderMultimer``: templates are embedded one at a time and accumulated in place (``.inplace`` of the fast
  template pair stack when ``inplace`` is set), so peak memory holds one template's pair activations.
"""
import torch
import torch.nn as nn

from ...common import residue_constants as rc
from ...utils.tensor_utils import const_like, tensor_tree_map
from ..nn import embedders_multimer as ref
from ..nn.embedders_multimer import _backbone_frames_and_mask, _one_hot, _template_pseudo_beta


class InputEmbedderMultimer(ref.InputEmbedderMultimer):
    def relpos(self, batch):
        pos, asym = batch["residue_index"], batch["asym_id"]
        w = self.linear_relpos.weight                      # [c_z, bins]
        wt = w.t()                                         # rows = bins
        same_chain = asym[..., None] == asym[..., None, :]
        offset = pos[..., None] - pos[..., None, :]
        clipped = torch.clamp(offset + self.max_relative_idx, 0, 2 * self.max_relative_idx)
        if not self.use_chain_relative:
            return wt[clipped] + self.linear_relpos.bias
        k = 2 * self.max_relative_idx + 2
        final = torch.where(same_chain, clipped, torch.full_like(clipped, 2 * self.max_relative_idx + 1))
        out = wt[final]                                    # one-hot over the first k bins
        entity = batch["entity_id"]
        same_entity = entity[..., None] == entity[..., None, :]
        out = out + same_entity[..., None].to(w.dtype) * wt[k]
        sym = batch["sym_id"]
        rel_sym = sym[..., None] - sym[..., None, :]
        clipped_chain = torch.clamp(rel_sym + self.max_relative_chain, 0, 2 * self.max_relative_chain)
        final_chain = torch.where(same_entity, clipped_chain, torch.full_like(clipped_chain, 2 * self.max_relative_chain + 1))
        out = out + wt[k + 1 + final_chain]
        return out + self.linear_relpos.bias


class TemplatePairEmbedderMultimer(ref.TemplatePairEmbedderMultimer):
    def forward(self, template_dgram, aatype_one_hot, query_embedding, pseudo_beta_mask, backbone_mask, multichain_mask_2d, unit_vector):
        pb2d = (pseudo_beta_mask[..., None] * pseudo_beta_mask[..., None, :]) * multichain_mask_2d
        bb2d = (backbone_mask[..., None] * backbone_mask[..., None, :]) * multichain_mask_2d
        act = self.dgram_linear(template_dgram * pb2d[..., None])
        act = act + self.query_embedding_linear(self.query_embedding_layer_norm(query_embedding))
        act = act + self.aatype_linear_1(aatype_one_hot)[..., None, :, :] + self.aatype_linear_2(aatype_one_hot)[..., None, :]
        # five single-channel linears as one [.., 5] x [5, c] product; their biases add up to one vector
        x, y, z = [u * bb2d for u in unit_vector]
        ch = torch.stack([pb2d, x, y, z, bb2d], dim=-1)
        w = torch.cat([self.pseudo_beta_mask_linear.weight, self.x_linear.weight, self.y_linear.weight, self.z_linear.weight,
                       self.backbone_mask_linear.weight], dim=-1)                       # [c, 5]
        b = (self.pseudo_beta_mask_linear.bias + self.x_linear.bias + self.y_linear.bias + self.z_linear.bias + self.backbone_mask_linear.bias)
        return act + torch.nn.functional.linear(ch.to(w.dtype), w, b)


class TemplateSingleEmbedderMultimer(ref.TemplateSingleEmbedderMultimer):
    pass


class TemplateEmbedderMultimer(ref.TemplateEmbedderMultimer):
    """Per-template loop with in-place accumulation of the pair embedding."""

    def forward(self, batch, z, padding_mask_2d, templ_dim, chunk_size, multichain_mask_2d, _mask_trans=True, inplace=False):
        n_templ = batch["template_aatype"].shape[templ_dim]
        dist = self.config.distogram
        acc = None
        for i in range(n_templ):
            idx = const_like(batch["template_aatype"], i, "templ_idx_%d" % i)
            single = tensor_tree_map(lambda t: torch.index_select(t, templ_dim, idx).squeeze(templ_dim), batch)
            pos = single["template_all_atom_positions"].float()
            msk = single["template_all_atom_mask"].float()
            pb, pb_mask = _template_pseudo_beta(single, pos, msk)
            d2 = torch.sum((pb[..., None, :] - pb[..., None, :, :]) ** 2, dim=-1, keepdim=True)
            lower = torch.linspace(dist["min_bin"], dist["max_bin"], dist["no_bins"], device=pos.device) ** 2
            upper = torch.cat([lower[1:], const_like(lower, [self.config.inf], "inf_%r" % (self.config.inf,))], dim=-1)
            dgram = ((d2 > lower) * (d2 < upper)).to(z.dtype)
            frames, bb_mask = _backbone_frames_and_mask(single["template_aatype"], pos, msk)
            ca = pos[..., rc.atom_order["CA"], :]
            vec = frames[..., None].invert_apply(ca[..., None, :, :])
            inv_norm = torch.rsqrt(self.config.eps + torch.sum(vec ** 2, dim=-1))
            unit = [(vec[..., k] * inv_norm).to(z.dtype) for k in range(3)]
            aatype_oh = _one_hot(single["template_aatype"], 22).to(z.dtype)
            pair_act = self.template_pair_embedder(dgram, aatype_oh, z, pb_mask.to(z.dtype), bb_mask.to(z.dtype), multichain_mask_2d.to(z.dtype), unit)
            del dgram, unit, vec, d2
            mask = padding_mask_2d.unsqueeze(-3).to(dtype=z.dtype)
            if inplace and hasattr(self.template_pair_stack, "inplace"):
                t = self.template_pair_stack.inplace([pair_act.unsqueeze(templ_dim)], mask, chunk_size=chunk_size, _mask_trans=_mask_trans)[0]
            else:
                t = self.template_pair_stack(pair_act.unsqueeze(templ_dim), mask, chunk_size=chunk_size, _mask_trans=_mask_trans)
            t = t.squeeze(templ_dim)
            del pair_act
            if acc is None:
                acc = t
            else:
                acc += t
            del t
        ret = {}
        if n_templ > 0:
            acc /= n_templ
            ret["template_pair_embedding"] = self.linear_t(torch.nn.functional.relu_(acc))
            aatype_oh_all = _one_hot(batch["template_aatype"], 22).to(z.dtype)
            ret.update(self.template_single_embedder(batch, batch["template_all_atom_positions"], aatype_oh_all))
        else:
            ret["template_pair_embedding"] = torch.zeros_like(z)
        return ret
