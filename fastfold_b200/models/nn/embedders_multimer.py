"""Embedders of the multimer model (AlphaFold-Multimer): chain-aware relative position encoding, and template
embedding from distances + backbone-frame unit vectors instead of the monomer model's 88-channel feature.

Same roles and parameter names as fastfold/model/nn/embedders_multimer.py (InputEmbedderMultimer :18-155,
TemplatePairEmbedderMultimer :158-235, TemplateSingleEmbedderMultimer :238-290, TemplateEmbedderMultimer :293-376).
The reference routes the geometry through struct-of-arrays classes (utils/geometry); here it is plain tensor code on
the monomer ``Rigid`` utilities, which gives the same numbers.
"""
import torch
import torch.nn as nn

from ...common import residue_constants as rc
from ...utils.rigid_utils import Rigid
from ...utils.tensor_utils import const_like, tensor_tree_map
from .primitives import LayerNorm, Linear
from .template import TemplatePairStack


def _one_hot(x, n):
    return torch.nn.functional.one_hot(x.long(), n)


class InputEmbedderMultimer(nn.Module):
    """Target-feature / MSA embedding with relative position features that know about chains: residues of different
    chains share one "other chain" bin, and the relative chain index (``sym_id``) of identical entities is encoded too."""

    def __init__(self, tf_dim, msa_dim, c_z, c_m, max_relative_idx, use_chain_relative, max_relative_chain, **kwargs):
        super().__init__()
        self.tf_dim, self.msa_dim, self.c_z, self.c_m = tf_dim, msa_dim, c_z, c_m
        self.linear_tf_z_i = Linear(tf_dim, c_z)
        self.linear_tf_z_j = Linear(tf_dim, c_z)
        self.linear_tf_m = Linear(tf_dim, c_m)
        self.linear_msa_m = Linear(msa_dim, c_m)
        self.max_relative_idx, self.use_chain_relative, self.max_relative_chain = max_relative_idx, use_chain_relative, max_relative_chain
        if use_chain_relative:
            self.no_bins = 2 * max_relative_idx + 2 + 1 + 2 * max_relative_chain + 2
        else:
            self.no_bins = 2 * max_relative_idx + 1
        self.linear_relpos = Linear(self.no_bins, c_z)

    def relpos(self, batch):
        pos = batch["residue_index"]
        asym = batch["asym_id"]
        same_chain = asym[..., None] == asym[..., None, :]
        offset = pos[..., None] - pos[..., None, :]
        clipped = torch.clamp(offset + self.max_relative_idx, 0, 2 * self.max_relative_idx)
        feats = []
        if self.use_chain_relative:
            final = torch.where(same_chain, clipped, (2 * self.max_relative_idx + 1) * torch.ones_like(clipped))
            feats.append(_one_hot(final, 2 * self.max_relative_idx + 2))
            entity = batch["entity_id"]
            same_entity = entity[..., None] == entity[..., None, :]
            feats.append(same_entity[..., None].to(feats[0].dtype))
            sym = batch["sym_id"]
            rel_sym = sym[..., None] - sym[..., None, :]
            clipped_chain = torch.clamp(rel_sym + self.max_relative_chain, 0, 2 * self.max_relative_chain)
            final_chain = torch.where(same_entity, clipped_chain, (2 * self.max_relative_chain + 1) * torch.ones_like(clipped_chain))
            feats.append(_one_hot(final_chain, 2 * self.max_relative_chain + 2))
        else:
            feats.append(_one_hot(clipped, 2 * self.max_relative_idx + 1))
        rel = torch.cat(feats, dim=-1).to(self.linear_relpos.weight.dtype)
        return self.linear_relpos(rel)

    def forward(self, batch):
        tf, msa = batch["target_feat"], batch["msa_feat"]
        tf = tf.to(self.linear_tf_m.weight.dtype)
        tf_emb_i = self.linear_tf_z_i(tf)
        tf_emb_j = self.linear_tf_z_j(tf)
        pair_emb = tf_emb_i[..., None, :] + tf_emb_j[..., None, :, :] + self.relpos(batch)
        n_clust = msa.shape[-3]
        tf_m = self.linear_tf_m(tf).unsqueeze(-3).expand(((-1,) * len(tf.shape[:-2]) + (n_clust, -1, -1)))
        return self.linear_msa_m(msa.to(tf.dtype)) + tf_m, pair_emb


class TemplatePairEmbedderMultimer(nn.Module):
    def __init__(self, c_z, c_out, c_dgram, c_aatype, **kwargs):
        super().__init__()
        self.dgram_linear = Linear(c_dgram, c_out)
        self.aatype_linear_1 = Linear(c_aatype, c_out)
        self.aatype_linear_2 = Linear(c_aatype, c_out)
        self.query_embedding_layer_norm = LayerNorm(c_z)
        self.query_embedding_linear = Linear(c_z, c_out)
        self.pseudo_beta_mask_linear = Linear(1, c_out)
        self.x_linear = Linear(1, c_out)
        self.y_linear = Linear(1, c_out)
        self.z_linear = Linear(1, c_out)
        self.backbone_mask_linear = Linear(1, c_out)

    def forward(self, template_dgram, aatype_one_hot, query_embedding, pseudo_beta_mask, backbone_mask, multichain_mask_2d, unit_vector):
        act = 0.0
        pb2d = (pseudo_beta_mask[..., None] * pseudo_beta_mask[..., None, :]) * multichain_mask_2d
        act = act + self.dgram_linear(template_dgram * pb2d[..., None])
        act = act + self.pseudo_beta_mask_linear(pb2d[..., None])
        act = act + self.aatype_linear_1(aatype_one_hot)[..., None, :, :]
        act = act + self.aatype_linear_2(aatype_one_hot)[..., None, :]
        bb2d = (backbone_mask[..., None] * backbone_mask[..., None, :]) * multichain_mask_2d
        x, y, z = [u * bb2d for u in unit_vector]
        act = act + self.x_linear(x[..., None])
        act = act + self.y_linear(y[..., None])
        act = act + self.z_linear(z[..., None])
        act = act + self.backbone_mask_linear(bb2d[..., None])
        act = act + self.query_embedding_linear(self.query_embedding_layer_norm(query_embedding))
        return act


class TemplateSingleEmbedderMultimer(nn.Module):
    """Per-residue template features (aatype one-hot + chi angles) -> extra MSA rows."""

    def __init__(self, c_in, c_m, **kwargs):
        super().__init__()
        self.template_single_embedder = Linear(c_in, c_m)
        self.template_projector = Linear(c_m, c_m)

    def forward(self, batch, atom_pos, aatype_one_hot):
        from ...data import data_transforms as dt
        out = {}
        n_templ = batch["template_aatype"].shape[-2]
        feats, masks = [], []
        for i in range(n_templ):
            prot = {"aatype": batch["template_aatype"][..., i, :], "all_atom_positions": atom_pos[..., i, :, :, :].float(),
                    "all_atom_mask": batch["template_all_atom_mask"][..., i, :, :].float()}
            prot = dt.atom37_to_torsion_angles("")(prot)
            sin_cos = prot["torsion_angles_sin_cos"][..., 3:, :]            # the four chi angles
            chi_mask = prot["torsion_angles_mask"][..., 3:]
            f = torch.cat([aatype_one_hot[..., i, :, :], sin_cos[..., 0] * chi_mask, sin_cos[..., 1] * chi_mask, chi_mask], dim=-1)
            feats.append(f)
            masks.append(chi_mask[..., 0])
        feat = torch.stack(feats, dim=-3).to(self.template_single_embedder.weight.dtype)
        mask = torch.stack(masks, dim=-2).to(feat.dtype)
        act = self.template_single_embedder(feat)
        act = torch.nn.functional.relu(act)
        out["template_single_embedding"] = self.template_projector(act)
        out["template_mask"] = mask
        return out


def _backbone_frames_and_mask(aatype, all_atom_positions, all_atom_mask):
    """Backbone frames in the multimer convention - origin CA, C on the POSITIVE x axis, N in the xy plane with y > 0
    (fastfold/utils/all_atom_multimer.py:447-493) - which is the monomer frame turned by 180 degrees about y.  Written
    through ``from_3_points``, whose first argument lies on the negative x axis: the mirror image of C through CA."""
    n, ca, c = (rc.atom_order[a] for a in ("N", "CA", "C"))
    origin = all_atom_positions[..., ca, :]
    frames = Rigid.from_3_points(p_neg_x_axis=2.0 * origin - all_atom_positions[..., c, :], origin=origin,
                                 p_xy_plane=all_atom_positions[..., n, :], eps=1e-8)
    mask = all_atom_mask[..., n] * all_atom_mask[..., ca] * all_atom_mask[..., c]
    return frames, mask


def _template_pseudo_beta(single, positions, masks):
    """The pseudo-beta atoms the data pipeline stored with the template (``make_pseudo_beta("template_")``), else computed."""
    if "template_pseudo_beta" in single and "template_pseudo_beta_mask" in single:
        return single["template_pseudo_beta"].float(), single["template_pseudo_beta_mask"].float()
    return _pseudo_beta(single["template_aatype"], positions, masks)


def _pseudo_beta(aatype, positions, masks):
    is_gly = aatype == rc.restype_order["G"]
    ca, cb = rc.atom_order["CA"], rc.atom_order["CB"]
    pb = torch.where(is_gly[..., None].expand(*((-1,) * len(is_gly.shape)), 3), positions[..., ca, :], positions[..., cb, :])
    pm = torch.where(is_gly, masks[..., ca], masks[..., cb])
    return pb, pm


class TemplateEmbedderMultimer(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.config = config
        self.template_pair_embedder = TemplatePairEmbedderMultimer(**config["template_pair_embedder"])
        self.template_single_embedder = TemplateSingleEmbedderMultimer(**config["template_single_embedder"])
        self.template_pair_stack = TemplatePairStack(**config["template_pair_stack"])
        self.linear_t = Linear(config.c_t, config.c_z)

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
            upper = torch.cat([lower[1:], lower.new_tensor([self.config.inf])], dim=-1)
            dgram = ((d2 > lower) * (d2 < upper)).to(z.dtype)
            frames, bb_mask = _backbone_frames_and_mask(single["template_aatype"], pos, msk)
            ca = pos[..., rc.atom_order["CA"], :]
            vec = frames[..., None].invert_apply(ca[..., None, :, :])             # CA_j in the frame of residue i
            inv_norm = torch.rsqrt(self.config.eps + torch.sum(vec ** 2, dim=-1))
            unit = [(vec[..., k] * inv_norm).to(z.dtype) for k in range(3)]
            aatype_oh = _one_hot(single["template_aatype"], 22).to(z.dtype)
            pair_act = self.template_pair_embedder(dgram, aatype_oh, z, pb_mask.to(z.dtype), bb_mask.to(z.dtype),
                                                   multichain_mask_2d.to(z.dtype), unit)
            t = self.template_pair_stack(pair_act.unsqueeze(templ_dim), padding_mask_2d.unsqueeze(-3).to(dtype=z.dtype), chunk_size=chunk_size,
                                         _mask_trans=_mask_trans).squeeze(templ_dim)
            acc = t if acc is None else acc + t
        ret = {}
        if n_templ > 0:
            t = acc / n_templ
            ret["template_pair_embedding"] = self.linear_t(torch.nn.functional.relu(t))
        else:
            ret["template_pair_embedding"] = torch.zeros_like(z)
        if n_templ > 0:
            aatype_oh_all = _one_hot(batch["template_aatype"], 22).to(z.dtype)
            ret.update(self.template_single_embedder(batch, batch["template_all_atom_positions"], aatype_oh_all))
        return ret
