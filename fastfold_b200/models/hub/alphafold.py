"""The full AlphaFold 2 model (Algorithm 2): embedders, recycling, template / extra-MSA / Evoformer stacks,
structure module and auxiliary heads, in the OpenFold module layout.

``AlphaFold(config)(batch)``: every feature tensor carries the recycling dimension LAST (``[..., n_cycles]``) and has
no batch dimension.  The trunk stacks are plain ``models.nn`` modules here; ``inject_fastnn(model)`` swaps them for
the DAP-aware fast modules (``.inplace`` variants are used when ``config.globals.inplace``).  Gradients flow
through the last recycling iteration only; activation checkpointing is enabled for that iteration only.
Same contract and output keys as fastfold/model/hub/alphafold.py:173-534.
"""
import torch
import torch.nn as nn

from ...common import residue_constants as rc
from ...utils.feats import atom14_to_atom37, build_extra_msa_feat, pseudo_beta_fn
from ...utils.tensor_utils import tensor_tree_map
from ..nn.embedders import ExtraMSAEmbedder, InputEmbedder, RecyclingEmbedder, TemplateEmbedder
from ..nn.evoformer import EvoformerStack, ExtraMSAStack
from ..nn.heads import AuxiliaryHeads
from ..nn.structure_module import StructureModule


class AlphaFold(nn.Module):
    def __init__(self, config):
        super().__init__()
        self.globals = config.globals
        self.config = config.model
        c = self.config
        self.template_config = c.template
        self.extra_msa_config = c.extra_msa
        if self.globals.get("is_multimer", False):
            from ..nn.embedders_multimer import InputEmbedderMultimer, TemplateEmbedderMultimer
            self.input_embedder = InputEmbedderMultimer(**c["input_embedder"])
            self.template_embedder = TemplateEmbedderMultimer(c.template)
        else:
            self.input_embedder = InputEmbedder(**c["input_embedder"])
            self.template_embedder = TemplateEmbedder(c.template)
        self.recycling_embedder = RecyclingEmbedder(**c["recycling_embedder"])
        self.extra_msa_embedder = ExtraMSAEmbedder(**c.extra_msa["extra_msa_embedder"])
        self.extra_msa_stack = ExtraMSAStack(is_multimer=self.globals.get("is_multimer", False), **c.extra_msa["extra_msa_stack"])
        self.evoformer = EvoformerStack(is_multimer=self.globals.get("is_multimer", False), **c["evoformer_stack"])
        self.structure_module = StructureModule(is_multimer=self.globals.get("is_multimer", False), **c["structure_module"])
        self.aux_heads = AuxiliaryHeads(c["heads"])

    # ------------------------------------------------------------------
    def iteration(self, feats, m_1_prev, z_prev, x_prev, _recycle=True):
        outputs = {}
        dtype = next(self.parameters()).dtype
        for k in feats:
            if feats[k].dtype == torch.float32:
                feats[k] = feats[k].to(dtype=dtype)
        batch_dims = feats["target_feat"].shape[:-2]
        n = feats["target_feat"].shape[-2]
        n_seq = feats["msa_feat"].shape[-3]
        device = feats["target_feat"].device
        seq_mask = feats["seq_mask"]
        pair_mask = seq_mask[..., None] * seq_mask[..., None, :]
        msa_mask = feats["msa_mask"]
        inplace = bool(self.globals.get("inplace", False)) and not (self.training or torch.is_grad_enabled())

        is_multimer = bool(self.globals.get("is_multimer", False))
        # Long sequences under DAP (``globals.shard_pair``): the pair tensor exists only as this rank's row shard
        # [N/P, N, c_z] from the embedders to the heads - the stacks neither scatter nor gather it, the structure module
        # attends row-parallel, recycling and the distogram head work on the shard.  Outputs ``pair`` and
        # ``distogram_logits`` are then row shards too.
        from ...parallel import core as _core
        P = _core.get_dap_size()
        shard = (bool(self.globals.get("shard_pair", False)) and P > 1 and n % P == 0 and not is_multimer and not self.config.template.enabled
                 and not torch.is_grad_enabled() and not batch_dims and hasattr(self.evoformer.blocks[-1], "keep_pair_sharded"))
        for stack in (self.evoformer, self.extra_msa_stack):
            if hasattr(stack.blocks[-1], "keep_pair_sharded"):
                stack.blocks[-1].keep_pair_sharded = shard
        row0 = _core.get_dap_rank() * (n // P) if shard else 0
        if is_multimer:
            m, z = self.input_embedder(feats)
        elif shard:
            m, z = self.input_embedder(feats["target_feat"], feats["residue_index"], feats["msa_feat"], rows=(row0, row0 + n // P))
        else:
            m, z = self.input_embedder(feats["target_feat"], feats["residue_index"], feats["msa_feat"])
        if None in [m_1_prev, z_prev, x_prev]:
            m_1_prev = m.new_zeros((*batch_dims, n, self.config.input_embedder.c_m), requires_grad=False)
            z_prev = z.new_zeros(z.shape, requires_grad=False)
            x_prev = z.new_zeros((*batch_dims, n, rc.atom_type_num, 3), requires_grad=False)
        x_prev = pseudo_beta_fn(feats["aatype"], x_prev, None)[0].to(dtype=z.dtype)
        if shard:
            m_1_prev_emb, z_prev_emb = self.recycling_embedder(m_1_prev, z_prev, x_prev, row0=row0)
        else:
            m_1_prev_emb, z_prev_emb = self.recycling_embedder(m_1_prev, z_prev, x_prev)
        if not _recycle:
            m_1_prev_emb = m_1_prev_emb * 0
            z_prev_emb = z_prev_emb * 0
        m = torch.cat([(m[..., 0, :, :] + m_1_prev_emb).unsqueeze(-3), m[..., 1:, :, :]], dim=-3)
        z = z + z_prev_emb
        del m_1_prev, z_prev, x_prev, m_1_prev_emb, z_prev_emb

        if self.config.template.enabled and is_multimer:
            template_feats = {k: v for k, v in feats.items() if k.startswith("template_")}
            asym = feats["asym_id"]
            multichain_mask_2d = asym[..., None] == asym[..., None, :]
            template_embeds = self.template_embedder(template_feats, z, pair_mask.to(dtype=z.dtype), len(batch_dims), self.globals.chunk_size,
                                                     multichain_mask_2d=multichain_mask_2d, inplace=inplace)
            z = z + template_embeds["template_pair_embedding"]
            if "template_single_embedding" in template_embeds:
                m = torch.cat([m, template_embeds["template_single_embedding"].to(m.dtype)], dim=-3)
                msa_mask = torch.cat([feats["msa_mask"], template_embeds["template_mask"].to(feats["msa_mask"].dtype)], dim=-2)
            del template_feats, template_embeds
        elif self.config.template.enabled:
            template_feats = {k: v for k, v in feats.items() if k.startswith("template_")}
            template_embeds = self.template_embedder(template_feats, z, pair_mask.to(dtype=z.dtype), len(batch_dims),
                                                     self.globals.chunk_size)
            z = z + template_embeds["template_pair_embedding"]
            if self.config.template.embed_angles:
                m = torch.cat([m, template_embeds["template_angle_embedding"]], dim=-3)
                torsion_angles_mask = feats["template_torsion_angles_mask"]
                msa_mask = torch.cat([feats["msa_mask"], torsion_angles_mask[..., 2]], dim=-2)
            del template_feats, template_embeds

        if self.config.extra_msa.enabled:
            a = self.extra_msa_embedder(build_extra_msa_feat(feats).to(dtype=z.dtype))
            extra_mask = feats["extra_msa_mask"].to(dtype=z.dtype)
            if inplace and hasattr(self.extra_msa_stack, "inplace"):
                zl = [z]
                del z
                zl = self.extra_msa_stack.inplace([a], zl, msa_mask=extra_mask, chunk_size=self.globals.chunk_size,
                                                  pair_mask=pair_mask.to(dtype=zl[0].dtype), _mask_trans=self.config._mask_trans)
                z = zl[0]
                del zl
            else:
                z = self.extra_msa_stack(a, z, msa_mask=extra_mask, chunk_size=self.globals.chunk_size,
                                         pair_mask=pair_mask.to(dtype=z.dtype), _mask_trans=self.config._mask_trans)
            del a

        if inplace and hasattr(self.evoformer, "inplace"):
            ml, zl = [m], [z]
            del m, z
            ml, zl, s = self.evoformer.inplace(ml, zl, msa_mask=msa_mask.to(dtype=ml[0].dtype), pair_mask=pair_mask.to(dtype=zl[0].dtype),
                                               chunk_size=self.globals.chunk_size, _mask_trans=self.config._mask_trans)
            m, z = ml[0], zl[0]
            del ml, zl
        else:
            m, z, s = self.evoformer(m, z, msa_mask=msa_mask.to(dtype=m.dtype), pair_mask=pair_mask.to(dtype=z.dtype),
                                     chunk_size=self.globals.chunk_size, _mask_trans=self.config._mask_trans)

        outputs["msa"] = m[..., :n_seq, :, :]
        outputs["pair"] = z
        outputs["single"] = s
        outputs["sm"] = self.structure_module(s, z, feats["aatype"], mask=feats["seq_mask"].to(dtype=s.dtype))
        outputs["final_atom_positions"] = atom14_to_atom37(outputs["sm"]["positions"][-1], feats)
        outputs["final_atom_mask"] = feats["atom37_atom_exists"]
        outputs["final_affine_tensor"] = outputs["sm"]["frames"][-1]
        m_1_prev = m[..., 0, :, :]
        z_prev = z
        x_prev = outputs["final_atom_positions"]
        return outputs, m_1_prev, z_prev, x_prev

    def embed_templates(self, batch, z, pair_mask, templ_dim):
        """Template embeddings for ``batch`` (the ``template_*`` features): ``{"template_pair_embedding": [*, N, N, c_z],
        "template_angle_embedding": ...}``.  The work is done by ``self.template_embedder`` (OpenFold-layout or, after
        ``inject_fastnn``, the fast one); the method keeps the entry point of fastfold/model/hub/alphafold.py:107-171."""
        return self.template_embedder(batch, z, pair_mask, templ_dim, self.globals.chunk_size)

    def _set_ckpt(self, enabled):
        bpc = self.globals.blocks_per_ckpt if enabled else None
        for mod in (self.template_embedder.template_pair_stack if hasattr(self.template_embedder, "template_pair_stack") else None, self.evoformer):
            if mod is not None:
                mod.blocks_per_ckpt = bpc

    def forward(self, batch):
        m_1_prev, z_prev, x_prev = None, None, None
        self._set_ckpt(False)
        is_grad_enabled = torch.is_grad_enabled()
        num_iters = batch["aatype"].shape[-1]
        for cycle_no in range(num_iters):
            feats = tensor_tree_map(lambda t: t[..., cycle_no], batch)
            is_final_iter = cycle_no == (num_iters - 1)
            with torch.set_grad_enabled(is_grad_enabled and is_final_iter):
                if is_final_iter:
                    self._set_ckpt(True)
                    if torch.is_autocast_enabled():
                        torch.clear_autocast_cache()
                outputs, m_1_prev, z_prev, x_prev = self.iteration(feats, m_1_prev, z_prev, x_prev, _recycle=(num_iters > 1))
        outputs.update(self.aux_heads(outputs))
        return outputs
