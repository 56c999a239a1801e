"""Swap the trunk stacks of an OpenFold-layout ``AlphaFold`` for the fast, DAP-aware modules.

``inject_fastnn(model)`` replaces ``model.evoformer`` and ``model.extra_msa_stack`` by ``models.fastnn`` stacks
built from the same weights - q/k/v fused into ``to_qkv``, the two triangle-multiplication projections (and gates)
fused into ``left_right_projection`` (``left_right_gate``), output-projection biases moved next to the fused
bias-dropout-add - and keeps each block's train / eval mode.  ``extract_fastnn`` is the inverse (fast stack ->
OpenFold-named ``state_dict`` entries), so checkpoints written from an injected model round-trip to the
OpenFold / AlphaFold-archive naming.  Input, recycling and template embedders stay the ``models.nn`` modules (they
are mathematically identical and replicated over DAP ranks).  Same role and name map as
fastfold/utils/inject_fastnn.py:24-152, 321-423.
"""
import torch

from ..models.fastnn import EvoformerStack as FastEvoformerStack
from ..models.fastnn import ExtraMSAStack as FastExtraMSAStack


def _cp(dst, src):
    with torch.no_grad():
        dst.copy_(src.to(dst.dtype))


def _copy_layernorm(fast, ori):
    _cp(fast.weight, ori.weight)
    _cp(fast.bias, ori.bias)


def _copy_linear(fast, ori):
    _cp(fast.weight, ori.weight)
    if getattr(fast, "bias", None) is not None and getattr(ori, "bias", None) is not None:
        _cp(fast.bias, ori.bias)


def _copy_attention(fast, ori, out_bias=None):
    """``ori``: nn.primitives.Attention; ``fast``: fastnn SelfAttention (+ module-level ``out_bias`` when fused)."""
    _cp(fast.to_qkv.weight, torch.cat([ori.linear_q.weight, ori.linear_k.weight, ori.linear_v.weight], dim=0))
    _cp(fast.gating_linear.weight, ori.linear_g.weight)
    _cp(fast.gating_bias, ori.linear_g.bias)
    _cp(fast.o_linear.weight, ori.linear_o.weight)
    if out_bias is not None:
        _cp(out_bias, ori.linear_o.bias)
    else:
        _cp(fast.o_linear.bias, ori.linear_o.bias)


def _copy_global_attention(fast, ori):
    _cp(fast.to_q.weight, ori.linear_q.weight)
    _cp(fast.to_kv.weight, torch.cat([ori.linear_k.weight, ori.linear_v.weight], dim=0))
    _cp(fast.gating_linear.weight, ori.linear_g.weight)
    _cp(fast.gating_bias, ori.linear_g.bias)
    _copy_linear(fast.o_linear, ori.linear_o)


def _copy_transition(fast, ori):
    _copy_layernorm(fast.norm, ori.layer_norm)
    _copy_linear(fast.linear1, ori.linear_1)
    _copy_linear(fast.linear2, ori.linear_2)


def _copy_tri_mul(fast, ori):
    _copy_layernorm(fast.layernorm1, ori.layer_norm_in)
    _copy_layernorm(fast.layernorm2, ori.layer_norm_out)
    if getattr(ori, "fused", False):
        _copy_linear(fast.left_right_projection, ori.linear_p)
        _copy_linear(fast.left_right_gate, ori.linear_g)
        _copy_linear(fast.output_gate, ori.linear_gate)
    else:
        _cp(fast.left_right_projection.weight, torch.cat([ori.linear_a_p.weight, ori.linear_b_p.weight], dim=0))
        _cp(fast.left_right_projection.bias, torch.cat([ori.linear_a_p.bias, ori.linear_b_p.bias], dim=0))
        _cp(fast.left_right_gate.weight, torch.cat([ori.linear_a_g.weight, ori.linear_b_g.weight], dim=0))
        _cp(fast.left_right_gate.bias, torch.cat([ori.linear_a_g.bias, ori.linear_b_g.bias], dim=0))
        _copy_linear(fast.output_gate, ori.linear_g)
    _cp(fast.output_projection.weight, ori.linear_z.weight)
    _cp(fast.output_bias, ori.linear_z.bias)
    fast._glu_cache = None


def _copy_tri_att(fast, ori):
    _copy_layernorm(fast.layernorm1, ori.layer_norm)
    _cp(fast.linear_b.weight, ori.linear.weight)
    _copy_attention(fast.attention, ori.mha, out_bias=fast.out_bias)


def _copy_core(fast_opm, fast_pair, fast_msa_transition, core):
    _copy_transition(fast_msa_transition, core.msa_transition)
    _copy_layernorm(fast_opm.layernormM, core.outer_product_mean.layer_norm)
    _copy_linear(fast_opm.linear_a, core.outer_product_mean.linear_1)
    _copy_linear(fast_opm.linear_b, core.outer_product_mean.linear_2)
    _copy_linear(fast_opm.o_linear, core.outer_product_mean.linear_out)
    _copy_tri_mul(fast_pair.TriangleMultiplicationOutgoing, core.tri_mul_out)
    _copy_tri_mul(fast_pair.TriangleMultiplicationIncoming, core.tri_mul_in)
    _copy_tri_att(fast_pair.TriangleAttentionStartingNode, core.tri_att_start)
    _copy_tri_att(fast_pair.TriangleAttentionEndingNode, core.tri_att_end)
    _copy_transition(fast_pair.PairTransition, core.pair_transition)


def _copy_row_attention(fast, ori):
    _copy_layernorm(fast.layernormM, ori.layer_norm_m)
    _copy_layernorm(fast.layernormZ, ori.layer_norm_z)
    _cp(fast.linear_b_weights, ori.linear_z.weight)
    _copy_attention(fast.attention, ori.mha, out_bias=fast.out_bias)


def copy_evoformer_block(fast, ori):
    _copy_row_attention(fast.msa.MSARowAttentionWithPairBias, ori.msa_att_row)
    _copy_layernorm(fast.msa.MSAColumnAttention.layernormM, ori.msa_att_col._msa_att.layer_norm_m)
    _copy_attention(fast.msa.MSAColumnAttention.attention, ori.msa_att_col._msa_att.mha)
    _copy_core(fast.communication, fast.pair, fast.msa.MSATransition, ori.core)


def copy_extra_msa_block(fast, ori):
    _copy_row_attention(fast.msa_stack.MSARowAttentionWithPairBias, ori.msa_att_row)
    _copy_layernorm(fast.msa_stack.MSAColumnAttention.layernormM, ori.msa_att_col.layer_norm_m)
    _copy_global_attention(fast.msa_stack.MSAColumnAttention.global_attention, ori.msa_att_col.global_attention)
    _copy_core(fast.communication, fast.pair_stack, fast.msa_stack.MSATransition, ori.core)


def _like(module, ref_module):
    p = next(ref_module.parameters())
    return module.to(device=p.device, dtype=p.dtype)


def inject_evoformer(model):
    ori = model.evoformer
    cfg = model.config.evoformer_stack
    fast = FastEvoformerStack(c_m=cfg.c_m, c_z=cfg.c_z, c_s=cfg.c_s, no_blocks=len(ori.blocks), blocks_per_ckpt=ori.blocks_per_ckpt,
                              clear_cache_between_blocks=False, is_multimer=bool(model.globals.get("is_multimer", False)))
    fast = _like(fast, ori)
    for fb, ob in zip(fast.blocks, ori.blocks):
        copy_evoformer_block(fb, ob)
        fb.train(ob.training)
    _copy_linear(fast.linear, ori.linear)
    fast.train(ori.training)
    model.evoformer = fast


def inject_extra_msa(model):
    ori = model.extra_msa_stack
    cfg = model.config.extra_msa.extra_msa_stack
    fast = FastExtraMSAStack(c_m=cfg.c_m, c_z=cfg.c_z, no_blocks=len(ori.blocks), clear_cache_between_blocks=False,
                             is_multimer=bool(model.globals.get("is_multimer", False)))
    fast = _like(fast, ori)
    for fb, ob in zip(fast.blocks, ori.blocks):
        copy_extra_msa_block(fb, ob)
        fb.train(ob.training)
    fast.train(ori.training)
    model.extra_msa_stack = fast


inject_extramsa = inject_extra_msa          # the reference's spelling (fastfold/utils/inject_fastnn.py:341)


def copy_template_pair_block(fast, ori):
    _copy_tri_att(fast.TriangleAttentionStartingNode, ori.tri_att_start)
    _copy_tri_att(fast.TriangleAttentionEndingNode, ori.tri_att_end)
    _copy_tri_mul(fast.TriangleMultiplicationOutgoing, ori.tri_mul_out)
    _copy_tri_mul(fast.TriangleMultiplicationIncoming, ori.tri_mul_in)
    _copy_transition(fast.PairTransition, ori.pair_transition)


def inject_template(model):
    """Swaps the template pair stack (and the pointwise attention wrapper) of the template embedder
    (fastfold/utils/inject_fastnn.py:356-388)."""
    from ..models.fastnn.template import TemplatePairStack as FastTemplatePairStack, TemplatePointwiseAttention as FastPointwise
    emb = model.template_embedder
    ori = emb.template_pair_stack
    cfg = model.config.template.template_pair_stack
    fast = FastTemplatePairStack(c_t=cfg.c_t, c_hidden_tri_att=cfg.c_hidden_tri_att, c_hidden_tri_mul=cfg.c_hidden_tri_mul,
                                 no_blocks=len(ori.blocks), no_heads=cfg.no_heads, pair_transition_n=cfg.pair_transition_n,
                                 dropout_rate=cfg.dropout_rate, blocks_per_ckpt=ori.blocks_per_ckpt, inf=cfg.get("inf", 1e9),
                                 tri_mul_first=bool(cfg.get("tri_mul_first", False)))
    fast = _like(fast, ori)
    for fb, ob in zip(fast.blocks, ori.blocks):
        copy_template_pair_block(fb, ob)
    _copy_layernorm(fast.layer_norm, ori.layer_norm)
    fast.train(ori.training)
    emb.template_pair_stack = fast
    if hasattr(emb, "template_pointwise_att"):
        pw = emb.template_pointwise_att
        fpw = FastPointwise(c_t=pw.c_t, c_z=pw.c_z, c_hidden=pw.c_hidden, no_heads=pw.no_heads, inf=pw.inf)
        fpw = _like(fpw, pw)
        fpw.load_state_dict(pw.state_dict())
        fpw.train(pw.training)
        emb.template_pointwise_att = fpw


def inject_fastnn(model):
    """Returns ``model`` with ``evoformer``, ``extra_msa_stack`` and the template pair stack replaced by their fast twins
    (weights copied)."""
    with torch.no_grad():
        inject_evoformer(model)
        if model.config.extra_msa.enabled:
            inject_extra_msa(model)
        if model.config.template.enabled:
            inject_template(model)
        from ..models.fastnn.embedders import inject_embedder
        inject_embedder(model)
    return model


# ---------------------------------------------------------------------------
# The reference's helper names (fastfold/utils/inject_fastnn.py:24-318): scripts that build a fast module by hand and fill
# it from an OpenFold-layout module call these directly.
# ---------------------------------------------------------------------------
copy_layernorm = _copy_layernorm
copy_linear = _copy_linear
copy_native_linear = _copy_linear
copy_attention = _copy_attention
copy_transition = _copy_transition
copy_triangle = _copy_tri_mul
copy_triangle_att = _copy_tri_att
copy_global_attention = _copy_global_attention
copy_evoformer_para = copy_evoformer_block
copy_extra_msa_para = copy_extra_msa_block
copy_template_pair_stack_para = copy_template_pair_block


def _copy_stacked(fast, oris):
    _cp(fast.weight, torch.cat([o.weight for o in oris], dim=0))
    if getattr(fast, "bias", None) is not None and all(getattr(o, "bias", None) is not None for o in oris):
        _cp(fast.bias, torch.cat([o.bias for o in oris], dim=0))


def copy_kv_linear(model_fast, ori_k, ori_v):
    """Fills a fused ``[k; v]`` projection from the two separate ones."""
    _copy_stacked(model_fast, [ori_k, ori_v])


def copy_qkv_linear(model_fast, ori_q, ori_k, ori_v):
    """Fills a fused ``[q; k; v]`` projection from the three separate ones."""
    _copy_stacked(model_fast, [ori_q, ori_k, ori_v])


def copy_left_right(model_fast, ori_left, ori_right):
    """Fills a fused ``[left; right]`` triangle-multiplication projection (or gate) from its two halves."""
    _copy_stacked(model_fast, [ori_left, ori_right])


def copy_native_att(model_fast, model_ori):
    """Attention kept in the OpenFold layout on both sides (template pointwise attention): separate q / k / v / g / o."""
    for name in ("linear_q", "linear_k", "linear_v", "linear_g", "linear_o"):
        if hasattr(model_ori, name) and getattr(model_ori, name) is not None:
            _copy_linear(getattr(model_fast, name), getattr(model_ori, name))


def copy_template_pair_block_para(fast_module, target_module):
    """Every block of a template pair stack; a block in eval mode puts its twin in eval mode."""
    with torch.no_grad():
        for fb, ob in zip(fast_module.blocks, target_module.blocks):
            copy_template_pair_block(fb, ob)
            if not ob.training:
                fb.eval()


def copy_template_para(block_fast, block_ori):
    """A whole monomer template embedder (angle embedder, pair embedder, pair stack, pointwise attention)."""
    _copy_linear(block_fast.template_angle_embedder.linear_1, block_ori.template_angle_embedder.linear_1)
    _copy_linear(block_fast.template_angle_embedder.linear_2, block_ori.template_angle_embedder.linear_2)
    _copy_linear(block_fast.template_pair_embedder.linear, block_ori.template_pair_embedder.linear)
    copy_template_pair_block_para(block_fast.template_pair_stack, block_ori.template_pair_stack)
    _copy_layernorm(block_fast.template_pair_stack.layer_norm, block_ori.template_pair_stack.layer_norm)
    copy_native_att(block_fast.template_pointwise_att.mha, block_ori.template_pointwise_att.mha)


def copy_template_multimer_para(block_fast, block_ori):
    """A whole multimer template embedder: the pair embedder's per-feature projections, the single embedder, the pair
    stack and the final projection."""
    fp, op = block_fast.template_pair_embedder, block_ori.template_pair_embedder
    for name in ("dgram_linear", "aatype_linear_1", "aatype_linear_2", "query_embedding_linear", "pseudo_beta_mask_linear",
                 "x_linear", "y_linear", "z_linear", "backbone_mask_linear"):
        _copy_linear(getattr(fp, name), getattr(op, name))
    _copy_layernorm(fp.query_embedding_layer_norm, op.query_embedding_layer_norm)
    fs, os_ = block_fast.template_single_embedder, block_ori.template_single_embedder
    _copy_linear(fs.template_single_embedder, os_.template_single_embedder)
    _copy_linear(fs.template_projector, os_.template_projector)
    copy_template_pair_block_para(block_fast.template_pair_stack, block_ori.template_pair_stack)
    _copy_layernorm(block_fast.template_pair_stack.layer_norm, block_ori.template_pair_stack.layer_norm)
    _copy_linear(block_fast.linear_t, block_ori.linear_t)


def inject_embedder(model):
    """Swaps the input and recycling embedders for the lean ones (fastfold/utils/inject_fastnn.py:376-415)."""
    from ..models.fastnn.embedders import inject_embedder as fn
    return fn(model)


# ---------------------------------------------------------------------------
# inverse direction: OpenFold-named tensors out of a fast stack
# ---------------------------------------------------------------------------
def _split(t, n):
    return torch.chunk(t.detach(), n, dim=0)


def _attention_entries(prefix, fast, out_bias=None):
    q, k, v = _split(fast.to_qkv.weight, 3)
    d = {prefix + "linear_q.weight": q, prefix + "linear_k.weight": k, prefix + "linear_v.weight": v,
         prefix + "linear_g.weight": fast.gating_linear.weight.detach(), prefix + "linear_g.bias": fast.gating_bias.detach(),
         prefix + "linear_o.weight": fast.o_linear.weight.detach()}
    d[prefix + "linear_o.bias"] = (out_bias if out_bias is not None else fast.o_linear.bias).detach()
    return d


def _ln_entries(prefix, ln):
    return {prefix + "weight": ln.weight.detach(), prefix + "bias": ln.bias.detach()}


def _lin_entries(prefix, lin):
    d = {prefix + "weight": lin.weight.detach()}
    if lin.bias is not None:
        d[prefix + "bias"] = lin.bias.detach()
    return d


def _tri_mul_entries(prefix, fast):
    d = {}
    d.update(_ln_entries(prefix + "layer_norm_in.", fast.layernorm1))
    d.update(_ln_entries(prefix + "layer_norm_out.", fast.layernorm2))
    (ap, bp), (apb, bpb) = _split(fast.left_right_projection.weight, 2), _split(fast.left_right_projection.bias, 2)
    (ag, bg), (agb, bgb) = _split(fast.left_right_gate.weight, 2), _split(fast.left_right_gate.bias, 2)
    d.update({prefix + "linear_a_p.weight": ap, prefix + "linear_b_p.weight": bp, prefix + "linear_a_p.bias": apb, prefix + "linear_b_p.bias": bpb,
              prefix + "linear_a_g.weight": ag, prefix + "linear_b_g.weight": bg, prefix + "linear_a_g.bias": agb, prefix + "linear_b_g.bias": bgb})
    d.update(_lin_entries(prefix + "linear_g.", fast.output_gate))
    d[prefix + "linear_z.weight"] = fast.output_projection.weight.detach()
    d[prefix + "linear_z.bias"] = fast.output_bias.detach()
    return d


def _tri_att_entries(prefix, fast):
    d = _ln_entries(prefix + "layer_norm.", fast.layernorm1)
    d[prefix + "linear.weight"] = fast.linear_b.weight.detach()
    d.update(_attention_entries(prefix + "mha.", fast.attention, fast.out_bias))
    return d


def _transition_entries(prefix, fast):
    d = _ln_entries(prefix + "layer_norm.", fast.norm)
    d.update(_lin_entries(prefix + "linear_1.", fast.linear1))
    d.update(_lin_entries(prefix + "linear_2.", fast.linear2))
    return d


def _core_entries(prefix, opm, pair, msa_transition):
    d = _transition_entries(prefix + "msa_transition.", msa_transition)
    d.update(_ln_entries(prefix + "outer_product_mean.layer_norm.", opm.layernormM))
    d.update(_lin_entries(prefix + "outer_product_mean.linear_1.", opm.linear_a))
    d.update(_lin_entries(prefix + "outer_product_mean.linear_2.", opm.linear_b))
    d.update(_lin_entries(prefix + "outer_product_mean.linear_out.", opm.o_linear))
    d.update(_tri_mul_entries(prefix + "tri_mul_out.", pair.TriangleMultiplicationOutgoing))
    d.update(_tri_mul_entries(prefix + "tri_mul_in.", pair.TriangleMultiplicationIncoming))
    d.update(_tri_att_entries(prefix + "tri_att_start.", pair.TriangleAttentionStartingNode))
    d.update(_tri_att_entries(prefix + "tri_att_end.", pair.TriangleAttentionEndingNode))
    d.update(_transition_entries(prefix + "pair_transition.", pair.PairTransition))
    return d


def _row_att_entries(prefix, fast):
    d = _ln_entries(prefix + "layer_norm_m.", fast.layernormM)
    d.update(_ln_entries(prefix + "layer_norm_z.", fast.layernormZ))
    d[prefix + "linear_z.weight"] = fast.linear_b_weights.detach()
    d.update(_attention_entries(prefix + "mha.", fast.attention, fast.out_bias))
    return d


def extract_fastnn(model):
    """OpenFold-named ``state_dict`` of an injected model (non-injected parts keep their own names)."""
    sd = {k: v for k, v in model.state_dict().items() if not (k.startswith("evoformer.") or k.startswith("extra_msa_stack."))}
    evo = model.evoformer
    if isinstance(evo, FastEvoformerStack):
        for i, b in enumerate(evo.blocks):
            p = "evoformer.blocks.%d." % i
            sd.update(_row_att_entries(p + "msa_att_row.", b.msa.MSARowAttentionWithPairBias))
            sd.update(_ln_entries(p + "msa_att_col._msa_att.layer_norm_m.", b.msa.MSAColumnAttention.layernormM))
            sd.update(_attention_entries(p + "msa_att_col._msa_att.mha.", b.msa.MSAColumnAttention.attention))
            sd.update(_core_entries(p + "core.", b.communication, b.pair, b.msa.MSATransition))
        sd.update(_lin_entries("evoformer.linear.", evo.linear))
    else:
        sd.update({k: v for k, v in model.state_dict().items() if k.startswith("evoformer.")})
    ex = model.extra_msa_stack
    if isinstance(ex, FastExtraMSAStack):
        for i, b in enumerate(ex.blocks):
            p = "extra_msa_stack.blocks.%d." % i
            sd.update(_row_att_entries(p + "msa_att_row.", b.msa_stack.MSARowAttentionWithPairBias))
            ga = b.msa_stack.MSAColumnAttention
            sd.update(_ln_entries(p + "msa_att_col.layer_norm_m.", ga.layernormM))
            k, v = _split(ga.global_attention.to_kv.weight, 2)
            sd.update({p + "msa_att_col.global_attention.linear_q.weight": ga.global_attention.to_q.weight.detach(),
                       p + "msa_att_col.global_attention.linear_k.weight": k, p + "msa_att_col.global_attention.linear_v.weight": v,
                       p + "msa_att_col.global_attention.linear_g.weight": ga.global_attention.gating_linear.weight.detach(),
                       p + "msa_att_col.global_attention.linear_g.bias": ga.global_attention.gating_bias.detach()})
            sd.update(_lin_entries(p + "msa_att_col.global_attention.linear_o.", ga.global_attention.o_linear))
            sd.update(_core_entries(p + "core.", b.communication, b.pair_stack, b.msa_stack.MSATransition))
    else:
        sd.update({k: v for k, v in model.state_dict().items() if k.startswith("extra_msa_stack.")})
    tps = getattr(getattr(model, "template_embedder", None), "template_pair_stack", None)
    from ..models.fastnn.template import TemplatePairStack as FastTemplatePairStack
    if isinstance(tps, FastTemplatePairStack):
        pre = "template_embedder.template_pair_stack."
        sd = {k: v for k, v in sd.items() if not k.startswith(pre)}
        for i, b in enumerate(tps.blocks):
            p = pre + "blocks.%d." % i
            sd.update(_tri_att_entries(p + "tri_att_start.", b.TriangleAttentionStartingNode))
            sd.update(_tri_att_entries(p + "tri_att_end.", b.TriangleAttentionEndingNode))
            sd.update(_tri_mul_entries(p + "tri_mul_out.", b.TriangleMultiplicationOutgoing))
            sd.update(_tri_mul_entries(p + "tri_mul_in.", b.TriangleMultiplicationIncoming))
            sd.update(_transition_entries(p + "pair_transition.", b.PairTransition))
        sd.update(_ln_entries(pre + "layer_norm.", tps.layer_norm))
    return sd
