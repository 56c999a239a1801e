"""AlphaFold parameter archives (``params_model_*.npz``) <-> the OpenFold-layout model.

``import_jax_weights_(model, npz_path, version="model_1")`` fills ``model`` (before ``inject_fastnn``) from an
archive whose keys follow ``alphafold/alphafold_iteration/<module path>//<param>``; the 48 Evoformer and 4 extra-MSA
blocks are stored stacked along a leading axis under ``.../__layer_stack_no_state/...``.  ``export_jax_weights``
writes the same scheme from a model (used for the round-trip test and to hand weights to JAX tooling).  The
translation table is built from the live module tree, so a parameter that is not covered raises instead of being
skipped.  Same role as fastfold/utils/import_weights.py:25-627.
"""
import numpy as np
import torch

PREFIX = "alphafold/alphafold_iteration/"


# Each leaf of the translation tree: (list of torch tensors to fill, kind, stacked)
#   kind 'lin_w'  : jax [in, out]            <-> torch [out, in]
#        'plain'  : identical layout (biases, LayerNorm scale / offset, point weights)
#        'mha_w'  : jax [c_in, H, d]         <-> torch [H*d, c_in]
#        'mha_b'  : jax [H, d]               <-> torch [H*d]
#        'mha_o'  : jax [H, d, c_out]        <-> torch [c_out, H*d]
#        'opm_w'  : jax [c, c, c_z]          <-> torch [c_z, c*c]
#        'mm_w'   : multimer layers, jax [out] (one input feature) or [in, a, b, ...]  <-> torch [out, in]; meta = (a, b, ...)
#        'mm_b'   : jax [a, b, ...]          <-> torch [a*b*...]
#        'lin_w_swap' / 'plain_swap': as 'lin_w' / 'plain' with the two halves of the output axis exchanged (the fused
#                   projection of the incoming triangle multiplication: the archive stores [right | left])
def _swap_halves(t, dim):
    a, b = t.chunk(2, dim=dim)
    return torch.cat((b, a), dim=dim)


def _to_torch(a, kind):
    t = torch.as_tensor(np.asarray(a))
    if kind == "lin_w":
        return t.transpose(-1, -2)
    if kind == "plain":
        return t
    if kind == "mha_w":
        return t.reshape(*t.shape[:-2], -1).transpose(-1, -2)
    if kind == "mha_b":
        return t.reshape(*t.shape[:-2], -1)
    if kind == "mha_o":
        return t.reshape(*t.shape[:-3], -1, t.shape[-1]).transpose(-1, -2)
    if kind == "opm_w":
        return t.reshape(*t.shape[:-3], -1, t.shape[-1]).transpose(-1, -2)
    if kind == "mm_w":
        return t.unsqueeze(-1) if t.dim() == 1 else t.reshape(t.shape[0], -1).transpose(-1, -2)
    if kind == "mm_b":
        return t.reshape(-1)
    if kind == "lin_w_swap":
        return _swap_halves(t.transpose(-1, -2), -2)
    if kind == "plain_swap":
        return _swap_halves(t, -1)
    raise ValueError(kind)


def _to_jax(t, kind, meta):
    t = t.detach().cpu().float()
    if kind == "lin_w":
        return t.transpose(-1, -2).contiguous().numpy()
    if kind == "plain":
        return t.numpy()
    if kind == "mha_w":
        H = meta
        w = t.transpose(-1, -2)
        return w.reshape(*w.shape[:-1], H, -1).contiguous().numpy()
    if kind == "mha_b":
        return t.reshape(*t.shape[:-1], meta, -1).numpy()
    if kind == "mha_o":
        w = t.transpose(-1, -2)
        return w.reshape(*w.shape[:-2], meta, -1, w.shape[-1]).contiguous().numpy()
    if kind == "opm_w":
        w = t.transpose(-1, -2)
        return w.reshape(*w.shape[:-2], meta, meta, w.shape[-1]).contiguous().numpy()
    if kind == "mm_w":
        if meta is None:                                # [out, 1] -> [out]
            return t.squeeze(-1).numpy()
        return t.transpose(-1, -2).reshape(t.shape[-1], *meta).contiguous().numpy()
    if kind == "mm_b":
        return t.reshape(*meta).numpy() if meta else t.numpy()
    if kind == "lin_w_swap":
        return _swap_halves(t, -2).transpose(-1, -2).contiguous().numpy()
    if kind == "plain_swap":
        return _swap_halves(t, -1).contiguous().numpy()
    raise ValueError(kind)


class _Leaf:
    __slots__ = ("tensors", "kind", "meta")

    def __init__(self, tensors, kind, meta=None):
        self.tensors = tensors if isinstance(tensors, list) else [tensors]
        self.kind = kind
        self.meta = meta


def _linear(l):
    d = {"weights": _Leaf(l.weight, "lin_w")}
    if l.bias is not None:
        d["bias"] = _Leaf(l.bias, "plain")
    return d


def _layer_norm(l):
    return {"scale": _Leaf(l.weight, "plain"), "offset": _Leaf(l.bias, "plain")}


def _attention(a):
    H = a.no_heads
    d = {"query_w": _Leaf(a.linear_q.weight, "mha_w", H), "key_w": _Leaf(a.linear_k.weight, "mha_w", H),
         "value_w": _Leaf(a.linear_v.weight, "mha_w", H), "output_w": _Leaf(a.linear_o.weight, "mha_o", H),
         "output_b": _Leaf(a.linear_o.bias, "plain")}
    if a.linear_g is not None:
        d["gating_w"] = _Leaf(a.linear_g.weight, "mha_w", H)
        d["gating_b"] = _Leaf(a.linear_g.bias, "mha_b", H)
    return d


def _global_attention(a):
    H = a.no_heads
    return {"query_w": _Leaf(a.linear_q.weight, "mha_w", H), "key_w": _Leaf(a.linear_k.weight, "lin_w"),
            "value_w": _Leaf(a.linear_v.weight, "lin_w"), "gating_w": _Leaf(a.linear_g.weight, "mha_w", H),
            "gating_b": _Leaf(a.linear_g.bias, "mha_b", H), "output_w": _Leaf(a.linear_o.weight, "mha_o", H),
            "output_b": _Leaf(a.linear_o.bias, "plain")}


def _tri_att(t):
    return {"query_norm": _layer_norm(t.layer_norm), "feat_2d_weights": _Leaf(t.linear.weight, "lin_w"), "attention": _attention(t.mha)}


def _linear_swapped(l):
    return {"weights": _Leaf(l.weight, "lin_w_swap"), "bias": _Leaf(l.bias, "plain_swap")}


def _linear_mm(l, meta=None):
    d = {"weights": _Leaf(l.weight, "mm_w", meta)}
    if l.bias is not None:
        d["bias"] = _Leaf(l.bias, "mm_b", meta)
    return d


def _tri_mul(t):
    if getattr(t, "fused", False):
        # the module computes incoming as sum_k a[k,i] b[k,j] with (a, b) = halves of the projection; the archive's fused
        # layer orders the halves the other way round for the incoming update (fastfold/utils/import_weights.py:610-627)
        proj = _linear if t._outgoing else _linear_swapped
        return {"left_norm_input": _layer_norm(t.layer_norm_in), "projection": proj(t.linear_p), "gate": proj(t.linear_g),
                "center_norm": _layer_norm(t.layer_norm_out), "output_projection": _linear(t.linear_z), "gating_linear": _linear(t.linear_gate)}
    # The module computes outgoing as sum_k a[i,k] b[j,k] and incoming as sum_k a[k,i] b[k,j].  AlphaFold's incoming update is
    # einsum('kjc,kic->ijc', left, right) = sum_k right[k,i] left[k,j]: its "left" is this module's b and its "right" this module's
    # a, for projections and gates alike (fastfold/utils/import_weights.py:226-239).
    left_p, right_p, left_g, right_g = ((t.linear_a_p, t.linear_b_p, t.linear_a_g, t.linear_b_g) if t._outgoing else
                                        (t.linear_b_p, t.linear_a_p, t.linear_b_g, t.linear_a_g))
    return {"layer_norm_input": _layer_norm(t.layer_norm_in), "left_projection": _linear(left_p), "right_projection": _linear(right_p),
            "left_gate": _linear(left_g), "right_gate": _linear(right_g), "center_layer_norm": _layer_norm(t.layer_norm_out),
            "output_projection": _linear(t.linear_z), "gating_linear": _linear(t.linear_g)}


def _transition(t):
    return {"input_layer_norm": _layer_norm(t.layer_norm), "transition1": _linear(t.linear_1), "transition2": _linear(t.linear_2)}


def _opm(o):
    return {"layer_norm_input": _layer_norm(o.layer_norm), "left_projection": _linear(o.linear_1), "right_projection": _linear(o.linear_2),
            "output_w": _Leaf(o.linear_out.weight, "opm_w", o.c_hidden), "output_b": _Leaf(o.linear_out.bias, "plain")}


def _msa_row(m):
    return {"query_norm": _layer_norm(m.layer_norm_m), "feat_2d_norm": _layer_norm(m.layer_norm_z),
            "feat_2d_weights": _Leaf(m.linear_z.weight, "lin_w"), "attention": _attention(m.mha)}


def _core(c):
    return {"msa_transition": _transition(c.msa_transition), "outer_product_mean": _opm(c.outer_product_mean),
            "triangle_multiplication_outgoing": _tri_mul(c.tri_mul_out), "triangle_multiplication_incoming": _tri_mul(c.tri_mul_in),
            "triangle_attention_starting_node": _tri_att(c.tri_att_start), "triangle_attention_ending_node": _tri_att(c.tri_att_end),
            "pair_transition": _transition(c.pair_transition)}


def _evo_block(b):
    d = {"msa_row_attention_with_pair_bias": _msa_row(b.msa_att_row),
         "msa_column_attention": {"query_norm": _layer_norm(b.msa_att_col._msa_att.layer_norm_m), "attention": _attention(b.msa_att_col._msa_att.mha)}}
    d.update(_core(b.core))
    return d


def _extra_block(b):
    d = {"msa_row_attention_with_pair_bias": _msa_row(b.msa_att_row),
         "msa_column_global_attention": {"query_norm": _layer_norm(b.msa_att_col.layer_norm_m),
                                         "attention": _global_attention(b.msa_att_col.global_attention)}}
    d.update(_core(b.core))
    return d


def _stack(trees):
    """Merges per-block trees into one tree whose leaves hold the list of per-block tensors (stacked in the archive)."""
    first = trees[0]
    if isinstance(first, _Leaf):
        return _Leaf([t.tensors[0] for t in trees], first.kind, first.meta)
    return {k: _stack([t[k] for t in trees]) for k in first}


def _template_block(b):
    return {"triangle_attention_starting_node": _tri_att(b.tri_att_start), "triangle_attention_ending_node": _tri_att(b.tri_att_end),
            "triangle_multiplication_outgoing": _tri_mul(b.tri_mul_out), "triangle_multiplication_incoming": _tri_mul(b.tri_mul_in),
            "pair_transition": _transition(b.pair_transition)}


def _ipa(i):
    return {"q_scalar": _linear(i.linear_q), "kv_scalar": _linear(i.linear_kv), "q_point_local": _linear(i.linear_q_points),
            "kv_point_local": _linear(i.linear_kv_points), "attention_2d": _linear(i.linear_b),
            "trainable_point_weights": _Leaf(i.head_weights, "plain"), "output_projection": _linear(i.linear_out)}


def _ipa_multimer(i):
    H = i.no_heads

    def pts(pp):
        return {"point_projection": _linear_mm(pp.linear, (H, 3 * pp.num_points))}
    return {"q_scalar_projection": _linear_mm(i.linear_q, (H, i.c_hidden)), "k_scalar_projection": _linear_mm(i.linear_k, (H, i.c_hidden)),
            "v_scalar_projection": _linear_mm(i.linear_v, (H, i.c_hidden)), "q_point_projection": pts(i.linear_q_points),
            "k_point_projection": pts(i.linear_k_points), "v_point_projection": pts(i.linear_v_points),
            "attention_2d": _linear(i.linear_b), "trainable_point_weights": _Leaf(i.head_weights, "plain"),
            "output_projection": _linear(i.linear_out)}


def translation_tree(model, version="model_1"):
    """Nested dict {haiku module path: ... {param name: _Leaf}} describing every parameter of ``model``.  The multimer
    layout (chain-relative position encoding, nine template-pair input layers, split IPA projections, ``quat_rigid``
    backbone update) is chosen when ``version`` contains "multimer" (fastfold/utils/import_weights.py:131,470-560)."""
    sm = model.structure_module
    is_multimer = "multimer" in version
    fold = {"invariant_point_attention": _ipa_multimer(sm.ipa) if is_multimer else _ipa(sm.ipa),
            "attention_layer_norm": _layer_norm(sm.layer_norm_ipa),
            "transition_layer_norm": _layer_norm(sm.transition.layer_norm),
            ("quat_rigid" if is_multimer else "affine_update"): ({"rigid": _linear(sm.bb_update.linear)} if is_multimer
                                                                 else _linear(sm.bb_update.linear)),
            "rigid_sidechain": {"input_projection": _linear(sm.angle_resnet.linear_in), "input_projection_1": _linear(sm.angle_resnet.linear_initial),
                                "unnormalized_angles": _linear(sm.angle_resnet.linear_out)}}
    for li, layer in enumerate(sm.transition.layers):
        sfx = "" if li == 0 else "_%d" % li       # only one transition layer in every published model
        fold["transition" + sfx] = _linear(layer.linear_1)
        fold["transition_1" + sfx] = _linear(layer.linear_2)
        fold["transition_2" + sfx] = _linear(layer.linear_3)
    for bi, blk in enumerate(sm.angle_resnet.layers):
        sfx = "" if bi == 0 else "_%d" % bi
        fold["rigid_sidechain"]["resblock1" + sfx] = _linear(blk.linear_1)
        fold["rigid_sidechain"]["resblock2" + sfx] = _linear(blk.linear_2)
    evo = {
        "preprocess_1d": _linear(model.input_embedder.linear_tf_m), "preprocess_msa": _linear(model.input_embedder.linear_msa_m),
        "left_single": _linear(model.input_embedder.linear_tf_z_i), "right_single": _linear(model.input_embedder.linear_tf_z_j),
        "prev_pos_linear": _linear(model.recycling_embedder.linear), "prev_msa_first_row_norm": _layer_norm(model.recycling_embedder.layer_norm_m),
        "prev_pair_norm": _layer_norm(model.recycling_embedder.layer_norm_z),
        "extra_msa_activations": _linear(model.extra_msa_embedder.linear),
        "extra_msa_stack": _stack([_extra_block(b) for b in model.extra_msa_stack.blocks]),
        "evoformer_iteration": _stack([_evo_block(b) for b in model.evoformer.blocks]),
        "single_activations": _linear(model.evoformer.linear),
    }
    if is_multimer:
        evo["~_relative_encoding"] = {"position_activations": _linear(model.input_embedder.linear_relpos)}
    else:
        evo["pair_activiations"] = _linear(model.input_embedder.linear_relpos)
    no_templ = not is_multimer and any(v in version for v in ("model_3", "model_4", "model_5"))
    if model.config.template.enabled and is_multimer:
        te = model.template_embedder
        pe = te.template_pair_embedder
        single = {"query_embedding_norm": _layer_norm(pe.query_embedding_layer_norm),
                  "template_embedding_iteration": _stack([_template_block(b) for b in te.template_pair_stack.blocks]),
                  "output_layer_norm": _layer_norm(te.template_pair_stack.layer_norm)}
        inputs = [(pe.dgram_linear, False), (pe.pseudo_beta_mask_linear, True), (pe.aatype_linear_1, False), (pe.aatype_linear_2, False),
                  (pe.x_linear, True), (pe.y_linear, True), (pe.z_linear, True), (pe.backbone_mask_linear, True),
                  (pe.query_embedding_linear, False)]
        for n, (lin, one_feature) in enumerate(inputs):
            single["template_pair_embedding_%d" % n] = _linear_mm(lin) if one_feature else _linear(lin)
        evo["template_embedding"] = {"single_template_embedding": single, "output_linear": _linear(te.linear_t)}
        evo["template_projection"] = _linear(te.template_single_embedder.template_projector)
        evo["template_single_embedding"] = _linear(te.template_single_embedder.template_single_embedder)
    elif model.config.template.enabled and not no_templ:
        te = model.template_embedder
        evo["template_embedding"] = {
            "single_template_embedding": {
                "embedding2d": _linear(te.template_pair_embedder.linear),
                "template_pair_stack": {"__layer_stack_no_state": _stack([_template_block(b) for b in te.template_pair_stack.blocks])},
                "output_layer_norm": _layer_norm(te.template_pair_stack.layer_norm)},
            "attention": _attention(te.template_pointwise_att.mha)}
        evo["template_single_embedding"] = _linear(te.template_angle_embedder.linear_1)
        evo["template_projection"] = _linear(te.template_angle_embedder.linear_2)
    h = model.aux_heads
    tree = {
        "evoformer": evo,
        "structure_module": {"single_layer_norm": _layer_norm(sm.layer_norm_s), "initial_projection": _linear(sm.linear_in),
                             "pair_layer_norm": _layer_norm(sm.layer_norm_z), "fold_iteration": fold},
        "predicted_lddt_head": {"input_layer_norm": _layer_norm(h.plddt.layer_norm), "act_0": _linear(h.plddt.linear_1),
                                "act_1": _linear(h.plddt.linear_2), "logits": _linear(h.plddt.linear_3)},
        "distogram_head": {"half_logits": _linear(h.distogram.linear)},
        "experimentally_resolved_head": {"logits": _linear(h.experimentally_resolved.linear)},
        "masked_msa_head": {"logits": _linear(h.masked_msa.linear)},
    }
    if hasattr(h, "tm"):
        tree["predicted_aligned_error_head"] = {"logits": _linear(h.tm.linear)}
    return tree


# scopes whose parameters are stored stacked over their blocks (leading axis = block index)
_STACKED = ("/extra_msa_stack/", "/evoformer_iteration/", "/__layer_stack_no_state/", "/template_embedding_iteration/")


def _flatten(tree, path=""):
    """{archive key: _Leaf}: module path elements joined by '/', parameter name after '//'."""
    out = {}
    for k, v in tree.items():
        if isinstance(v, _Leaf):
            out[path.rstrip("/") + "//" + k] = v
        else:
            out.update(_flatten(v, path + k + "/"))
    return out


def flat_translation(model, version="model_1"):
    return {PREFIX + k: v for k, v in _flatten(translation_tree(model, version)).items()}


# ---------------------------------------------------------------------------
# The reference's vocabulary for the same table (fastfold/utils/import_weights.py:25-70): a ``Param`` names the target
# tensor(s), how the archive's array maps onto them (``ParamType``) and whether the archive entry stacks one array per block.
# ---------------------------------------------------------------------------
import enum


class ParamType(enum.Enum):
    LinearWeight = "lin_w"
    LinearWeightMHA = "mha_w"
    LinearMHAOutputWeight = "mha_o"
    LinearBiasMHA = "mha_b"
    LinearWeightOPM = "opm_w"
    LinearWeightMultimer = "mm_w"
    LinearBiasMultimer = "mm_b"
    LinearWeightSwapped = "lin_w_swap"
    OtherSwapped = "plain_swap"
    Other = "plain"


class Param:
    """``param``: the model tensor, or the list of per-block tensors of a stacked entry; ``param_type``; ``stacked``."""

    def __init__(self, param, param_type=ParamType.Other, stacked=False, meta=None):
        self.param, self.param_type, self.stacked, self.meta = param, param_type, stacked, meta

    def __repr__(self):
        return "Param(%s, stacked=%s)" % (self.param_type.name, self.stacked)


def get_translation_dict(model, version="model_1"):
    """``{archive key: Param}`` for every array of an AlphaFold parameter archive that ``model`` consumes."""
    out = {}
    for key, leaf in flat_translation(model, version).items():
        stacked = len(leaf.tensors) > 1 or any(tag in key for tag in _STACKED)
        out[key] = Param(leaf.tensors if stacked else leaf.tensors[0], ParamType(leaf.kind), stacked, leaf.meta)
    return out


def stacked(param_dict_list, out=None):
    """Merges a list of identically shaped (nested) ``{name: Param}`` trees - one per block - into one tree whose leaves are
    stacked ``Param``s holding the list of per-block tensors (fastfold/utils/import_weights.py:81-107)."""
    out = {} if out is None else out
    first = param_dict_list[0]
    for k, v0 in first.items():
        column = [d[k] for d in param_dict_list]
        if isinstance(v0, dict):
            out[k] = stacked(column, out={})
        elif isinstance(v0, Param):
            out[k] = Param([p.param for p in column], v0.param_type, True, v0.meta)
    return out


def assign(translation_dict, orig_weights):
    """Copies the arrays of ``orig_weights`` into the tensors of a flat ``{archive key: Param}`` table, applying each entry's
    layout transformation; a stacked entry is split along its leading axis (fastfold/utils/import_weights.py:110-129)."""
    with torch.no_grad():
        for key, param in translation_dict.items():
            t = _to_torch(orig_weights[key], param.param_type.value)
            dsts, srcs = (param.param, torch.unbind(t, dim=0)) if param.stacked else ([param.param], [t])
            if len(dsts) != len(srcs):
                raise ValueError("%s: %d arrays for %d tensors" % (key, len(srcs), len(dsts)))
            for dst, src in zip(dsts, srcs):
                if dst.numel() != src.numel():
                    raise ValueError("%s: archive shape %s does not fit parameter shape %s" % (key, tuple(src.shape), tuple(dst.shape)))
                dst.copy_(src.reshape(dst.shape).to(dst.dtype))


def import_jax_weights_(model, npz_path, version="model_1"):
    data = np.load(npz_path) if isinstance(npz_path, str) else npz_path
    flat = flat_translation(model, version)
    missing = [k for k in flat if k not in data]
    if missing:
        raise KeyError("archive lacks %d expected keys, e.g. %s" % (len(missing), missing[:3]))
    with torch.no_grad():
        for key, leaf in flat.items():
            t = _to_torch(data[key], leaf.kind)
            if any(sc in key for sc in _STACKED):
                if t.shape[0] != len(leaf.tensors):
                    raise ValueError("%s: %d stacked layers in the archive, %d blocks in the model" % (key, t.shape[0], len(leaf.tensors)))
                for dst, src in zip(leaf.tensors, torch.unbind(t, dim=0)):
                    dst.copy_(src.reshape(dst.shape).to(dst.dtype))
            else:
                leaf.tensors[0].copy_(t.reshape(leaf.tensors[0].shape).to(leaf.tensors[0].dtype))
    covered = {id(t) for leaf in flat.values() for t in leaf.tensors}
    # models 3-5 have no template parameters in their archives; the (unused) template modules keep their init
    left = [n for n, p in model.named_parameters() if id(p) not in covered and not n.startswith("template_embedder.")]
    if left:
        raise RuntimeError("parameters without an archive entry: %s" % left[:5])
    return model


def export_jax_weights(model, version="model_1"):
    """{archive key: numpy array} in the AlphaFold naming / layout (inverse of ``import_jax_weights_``)."""
    out = {}
    for key, leaf in flat_translation(model, version).items():
        arrs = [_to_jax(t, leaf.kind, leaf.meta) for t in leaf.tensors]
        stacked = any(sc in key for sc in _STACKED)
        out[key] = np.stack(arrs, axis=0) if stacked else arrs[0]
    return out


def import_openfold_state_dict_(model, state_dict, strict=True):
    """Loads an OpenFold-style ``state_dict`` (``evoformer.blocks.0.msa_att_row.mha.linear_q.weight`` ...), also when the
    keys carry a ``model.`` / ``module.`` prefix as written by training wrappers."""
    sd = {}
    for k, v in state_dict.items():
        for pre in ("module.", "model."):
            if k.startswith(pre):
                k = k[len(pre):]
        sd[k] = v
    return model.load_state_dict(sd, strict=strict)
