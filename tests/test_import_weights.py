"""Parameter-archive round trip: export in the AlphaFold key scheme, import into a fresh model, compare every tensor.

Covers what the reference leaves untested (import of archives / OpenFold state_dicts) without needing the published
weights: the archive is synthesised from a random-init model, so the test checks key coverage and the layout
transforms (transposes, head reshapes, stacked trunks), including the template stack and the pTM head.
"""
import io

import numpy as np
import pytest
import torch

from fastfold_b200.config import model_config
from fastfold_b200.models.hub import AlphaFold
from fastfold_b200.utils.import_weights import (PREFIX, export_jax_weights, import_jax_weights_, import_openfold_state_dict_)


def _model(name, seed):
    c = model_config(name)
    c.model.evoformer_stack.no_blocks = 3
    c.model.extra_msa.extra_msa_stack.no_blocks = 2
    torch.manual_seed(seed)
    m = AlphaFold(c)
    with torch.no_grad():
        for p in m.parameters():
            p.copy_(torch.randn_like(p))
    return m


@pytest.mark.parametrize("name", ["model_1_ptm", "model_3"])
def test_archive_round_trip(name):
    src = _model(name, 0)
    arch = export_jax_weights(src, version=name)
    assert all(k.startswith(PREFIX) and "//" in k for k in arch)
    key = PREFIX + "evoformer/evoformer_iteration/msa_row_attention_with_pair_bias/attention//query_w"
    assert arch[key].shape == (3, 256, 8, 32)
    assert arch[PREFIX + "evoformer/evoformer_iteration/outer_product_mean//output_w"].shape == (3, 32, 32, 128)
    assert arch[PREFIX + "structure_module/fold_iteration/invariant_point_attention//trainable_point_weights"].shape == (12,)
    if name == "model_1_ptm":
        k = PREFIX + "evoformer/template_embedding/single_template_embedding/template_pair_stack/__layer_stack_no_state/pair_transition/transition1//weights"
        assert arch[k].shape == (2, 64, 128)
        assert PREFIX + "predicted_aligned_error_head/logits//weights" in arch
    buf = io.BytesIO()
    np.savez(buf, **arch)
    buf.seek(0)
    dst = _model(name, 1)
    import_jax_weights_(dst, np.load(buf), version=name)
    a, b = src.state_dict(), dst.state_dict()
    assert a.keys() == b.keys()
    for k in a:
        if name == "model_3" and k.startswith("template_embedder."):
            continue        # no template parameters in the archives of models 3-5
        assert torch.equal(a[k], b[k]), k


def test_openfold_state_dict_import():
    src, dst = _model("model_3", 0), _model("model_3", 1)
    sd = {"module." + k: v for k, v in src.state_dict().items()}
    import_openfold_state_dict_(dst, sd)
    for k, v in src.state_dict().items():
        assert torch.equal(v, dst.state_dict()[k])


@pytest.mark.parametrize("fused", [False, True])
def test_multimer_archive_round_trip(fused):
    """Multimer layout: chain-relative position layer, nine template-pair input layers (five with one input feature,
    stored as vectors), split IPA projections stored [c_s, H, ...], ``quat_rigid`` backbone update, and - with the fused
    triangle-multiplication layout of the v3 weights - the exchanged halves of the incoming update's projection."""
    from fastfold_b200.models.nn.pair import set_fused_triangle_multiplication
    name = "model_1_multimer_v3" if fused else "model_1_multimer"
    set_fused_triangle_multiplication(fused)
    try:
        c = model_config(name)
        c.model.evoformer_stack.no_blocks = 2
        c.model.extra_msa.extra_msa_stack.no_blocks = 1
        models = []
        for seed in (0, 1):
            torch.manual_seed(seed)
            m = AlphaFold(c)
            with torch.no_grad():
                for p in m.parameters():
                    p.copy_(torch.randn_like(p))
            models.append(m)
    finally:
        set_fused_triangle_multiplication(False)
    src, dst = models
    arch = export_jax_weights(src, version=name)
    ipa = PREFIX + "structure_module/fold_iteration/invariant_point_attention/"
    H, ch = src.structure_module.ipa.no_heads, src.structure_module.ipa.c_hidden
    assert arch[ipa + "q_scalar_projection//weights"].shape == (384, H, ch)
    assert arch[ipa + "k_point_projection/point_projection//weights"].shape == (384, H, 3 * src.structure_module.ipa.no_qk_points)
    assert arch[ipa + "v_point_projection/point_projection//bias"].shape == (H, 3 * src.structure_module.ipa.no_v_points)
    assert PREFIX + "structure_module/fold_iteration/quat_rigid/rigid//weights" in arch
    assert PREFIX + "evoformer/~_relative_encoding/position_activations//weights" in arch
    st = PREFIX + "evoformer/template_embedding/single_template_embedding/"
    assert arch[st + "template_pair_embedding_4//weights"].shape == (64,) and arch[st + "template_pair_embedding_0//weights"].shape == (39, 64)
    assert arch[st + "template_embedding_iteration/pair_transition/transition1//weights"].shape[0] == 2
    tri = PREFIX + "evoformer/evoformer_iteration/triangle_multiplication_incoming/"
    if fused:
        w = src.evoformer.blocks[0].core.tri_mul_in.linear_p.weight.detach()          # [2c, c_z], halves (a | b)
        a, b = w.chunk(2, dim=0)
        assert np.array_equal(arch[tri + "projection//weights"][0], torch.cat((b, a), 0).t().numpy())
        wo = src.evoformer.blocks[0].core.tri_mul_out.linear_p.weight.detach()
        assert np.array_equal(arch[tri.replace("incoming", "outgoing") + "projection//weights"][0], wo.t().numpy())
    else:
        assert tri + "left_projection//weights" in arch
    import_jax_weights_(dst, arch, version=name)
    a, b = src.state_dict(), dst.state_dict()
    assert a.keys() == b.keys()
    for k in a:
        assert torch.equal(a[k], b[k]), k
