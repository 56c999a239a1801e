"""Regression tests for faults found by review: template-stack dropout under checkpointing, status propagation,
checkpoint loading of template models, the replicated-parameter filter."""
import copy

import pytest
import torch

from fastfold_b200.config import model_config
from fastfold_b200.models.fastnn.template import TemplatePairStack
from fastfold_b200.runtime.trainer import check_device_status, default_replicated_param_filter


def _stack(blocks_per_ckpt):
    torch.manual_seed(3)
    s = TemplatePairStack(c_t=16, c_hidden_tri_att=4, c_hidden_tri_mul=16, no_blocks=2, no_heads=2, pair_transition_n=2, dropout_rate=0.25,
                          blocks_per_ckpt=blocks_per_ckpt)
    with torch.no_grad():
        for p in s.parameters():
            if p.dim() >= 2 and float(p.abs().sum()) == 0.0:
                p.normal_(0.0, 0.1)
    return s.train()


def test_template_stack_checkpoint_uses_first_pass_masks():
    """With dropout active, the checkpointed stack (recomputation in backward) and the plain stack give the same
    gradients: the masks are drawn once, outside the checkpoint boundary."""
    t = torch.randn(2, 12, 12, 16)
    mask = torch.ones(2, 12, 12)
    grads = []
    for bpc in (None, 1):
        s = _stack(bpc)
        x = t.clone().requires_grad_(True)
        torch.manual_seed(11)
        out = s(x, mask)
        out.square().sum().backward()
        grads.append((x.grad.clone(), [p.grad.clone() for p in s.parameters()]))
    assert torch.allclose(grads[0][0], grads[1][0], rtol=1e-4, atol=1e-5)
    for a, b in zip(grads[0][1], grads[1][1]):
        assert torch.allclose(a, b, rtol=1e-4, atol=1e-5)


def test_status_check_raises_on_reported_failure():
    check_device_status(reader=lambda: [0, 0, 0, 0, 0, 0, 0, 0])
    with pytest.raises(RuntimeError, match="device status 4"):
        check_device_status(reader=lambda: [4, 1, 0, 0, 0x203, 0, 0, 0])


def test_replicated_filter():
    f = default_replicated_param_filter
    assert not f("evoformer.blocks.3.msa.MSATransition.linear1.weight")
    assert not f("extra_msa_stack.blocks.0.communication.o_linear.bias")
    assert not f("template_embedder.template_pair_stack.blocks.1.PairTransition.norm.weight")
    assert f("template_embedder.template_pair_stack.layer_norm.weight")
    assert f("evoformer.linear.weight") and f("structure_module.ipa.linear_q.weight") and f("input_embedder.linear_tf_z.weight")
    assert not f("blocks.0.pair.PairTransition.linear1.weight") and f("linear.weight")


def test_checkpoint_loader_handles_injected_template_stack(tmp_path):
    """OpenFold-named tensors of a template-enabled model load into the injected (fast-named) model."""
    from fastfold_b200.models.hub import AlphaFold
    from fastfold_b200.runtime.checkpoint import _load_openfold_named
    from fastfold_b200.utils.inject_fastnn import extract_fastnn, inject_fastnn
    cfg = model_config("model_1")
    cfg.model.evoformer_stack.no_blocks = 1
    cfg.model.extra_msa.extra_msa_stack.no_blocks = 1
    torch.manual_seed(0)
    src = AlphaFold(cfg)
    with torch.no_grad():
        for p in src.parameters():
            p.normal_(0.0, 0.05)
    sd = {k: v.clone() for k, v in src.state_dict().items()}
    torch.manual_seed(1)
    dst = inject_fastnn(AlphaFold(cfg))
    _load_openfold_named(dst, sd)
    back = extract_fastnn(dst)
    assert set(back) == set(sd)
    for k in sd:
        assert torch.allclose(back[k].float(), sd[k].float(), atol=1e-6), k
