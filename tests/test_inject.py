"""fastnn modules against their OpenFold-layout twins with injected weights (CPU, fp32), and the name round trip.

Mirrors the reference's module / stack / end-to-end parity tests (tests/test_fastnn/test_evoformer_stack.py:76-81,
tests/test_inference.py:74-75) with random-init weights and synthetic features instead of downloaded fixtures.
"""
import copy

import pytest
import torch

from fastfold_b200.config import model_config, set_shared
from fastfold_b200.models.fastnn import set_chunk_size
from fastfold_b200.models.hub import AlphaFold
from fastfold_b200.utils.inject_fastnn import extract_fastnn, inject_fastnn
from fastfold_b200.utils.synthetic import random_features


def _small_model(templates=False):
    c = model_config("model_1" if templates else "model_3")
    c.model.evoformer_stack.no_blocks = 2
    c.model.extra_msa.extra_msa_stack.no_blocks = 2
    c.model.structure_module.no_blocks = 2
    set_shared(c, "chunk_size", None)
    torch.manual_seed(0)
    m = AlphaFold(c).eval()
    g = torch.Generator().manual_seed(1)
    with torch.no_grad():
        for p in m.parameters():      # zero-initialised ("final") layers would hide differences
            if p.dim() >= 2 and float(p.abs().sum()) == 0.0:
                p.copy_(torch.randn(p.shape, generator=g) * 0.05)
    return m, c


@pytest.mark.parametrize("chunk", [None, 3])
@pytest.mark.parametrize("inplace", [False, True])
def test_inference_matches_reference_layout(chunk, inplace):
    ref, cfg = _small_model()
    batch = random_features(13, 7, 9, n_recycle=1, seed=3)
    with torch.no_grad():
        want = ref(copy.deepcopy(batch))
    fast = inject_fastnn(copy.deepcopy(ref))
    fast.globals.inplace = inplace
    set_chunk_size(chunk)
    try:
        with torch.no_grad():
            got = fast(copy.deepcopy(batch))
    finally:
        set_chunk_size(None)
    assert (got["final_atom_positions"] - want["final_atom_positions"]).abs().max() < 5e-4
    assert (got["pair"] - want["pair"]).abs().mean() < 2e-3
    assert (got["msa"] - want["msa"]).abs().mean() < 2e-3


def test_extract_round_trip():
    ref, cfg = _small_model()
    fast = inject_fastnn(copy.deepcopy(ref))
    sd = extract_fastnn(fast)
    want = ref.state_dict()
    assert set(sd.keys()) == set(want.keys())
    for k, v in want.items():
        assert torch.equal(sd[k], v), k


def test_template_stack_injection_matches_reference_layout():
    """model_1 (templates on): the injected fast template pair stack reproduces the OpenFold-layout one."""
    ref, cfg = _small_model(templates=True)
    batch = random_features(13, 7, 9, n_templ=2, n_recycle=0, seed=5)
    with torch.no_grad():
        want = ref(copy.deepcopy(batch))
    fast = inject_fastnn(copy.deepcopy(ref))
    from fastfold_b200.models.fastnn.template import TemplatePairStack
    assert isinstance(fast.template_embedder.template_pair_stack, TemplatePairStack)
    with torch.no_grad():
        got = fast(copy.deepcopy(batch))
    assert (got["pair"] - want["pair"]).abs().mean() < 2e-3
    assert (got["final_atom_positions"] - want["final_atom_positions"]).abs().max() < 5e-4


def test_extract_round_trip_with_templates():
    ref, cfg = _small_model(templates=True)
    fast = inject_fastnn(copy.deepcopy(ref))
    sd = extract_fastnn(fast)
    want = ref.state_dict()
    assert set(sd.keys()) == set(want.keys())
    for k, v in want.items():
        assert torch.equal(sd[k], v), k
