"""Fast (DAP-aware) modules against the OpenFold-layout modules they replace, one module per test, with and without
chunking - the module list of the reference's tests/test_fastnn/ (test_msa_att_row, test_msa_att_col,
test_msa_global_att_col, test_out_product_mean, test_evoformer_stack, test_extramsa_stack), on the CPU in fp32.
The fast modules return the residual stream (input + update); the OpenFold-layout modules return the update."""
import pytest
import torch

from fastfold_b200.models import fastnn
from fastfold_b200.models import nn as ref
from fastfold_b200.models.fastnn import ops as fops
from fastfold_b200.models.nn.evoformer import EvoformerStack as RefEvoformerStack, ExtraMSAStack as RefExtraMSAStack
from fastfold_b200.models.nn.msa import MSAColumnAttention, MSAColumnGlobalAttention, MSARowAttentionWithPairBias
from fastfold_b200.models.nn.pair import OuterProductMean
import importlib

inj = importlib.import_module("fastfold_b200.utils.inject_fastnn")          # ``fastfold_b200.utils.inject_fastnn`` is also a function

S, N, C_M, C_Z = 6, 10, 32, 16


@pytest.fixture(autouse=True)
def _reset_chunk():
    yield
    fops.set_chunk_size(None)


def _randomize(module, seed):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for p in module.parameters():
            p.copy_(torch.randn(p.shape, generator=g) * 0.2)
    return module.eval()


def _inputs(seed=0):
    g = torch.Generator().manual_seed(seed)
    m = torch.randn(S, N, C_M, generator=g)
    z = torch.randn(N, N, C_Z, generator=g)
    msa_mask = (torch.rand(S, N, generator=g) > 0.15).float()
    msa_mask[0] = 1
    pair_mask = (torch.rand(N, N, generator=g) > 0.1).float()
    return m, z, msa_mask, pair_mask


@pytest.mark.parametrize("chunk", [None, 4])
def test_msa_att_row(chunk):
    m, z, msa_mask, _ = _inputs()
    ori = _randomize(MSARowAttentionWithPairBias(C_M, C_Z, 8, 4), 1)
    fast = fastnn.msa.MSARowAttentionWithPairBias(d_node=C_M, d_pair=C_Z, c=8, n_head=4).eval()
    inj._copy_row_attention(fast, ori)
    fops.set_chunk_size(chunk)
    with torch.no_grad():
        want = m + ori(m, z=z, mask=msa_mask, chunk_size=chunk)
        got = fast(m[None], z[None], msa_mask[None])[0]
    assert (got - want).abs().max() < 2e-5


@pytest.mark.parametrize("chunk", [None, 4])
def test_msa_att_col(chunk):
    m, _, msa_mask, _ = _inputs(1)
    ori = _randomize(MSAColumnAttention(C_M, 8, 4), 2)
    fast = fastnn.msa.MSAColumnAttention(d_node=C_M, c=8, n_head=4).eval()
    inj._copy_layernorm(fast.layernormM, ori._msa_att.layer_norm_m)
    inj._copy_attention(fast.attention, ori._msa_att.mha)
    fops.set_chunk_size(chunk)
    with torch.no_grad():
        want = m + ori(m, mask=msa_mask, chunk_size=chunk)
        got = fast(m[None], msa_mask[None])[0]
    assert (got - want).abs().max() < 2e-5


@pytest.mark.parametrize("chunk", [None, 4])
def test_msa_global_att_col(chunk):
    m, _, msa_mask, _ = _inputs(2)
    ori = _randomize(MSAColumnGlobalAttention(C_M, 8, 4), 3)
    fast = fastnn.msa.MSAColumnGlobalAttention(d_node=C_M, c=8, n_head=4).eval()
    inj._copy_layernorm(fast.layernormM, ori.layer_norm_m)
    inj._copy_global_attention(fast.global_attention, ori.global_attention)
    fops.set_chunk_size(chunk)
    with torch.no_grad():
        want = m + ori(m, mask=msa_mask, chunk_size=chunk)
        got = fast(m[None], msa_mask[None])[0]
    assert (got - want).abs().max() < 2e-5


@pytest.mark.parametrize("chunk", [None, 4])
def test_out_product_mean(chunk):
    m, z, msa_mask, _ = _inputs(3)
    ori = _randomize(OuterProductMean(C_M, C_Z, 8), 4)
    fast = fastnn.ops.OutProductMean(n_feat=C_M, n_feat_out=C_Z, n_feat_proj=8).eval()
    inj._copy_layernorm(fast.layernormM, ori.layer_norm)
    inj._copy_linear(fast.linear_a, ori.linear_1)
    inj._copy_linear(fast.linear_b, ori.linear_2)
    inj._copy_linear(fast.o_linear, ori.linear_out)
    fops.set_chunk_size(chunk)
    with torch.no_grad():
        want = z + ori(m, mask=msa_mask, chunk_size=chunk)
        got = fast(m[None], msa_mask[None], z[None])[0]
    assert (got - want).abs().max() < 2e-5


def _stack_cfg(c_hidden_msa_att):
    # hidden sizes of the published model (the fast modules are built for them); small c_m / c_z keep the test quick
    return dict(c_m=C_M, c_z=C_Z, c_hidden_msa_att=c_hidden_msa_att, c_hidden_opm=32, c_hidden_mul=C_Z, c_hidden_pair_att=C_Z // 4, no_heads_msa=8,
                no_heads_pair=4, transition_n=4, msa_dropout=0.15, pair_dropout=0.25, inf=1e9, eps=1e-8)


@pytest.mark.parametrize("chunk", [None, 4])
def test_evoformer_stack(chunk):
    m, z, msa_mask, pair_mask = _inputs(4)
    ori = _randomize(RefEvoformerStack(c_s=24, no_blocks=3, blocks_per_ckpt=None, clear_cache_between_blocks=False, **_stack_cfg(32)), 5)
    fast = fastnn.EvoformerStack(c_m=C_M, c_z=C_Z, c_s=24, no_blocks=3, blocks_per_ckpt=None).eval()
    for fb, ob in zip(fast.blocks, ori.blocks):
        inj.copy_evoformer_block(fb, ob)
    inj._copy_linear(fast.linear, ori.linear)
    fops.set_chunk_size(chunk)
    with torch.no_grad():
        m1, z1, s1 = ori(m, z, msa_mask=msa_mask, pair_mask=pair_mask, chunk_size=chunk, _mask_trans=False)   # as the model config sets it
        m2, z2, s2 = fast(m, z, msa_mask=msa_mask, pair_mask=pair_mask, chunk_size=chunk, _mask_trans=False)
    for a, b in ((m1, m2), (z1, z2), (s1, s2)):          # the reference's gate: mean absolute difference below 2e-3
        assert torch.isfinite(b).all() and (a - b).abs().mean() < 2e-3 * max(1.0, float(a.abs().mean()))


@pytest.mark.parametrize("chunk", [None, 4])
def test_extramsa_stack(chunk):
    m, z, msa_mask, pair_mask = _inputs(5)
    ori = _randomize(RefExtraMSAStack(no_blocks=2, ckpt=False, clear_cache_between_blocks=False, **_stack_cfg(8)), 6)
    fast = fastnn.ExtraMSAStack(c_m=C_M, c_z=C_Z, no_blocks=2).eval()
    for fb, ob in zip(fast.blocks, ori.blocks):
        inj.copy_extra_msa_block(fb, ob)
    fops.set_chunk_size(chunk)
    with torch.no_grad():
        z1 = ori(m, z, chunk_size=chunk, msa_mask=msa_mask, pair_mask=pair_mask, _mask_trans=False)
        z2 = fast(m, z, chunk_size=chunk, msa_mask=msa_mask, pair_mask=pair_mask, _mask_trans=False)
    assert torch.isfinite(z2).all() and (z1 - z2).abs().mean() < 2e-3 * max(1.0, float(z1.abs().mean()))
