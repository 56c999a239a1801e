"""The reference's import paths and call signatures (README usage, inference.py:42, benchmark/perf.py:7-8)."""
import torch


def test_reference_import_paths():
    from fastfold.distributed import init_dap, scatter, gather, row_to_col, col_to_row, _split, _gather, _reduce, copy, reduce  # noqa: F401
    from fastfold.distributed.comm_async import (gather_async, gather_async_opp, All_to_All_Async, All_to_All_Async_Opp,  # noqa: F401
                                                 broadcast_sync, broadcast_async, broadcast_async_opp, get_rank, get_world_size)
    from fastfold.model.fastnn import (Evoformer, EvoformerStack, ExtraMSAStack, MSACore, ExtraMSACore, ExtraMSABlock,  # noqa: F401
                                       OutProductMean, PairCore, set_chunk_size)
    from fastfold.model.fastnn.kernel import (LayerNorm, fused_softmax, fused_attention_core, bias_dropout_add, bias_sigmod_ele,  # noqa: F401
                                              bias_ele_dropout_residual)
    from fastfold.model.hub import AlphaFold, AlphaFoldLoss, AlphaFoldLRScheduler  # noqa: F401
    from fastfold.utils.inject_fastnn import inject_fastnn  # noqa: F401
    from fastfold.utils import inject_fastnn as inject2  # noqa: F401
    from fastfold.utils.import_weights import import_jax_weights_  # noqa: F401
    from fastfold.config import model_config  # noqa: F401
    import fastfold_b200.models.fastnn as real
    assert Evoformer is real.Evoformer


def test_evoformer_default_constructor_and_call():
    from fastfold.model.fastnn import Evoformer
    blk = Evoformer().eval()          # README spelling: no arguments
    m, z = torch.randn(4, 8, 256), torch.randn(8, 8, 128)
    with torch.no_grad():
        om, oz = blk(m, z, torch.ones(4, 8), torch.ones(8, 8), chunk_size=None, _mask_trans=True)
    assert om.shape == m.shape and oz.shape == z.shape
    ml, zl = [m.clone()], [z.clone()]
    with torch.no_grad():
        ml, zl = blk.inplace(ml, zl, torch.ones(4, 8), torch.ones(8, 8))
    assert torch.allclose(ml[0], om, atol=1e-5) and torch.allclose(zl[0], oz, atol=1e-5)


def test_kernel_api_cpu_semantics():
    from fastfold.model.fastnn.kernel import bias_dropout_add, bias_ele_dropout_residual, bias_sigmod_ele, fused_softmax
    torch.manual_seed(0)
    x, b, r = torch.randn(1, 3, 5, 8), torch.randn(8), torch.randn(1, 3, 5, 8)
    ones = torch.ones(1, 1, 5, 8)
    assert torch.allclose(bias_dropout_add(x, b, ones, r, prob=0.3, training=False), r + x + b, atol=1e-6)
    g = torch.rand(1, 3, 5, 8)
    assert torch.allclose(bias_ele_dropout_residual(x, b, g, ones, r, prob=0.3, training=False), r + g * (x + b), atol=1e-6)
    assert torch.allclose(bias_sigmod_ele(x, b, r), torch.sigmoid(x + b) * r, atol=1e-6)
    lg = torch.randn(1, 2, 3, 4, 4)
    mask = torch.tensor([[[1., 1, 0, 1], [1, 1, 1, 1]]])
    y = fused_softmax(lg, mask)
    assert torch.allclose(y.sum(-1), torch.ones(1, 2, 3, 4)) and float(y[0, 0, :, :, 2].abs().max()) < 1e-6
