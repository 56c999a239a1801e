"""The reference's ``fastfold.model.fastnn.kernel`` surface (kernel/__init__.py:1-13) on the sm_100a kernels."""
from .attention import fused_attention_core
from .fused_ops import bias_dropout_add, bias_ele_dropout_residual, bias_sigmod_ele
from .layer_norm import FusedLayerNorm as LayerNorm
from .softmax import fused_softmax

__all__ = ["LayerNorm", "fused_softmax", "fused_attention_core", "bias_dropout_add", "bias_sigmod_ele", "bias_ele_dropout_residual"]


def _set_jit_fusion_options():
    """The reference configures TorchScript's fusers here (kernel/jit/options.py:6-30).  Nothing is scripted in this
    package - the fusions are GEMM epilogues and CUDA kernels - so there is nothing to configure."""

