"""Hot ops of fastfold_b200: sm_100a kernels on CUDA tensors, PyTorch reference on CPU tensors."""
from .layer_norm import LayerNorm, FusedLayerNorm, layer_norm, layer_norm_transposed
from .softmax import fused_softmax
from .fused_ops import (bias_sigmod_ele, bias_dropout_add, bias_ele_dropout_residual, glu_mask, glu_mask_t, colsum,
                        global_attention_core, global_attention_ref)
from . import gemm as gemm_mod
from .gemm import gemm, gemm_ref, linear, linear_t, linear_t_multi, bmm_nt, weight_grad

__all__ = [
    "LayerNorm", "FusedLayerNorm", "layer_norm", "layer_norm_transposed", "fused_softmax", "bias_sigmod_ele",
    "bias_dropout_add", "bias_ele_dropout_residual", "glu_mask", "colsum", "gemm", "gemm_ref", "linear", "bmm_nt",
    "weight_grad",
]
