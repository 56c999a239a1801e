from .msa import MSACore, ExtraMSACore, ExtraMSABlock, ExtraMSAStack
from .ops import OutProductMean, set_chunk_size, get_chunk_size
from .triangle import PairCore
from .evoformer import Evoformer, EvoformerStack

__all__ = [
    "MSACore", "OutProductMean", "PairCore", "set_chunk_size", "get_chunk_size", "ExtraMSACore", "ExtraMSABlock",
    "ExtraMSAStack", "Evoformer", "EvoformerStack",
]
