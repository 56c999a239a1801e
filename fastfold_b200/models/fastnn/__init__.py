from .msa import MSACore, ExtraMSACore, ExtraMSABlock, ExtraMSAStack
from .ops import OutProductMean, set_chunk_size, get_chunk_size
from .triangle import PairCore
from .evoformer import Evoformer, EvoformerStack
from .template import TemplatePairBlock, TemplatePairStack

__all__ = [
    "MSACore", "OutProductMean", "PairCore", "TemplatePairBlock", "TemplatePairStack", "set_chunk_size", "get_chunk_size", "ExtraMSACore",
    "ExtraMSABlock", "ExtraMSAStack", "Evoformer", "EvoformerStack",
]
