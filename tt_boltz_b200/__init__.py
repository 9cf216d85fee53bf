"""B200-native (sm_100a) Boltz-2 Pairformer trunk: hand-written CUDA kernels behind the
reference's PairformerModule / PairformerLayer call surface.  See include/b200pf.h for the C ABI."""
from .pairformer import (B200PairformerLayer, B200PairformerModule, B200PairformerNoSeqLayer,
                         B200PairformerNoSeqModule, B200PairUpdateBlock)

from .msa import B200MSALayer, B200MSAModule, B200MSAStack, B200MSATransition, B200OuterProductMean, B200PairWeightedAveraging
from .recycling import B200DistogramModule, B200RecyclingTrunk

__all__ = ["B200DistogramModule", "B200MSALayer", "B200MSAModule", "B200MSAStack", "B200MSATransition", "B200OuterProductMean", "B200PairWeightedAveraging", "B200RecyclingTrunk", "B200PairformerLayer", "B200PairformerModule", "B200PairformerNoSeqLayer", "B200PairformerNoSeqModule", "B200PairUpdateBlock"]
