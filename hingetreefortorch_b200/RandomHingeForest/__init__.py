"""nn.Module layer of the hinge tree drop-in (same exported names as the reference package, plus
LinearBatchNorm1d, the tensor-core front of the reference's Linear -> BatchNorm1d -> forest pipeline, and
LinearBatchNormForest, that front and a forest as one step)."""
from ._RandomHingeForest import (  # noqa: F401
    RandomHingeForest, RandomHingeFern, RandomHingeTrie,
    SparseRandomHingeForest, SparseRandomHingeFern,
    RandomHingeForestFusedLinear, RandomHingeFernFusedLinear,
    SparseRandomHingeForestFusedLinear, SparseRandomHingeFernFusedLinear,
    RandomHingeForestFusion, RandomHingeFernFusion,
    RandomHingeForestFusionFusedLinear, RandomHingeFernFusionFusedLinear,
)
from ._HingeTreeConv import (  # noqa: F401
    HingeTreeConv1d, HingeTreeConv2d, HingeTreeConv3d, HingeFernConv1d, HingeFernConv2d, HingeFernConv3d,
)
from ._LinearBatchNorm import LinearBatchNorm1d, LinearBatchNormForest  # noqa: F401
