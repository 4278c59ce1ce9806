"""Autograd functions of the hinge tree drop-in (same exported names as the reference package)."""
from ._HingeTree import (  # noqa: F401
    contract, expand, Contract, Expand,
    HingeTree, HingeFern, SparseHingeTree, SparseHingeFern,
    HingeTreeFusedLinear, HingeFernFusedLinear, SparseHingeTreeFusedLinear, SparseHingeFernFusedLinear,
    HingeTreeFusion, HingeFernFusion, HingeTreeFusionFusedLinear, HingeFernFusionFusedLinear,
    HingeTreeConv1d, HingeTreeConv2d, HingeTreeConv3d, HingeFernConv1d, HingeFernConv2d, HingeFernConv3d,
    HingeTrie,
)
