from .cross_entropy import FusedCrossEntropy, OpFusedCrossEntropy, VPFusedCrossEntropy
from . import _function  # noqa: F401
