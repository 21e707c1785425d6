from .cross_entropy import FusedCrossEntropy, OpFusedCrossEntropy, VPFusedCrossEntropy
