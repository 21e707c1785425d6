"""Plain (non tensor-parallel) linear layer on sharded parameters (reference: ``bmtrain/nn/linear.py:6-56``)."""
import torch

from ..layer import DistributedModule
from ..ops import gemm as _gemm
from ..parameter import DistributedParameter


class OpLinear(torch.autograd.Function):
    """``x W^T + b`` with explicit dgrad / wgrad / bgrad."""

    @staticmethod
    def forward(ctx, x, weight, bias=None):
        return _gemm.LinearFunction.forward(ctx, x, weight, bias)

    @staticmethod
    def backward(ctx, grad_output):
        return _gemm.LinearFunction.backward(ctx, grad_output)


class Linear(DistributedModule):
    """``y = x W^T + b`` with ``W`` of shape (out_features, in_features), Xavier-normal initialised."""

    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype=None) -> None:
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight = DistributedParameter(
            torch.empty(out_features, in_features, dtype=dtype, device="meta"),
            init_method=torch.nn.init.xavier_normal_)
        if bias:
            self.bias = DistributedParameter(torch.empty(out_features, dtype=dtype, device="meta"),
                                             init_method=torch.nn.init.zeros_)
        else:
            self.register_parameter("bias", None)

    def forward(self, input):
        return _gemm.linear(input, self.weight, self.bias)

    def extra_repr(self) -> str:
        return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}"
