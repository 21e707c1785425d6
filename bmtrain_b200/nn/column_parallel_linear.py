"""Column-parallel linear: the output features are split over the tensor-parallel group
(reference: ``bmtrain/nn/column_parallel_linear.py:9-80``)."""
import torch

from ..global_var import config
from ..layer import DistributedModule
from ..parameter import DistributedParameter
from .parallel_linear_func import OpParallelLinear


class ColumnParallelLinear(DistributedModule):
    """``y_local = gather_tokens(x) W_r^T + b_r`` with ``W_r`` = rows ``[r*out/tp, (r+1)*out/tp)`` of the full weight.

    Args:
        gather_input: ``x`` holds 1/tp of the tokens (sequence-sharded); gather them first.
        gather_output: return the full feature dim instead of this rank's slice.
        async_gather_chunks: accepted for compatibility (overlap is tile-granular inside the fused kernel).
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype=None,
                 gather_output=False, gather_input=True, async_gather_chunks=2):
        super().__init__()
        assert in_features % 1 == 0
        self.in_features = in_features
        self.out_features = out_features
        self.gather_output = gather_output
        self.gather_input = gather_input
        self.async_gather_chunks = async_gather_chunks
        tp_size = config["tp_size"]
        assert out_features % tp_size == 0
        self.out_features_per_partition = out_features // tp_size
        self.weight = DistributedParameter(
            torch.empty(self.out_features_per_partition, in_features, dtype=dtype, device="meta"),
            init_method=torch.nn.init.xavier_normal_, tp_split_dim=0, tp_mode=True)
        if bias:
            self.bias = DistributedParameter(
                torch.empty(self.out_features_per_partition, dtype=dtype, device="meta"),
                init_method=torch.nn.init.zeros_, tp_split_dim=0, tp_mode=True)
        else:
            self.register_parameter("bias", None)

    def forward(self, input):
        return OpParallelLinear.apply(input, self.weight, self.bias, self.gather_input, self.gather_output,
                                      False, None, self.async_gather_chunks)

    def extra_repr(self) -> str:
        return (f"in_features={self.in_features}, out_features={self.out_features_per_partition}, "
                f"bias={self.bias is not None}")
