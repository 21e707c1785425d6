"""Column-parallel linear: the output features are split over the tensor-parallel group
(reference: ``bmtrain/nn/column_parallel_linear.py:9-80``)."""
from ..global_var import config
from ._tp_linear import ShardedLinearBase
from .parallel_linear_func import OpParallelLinear


class ColumnParallelLinear(ShardedLinearBase):
    """``y_local = gather_tokens(x) W_r^T + b_r`` with ``W_r`` = rows ``[r*out/tp, (r+1)*out/tp)`` of the full weight.

    Args:
        gather_input: ``x`` holds 1/tp of the tokens (sequence-sharded); gather them first.
        gather_output: return the full feature dim instead of this rank's slice.
        async_gather_chunks: accepted for compatibility (overlap is tile-granular inside the fused kernel).
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype=None,
                 gather_output=False, gather_input=True, async_gather_chunks=2):
        super().__init__(in_features, out_features, bias, dtype, split_dim=0)
        self.out_features_per_partition = out_features // config["tp_size"]
        self.gather_output, self.gather_input = gather_output, gather_input
        self.async_gather_chunks = async_gather_chunks

    def forward(self, input):
        return OpParallelLinear.apply(input, self.weight, self.bias, self.gather_input, self.gather_output,
                                      False, None, self.async_gather_chunks)
