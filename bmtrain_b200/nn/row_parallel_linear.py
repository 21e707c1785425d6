"""Row-parallel linear: the input features are split over the tensor-parallel group
(reference: ``bmtrain/nn/row_parallel_linear.py:9-88``)."""
import torch

from ..global_var import config
from ._tp_linear import ShardedLinearBase
from .parallel_linear_func import OpParallelLinear, ReduceType


class _AddReplicatedBias(torch.autograd.Function):
    """``out + bias`` where ``out`` holds only this rank's share of the tokens but ``bias`` is replicated over the
    tensor-parallel group: the bias gradient is the sum over *all* tokens, so it is all-reduced over the group
    (the reference leaves the per-rank partial sums: ``bmtrain/nn/row_parallel_linear.py:81-82``)."""

    @staticmethod
    def forward(ctx, out, bias):
        return out + bias

    @staticmethod
    def backward(ctx, grad):
        gb = grad.reshape(-1, grad.shape[-1]).sum(0)
        comm = config["tp_comm"]
        if comm is not None:
            comm.all_reduce(gb, "sum")
        return grad, gb


class RowParallelLinear(ShardedLinearBase):
    """``y = reduce(x_r W_r^T) + b`` with ``W_r`` = columns ``[r*in/tp, (r+1)*in/tp)`` of the full weight.

    By default the partial products are reduce-scattered over the token dim
    (each rank keeps 1/tp of the tokens); ``all_reduce_output=True`` returns all
    tokens on every rank.  ``split_input=True`` takes the full feature dim and
    slices it.  The bias is replicated and added after the reduction.
    """

    def __init__(self, in_features: int, out_features: int, bias: bool = True, dtype=None,
                 split_input=False, all_reduce_output=False, async_chunks=2):
        super().__init__(in_features, out_features, bias, dtype, split_dim=1)
        self.in_features_per_partition = in_features // config["tp_size"]
        self.split_input, self.all_reduce_output, self.async_chunks = split_input, all_reduce_output, async_chunks

    def forward(self, input):
        reduce_type = ReduceType.ALL_REDUCE.value if self.all_reduce_output else ReduceType.REDUCE_SCATTER.value
        out = OpParallelLinear.apply(input, self.weight, None, self.split_input, False, self.split_input,
                                     reduce_type, self.async_chunks)
        if self.bias is None:
            return out
        if config["tp_size"] > 1 and not self.all_reduce_output:
            return _AddReplicatedBias.apply(out, self.bias)
        return out + self.bias
