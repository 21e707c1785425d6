"""Shared construction of the two tensor-parallel linears: which dimension of the full ``(out, in)`` weight is cut
over the tensor-parallel group, and whether the bias is cut with it."""
import torch

from ..global_var import config
from ..layer import DistributedModule
from ..parameter import DistributedParameter


class ShardedLinearBase(DistributedModule):
    """Holds ``weight`` = the slice of the full ``(out_features, in_features)`` matrix along ``split_dim`` that belongs
    to this tensor-parallel rank, and ``bias`` (cut along the output features when ``split_dim == 0``, replicated
    otherwise)."""

    def __init__(self, in_features: int, out_features: int, bias: bool, dtype, split_dim: int):
        super().__init__()
        tp = config["tp_size"]
        full = [out_features, in_features]
        if full[split_dim] % tp:
            raise ValueError(f"{'out_features' if split_dim == 0 else 'in_features'}={full[split_dim]} "
                             f"is not divisible by the tensor-parallel size {tp}")
        self.in_features, self.out_features = in_features, out_features
        local = list(full)
        local[split_dim] //= tp
        self.weight = DistributedParameter(torch.empty(*local, dtype=dtype, device="meta"),
                                           init_method=torch.nn.init.xavier_normal_, tp_split_dim=split_dim, tp_mode=True)
        if bias:
            self.bias = DistributedParameter(torch.empty(local[0], dtype=dtype, device="meta"),
                                             init_method=torch.nn.init.zeros_,
                                             tp_split_dim=0 if split_dim == 0 else -1, tp_mode=True)
        else:
            self.register_parameter("bias", None)

    def extra_repr(self) -> str:
        out_local, in_local = self.weight._original_shape
        return f"in_features={in_local}, out_features={out_local}, bias={self.bias is not None}"
