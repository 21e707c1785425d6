"""Names accepted by the tensor-level communication calls (reference: ``bmtrain/nccl/enums.py``)."""
import torch

REDUCE_OPS = ("sum", "prod", "max", "min", "avg")
DTYPE_NAMES = {
    torch.int8: "int8", torch.uint8: "uint8", torch.int32: "int32", torch.int64: "int64",
    torch.float16: "float16", torch.bfloat16: "bfloat16", torch.float32: "float32", torch.float64: "float64",
}
