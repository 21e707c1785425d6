"""Vocabulary-parallel embedding (reference: ``bmtrain/nn/parallel_embedding.py:12-59``).

The table ``(vocab, d)`` is split by rows over the tensor-parallel group.
Lookup is Megatron-style: every rank looks up the ids that fall in its shard
(zeros elsewhere) and the partial embeddings are summed over the group -- the
reference instead all-gathers the whole table on every call.  With
``projection=True`` the module is the LM head: tokens are all-gathered and
multiplied by the local vocabulary shard, giving logits ``(..., vocab / tp)``.
"""
import torch

from ..global_var import config
from ..layer import DistributedModule
from ..ops import embedding as _emb
from ..parameter import DistributedParameter, ParameterInitializer
from .parallel_linear_func import OpParallelLinear


class _VocabParallelLookup(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight, start):
        comm = config["tp_comm"]
        local = ids - start
        inside = (local >= 0) & (local < weight.shape[0])
        out = _emb.embedding_forward(torch.where(inside, local, torch.full_like(local, -1)), weight)
        if comm is not None:
            comm.all_reduce(out, "sum")
        ctx.save_for_backward(local, inside)
        ctx.rows = weight.shape[0]
        return out

    @staticmethod
    def backward(ctx, grad):
        local, inside = ctx.saved_tensors
        idx = torch.where(inside, local, torch.full_like(local, -1))
        return None, _emb.embedding_backward(idx, grad.contiguous(), ctx.rows), None


class VPEmbedding(DistributedModule):
    """Embedding whose vocabulary is sharded over the tensor-parallel group."""

    def __init__(self, vocab_size: int, embedding_size: int, dtype: torch.dtype = torch.half,
                 init_mean: float = 0.0, init_std: float = 1):
        super().__init__()
        self.dim_model = embedding_size
        tp = config["tp_size"]
        assert vocab_size % tp == 0
        self.vocab_size_per_partition = vocab_size // tp
        self.start_index = config["tp_rank"] * self.vocab_size_per_partition
        self.end_index = (config["tp_rank"] + 1) * self.vocab_size_per_partition
        self.weight = DistributedParameter(
            torch.empty(self.vocab_size_per_partition, embedding_size, dtype=dtype, device="meta"),
            init_method=ParameterInitializer(torch.nn.init.normal_, mean=init_mean, std=init_std),
            tp_split_dim=0, tp_mode=True)

    def forward(self, x: torch.Tensor, projection: bool = False):
        if not projection:
            return _VocabParallelLookup.apply(x, self.weight, self.start_index)
        if config["tp_size"] > 1:
            # (tokens/tp, ...) on every rank -> all tokens, sequence-major per sample
            return OpParallelLinear.apply(x, self.weight, None, True, False, False, None, 1)
        return OpParallelLinear.apply(x, self.weight, None, False, False, False, None, 1)


ParallelEmbedding = VPEmbedding
