"""Vocabulary-parallel embedding (reference: ``bmtrain/nn/parallel_embedding.py:12-59``).

The table ``(vocab, d)`` is split by rows over the tensor-parallel group.
Lookup: token ids (sharded along dim 0 over the same group, as the sequence-parallel activations are) are
all-gathered, every rank looks up the ids that fall in its shard (zeros elsewhere) and a reduce-scatter over the
token dim sums the shards and returns each rank's own tokens -- the reference instead all-gathers the whole
table on every call.  With
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
    """Lookup in a row-sharded table for tokens that are themselves sharded (dim 0) over the same group.

    Token ids are tiny, so they are all-gathered; every rank looks up the ids that fall into its vocabulary shard
    (zeros elsewhere) for *all* tokens and a reduce-scatter over the token dim both sums the shards' contributions
    and hands every rank the embeddings of its own tokens.  Backward all-gathers the gradient and scatter-adds the
    rows this rank owns."""

    @staticmethod
    def forward(ctx, ids, weight, start):
        comm = config["tp_comm"]
        tp = comm.size if comm is not None else 1
        ids = ids.contiguous()
        if tp > 1:
            all_ids = torch.empty((tp * ids.shape[0],) + tuple(ids.shape[1:]), dtype=ids.dtype, device=ids.device)
            comm.all_gather_into(all_ids, ids)
        else:
            all_ids = ids
        local = all_ids - start
        inside = (local >= 0) & (local < weight.shape[0])
        idx = torch.where(inside, local, torch.full_like(local, -1))
        partial = _emb.embedding_forward(idx, weight)
        if tp > 1:
            out = torch.empty((ids.shape[0],) + tuple(partial.shape[1:]), dtype=partial.dtype, device=partial.device)
            comm.reduce_scatter_into(out, partial.contiguous(), "sum")
        else:
            out = partial
        ctx.save_for_backward(idx)
        ctx.rows, ctx.tp = weight.shape[0], tp
        return out

    @staticmethod
    def backward(ctx, grad):
        (idx,) = ctx.saved_tensors
        comm = config["tp_comm"]
        grad = grad.contiguous()
        if ctx.tp > 1:
            g_all = torch.empty((ctx.tp * grad.shape[0],) + tuple(grad.shape[1:]), dtype=grad.dtype, device=grad.device)
            comm.all_gather_into(g_all, grad)
        else:
            g_all = grad
        return None, _emb.embedding_backward(idx, g_all, ctx.rows), None


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
