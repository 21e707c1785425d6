"""GPT-2 style decoder (layout of the reference example: ``example/models/gpt.py``, ``example/layers/*.py``).

Pre-LN blocks: LN -> attention -> residual -> LN -> FFN -> residual; learned
position embedding; final LN; LM head tied to the word embedding.  Blocks are
``bmt.Block``s in a ``TransformerBlockList`` (or a ``PipelineTransformerBlockList``
when pipeline parallelism is on); with ``tp_size > 1`` the projections are
column/row parallel and activations between them are sequence-sharded.
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch

from .. import inspect as bmt_inspect
from ..block_layer import Block, TransformerBlockList
from ..global_var import config
from ..layer import DistributedModule
from ..nn import ColumnParallelLinear, Embedding, LayerNorm, Linear, RowParallelLinear, VPEmbedding
from ..ops import attention as _attn
from ..ops import gpt_block as _gpt_block


# The per-operator module path below stays available (set BMT_FUSED_BLOCK=0) for debugging and as the general fallback.
_FUSED_BLOCK = os.environ.get("BMT_FUSED_BLOCK", "1") != "0"


class Attention(DistributedModule):
    """Multi-head self attention with a fused QKV projection."""

    def __init__(self, dim_model: int, dim_head: int, num_heads: int, bias: bool = True, dtype=None):
        super().__init__()
        tp = config["tp_size"]
        inner = dim_head * num_heads
        if tp > 1:
            assert num_heads % tp == 0
            self.project_qkv = ColumnParallelLinear(dim_model, 3 * inner, bias=bias, dtype=dtype)
            self.project_out = RowParallelLinear(inner, dim_model, bias=bias, dtype=dtype)
        else:
            self.project_qkv = Linear(dim_model, 3 * inner, bias=bias, dtype=dtype)
            self.project_out = Linear(inner, dim_model, bias=bias, dtype=dtype)
        self.num_heads = num_heads
        self.local_heads = num_heads // tp
        self.dim_head = dim_head
        self.dim_model = dim_model

    def forward(self, hidden: torch.Tensor, mask: Optional[torch.Tensor], causal: bool = False) -> torch.Tensor:
        tp = config["tp_size"]
        qkv = self.project_qkv(hidden)
        if tp > 1:
            # hidden is (s/tp, b, d) sequence-sharded; the gathered projection is (s, b, 3*inner/tp)
            s, b = qkv.shape[0], qkv.shape[1]
            qkv = qkv.view(s, b, self.local_heads, 3, self.dim_head).permute(1, 0, 2, 3, 4)
        else:
            b, s = qkv.shape[0], qkv.shape[1]
            qkv = qkv.view(b, s, self.local_heads, 3, self.dim_head)
        q, k, v = qkv[:, :, :, 0], qkv[:, :, :, 1], qkv[:, :, :, 2]
        out = _attn.attention(q, k, v, 1.0 / math.sqrt(self.dim_head), causal=causal, mask=mask)
        if tp > 1:
            out = out.permute(1, 0, 2, 3).reshape(s, b, self.local_heads * self.dim_head)
        else:
            out = out.reshape(b, s, self.local_heads * self.dim_head)
        return self.project_out(out)


class Feedforward(DistributedModule):
    def __init__(self, dim_model: int, dim_ff: int, bias: bool = True, dtype=None, activation: str = "relu"):
        super().__init__()
        if config["tp_size"] > 1:
            self.w_in = ColumnParallelLinear(dim_model, dim_ff, bias=bias, dtype=dtype)
            self.w_out = RowParallelLinear(dim_ff, dim_model, bias=bias, dtype=dtype)
        else:
            self.w_in = Linear(dim_model, dim_ff, bias=bias, dtype=dtype)
            self.w_out = Linear(dim_ff, dim_model, bias=bias, dtype=dtype)
        self.activation = activation

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        h = self.w_in(x)
        h = torch.relu(h) if self.activation == "relu" else torch.nn.functional.gelu(h)
        return self.w_out(h)


class TransformerEncoder(DistributedModule):
    """One pre-LN block."""

    def __init__(self, dim_model: int, dim_head: int, num_heads: int, dim_ff: int, bias: bool = True, dtype=None,
                 activation: str = "relu", causal: bool = False):
        super().__init__()
        self.ln_attn = LayerNorm(dim_model, dtype=dtype)
        self.attn = Attention(dim_model, dim_head, num_heads, bias=bias, dtype=dtype)
        self.ln_ff = LayerNorm(dim_model, dtype=dtype)
        self.ff = Feedforward(dim_model, dim_ff, bias=bias, dtype=dtype, activation=activation)
        self.causal = causal

    # the ZeRO block may leave the gather of this weight to the GEMM that consumes it
    _bmt_first_gemm = "attn.project_qkv.weight"
    _bmt_deferred_gather = None

    def _bmt_can_fuse_first_gemm(self, hidden, *rest) -> bool:
        return torch.is_tensor(hidden) and self._fused_ok(hidden) and not bmt_inspect.tensor.debug.get("_inspect_tensor", False)

    def _fused_ok(self, hidden: torch.Tensor) -> bool:
        return (hidden.is_cuda and hidden.dim() == 3 and config["tp_size"] == 1 and _FUSED_BLOCK and self.attn.project_qkv.bias is not None
                and hidden.dtype in (torch.float16, torch.bfloat16) and self.attn.dim_head % 8 == 0)

    def forward(self, hidden: torch.Tensor, mask: Optional[torch.Tensor] = None, position_bias=None):
        bmt_inspect.record_tensor(hidden, "hidden")
        if self._fused_ok(hidden):
            # one native call per direction for the whole block (csrc/block_exec.cu)
            a, f = self.attn, self.ff
            deferred, self._bmt_deferred_gather = self._bmt_deferred_gather, None
            return _gpt_block.gpt_block(
                hidden, mask, a.num_heads, a.dim_head, f.activation, self.ln_attn.eps, self.causal,
                self.ln_attn.weight, self.ln_attn.bias, a.project_qkv.weight, a.project_qkv.bias,
                a.project_out.weight, a.project_out.bias, self.ln_ff.weight, self.ln_ff.bias,
                f.w_in.weight, f.w_in.bias, f.w_out.weight, f.w_out.bias, deferred=deferred)
        x = self.ln_attn(hidden)
        x = self.attn(x, mask, self.causal)
        hidden = hidden + x
        x = self.ln_ff(hidden)
        x = self.ff(x)
        return hidden + x.view_as(hidden)


class GPT(DistributedModule):
    """Decoder-only transformer.

    ``forward(input, pos, mask)`` with ``input``/``pos`` (batch, seq) int64 and
    ``mask`` (batch, seq) bool returns logits (batch, seq, vocab) -- or
    (seq, batch, vocab / tp) sequence-first vocabulary shards when tensor
    parallelism is on.  The attention mask is ``mask[b,i] & mask[b,j] & (pos[b,j] <= pos[b,i])``.
    """

    def __init__(self, num_layers: int, vocab_size: int, dim_model: int, dim_head: int, num_heads: int, dim_ff: int,
                 max_distance: int, bias: bool = True, dtype=None, activation: str = "relu",
                 zero_level: int = 3, use_checkpoint: bool = True, dense_mask: bool = True):
        super().__init__()
        self.max_distance = max_distance
        self.dense_mask = dense_mask
        if config["tp_size"] > 1:
            self.word_emb = VPEmbedding(vocab_size, dim_model, dtype=dtype)
        else:
            self.word_emb = Embedding(vocab_size, dim_model, dtype=dtype)
        self.pos_emb = Embedding(max_distance, dim_model, dtype=dtype)

        def make_block():
            return TransformerEncoder(dim_model, dim_head, num_heads, dim_ff, bias, dtype, activation, causal=not dense_mask)

        if config["pipe_size"] > 1:
            from ..pipe_layer import PipelineTransformerBlockList

            self.transformers = PipelineTransformerBlockList(
                [Block(make_block(), use_checkpoint=use_checkpoint, mode="PIPE") for _ in range(num_layers)])
        else:
            self.transformers = TransformerBlockList(
                [Block(make_block(), use_checkpoint=use_checkpoint, zero_level=zero_level) for _ in range(num_layers)])
        self.layernorm = LayerNorm(dim_model, dtype=dtype)

    def forward(self, input: torch.Tensor, pos: torch.Tensor, mask: torch.Tensor) -> torch.Tensor:
        tp = config["tp_size"]
        if self.dense_mask:
            mask_2d = mask[:, None, :] & mask[:, :, None] & (pos[:, None, :] <= pos[:, :, None])
        else:
            mask_2d = None
        if tp > 1:
            # sequence-first, sequence-sharded activations: (s/tp, b, d)
            r = config["tp_rank"]
            input = input.chunk(tp, dim=1)[r].t().contiguous()
            pos = pos.chunk(tp, dim=1)[r].t().contiguous()
        out = self.pos_emb(pos) + self.word_emb(input)
        out = self.transformers(out, mask_2d, None)
        out = self.layernorm(out)
        logits = self.word_emb(out, projection=True)
        bmt_inspect.record_tensor(logits, "logits")
        return logits
