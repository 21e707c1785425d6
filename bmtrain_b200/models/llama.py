"""Llama-shaped decoder: RMSNorm, rotary position embedding, SwiGLU FFN, grouped-query attention.

The reference ships no such model; it is here because the 13B / 70B shaped
configurations need one.  Built from the same sharded-parameter modules as
:mod:`bmtrain_b200.models.gpt`.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ..block_layer import Block, TransformerBlockList
from ..global_var import config
from ..layer import DistributedModule
from ..nn import ColumnParallelLinear, Embedding, Linear, RMSNorm, RowParallelLinear, VPEmbedding
from ..ops import attention as _attn
from ..ops import elementwise as _ew


class LlamaAttention(DistributedModule):
    def __init__(self, dim_model: int, num_heads: int, num_kv_heads: int, dim_head: int, dtype=None, rope_theta: float = 10000.0):
        super().__init__()
        tp = config["tp_size"]
        assert num_heads % tp == 0 and num_kv_heads % tp == 0 and num_heads % num_kv_heads == 0
        self.h, self.hk, self.dh = num_heads // tp, num_kv_heads // tp, dim_head
        out_qkv = (num_heads + 2 * num_kv_heads) * dim_head
        if tp > 1:
            self.project_qkv = ColumnParallelLinear(dim_model, out_qkv, bias=False, dtype=dtype)
            self.project_out = RowParallelLinear(num_heads * dim_head, dim_model, bias=False, dtype=dtype)
        else:
            self.project_qkv = Linear(dim_model, out_qkv, bias=False, dtype=dtype)
            self.project_out = Linear(num_heads * dim_head, dim_model, bias=False, dtype=dtype)
        self.rope_theta = rope_theta

    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        tp = config["tp_size"]
        qkv = self.project_qkv(hidden)
        if tp > 1:
            s, b = qkv.shape[0], qkv.shape[1]
            qkv = qkv.view(s, b, self.hk, self.h // self.hk + 2, self.dh).permute(1, 0, 2, 3, 4)
        else:
            b, s = qkv.shape[0], qkv.shape[1]
            qkv = qkv.view(b, s, self.hk, self.h // self.hk + 2, self.dh)
        q, k, v = _ew.rope_qkv(qkv, self.h // self.hk, self.rope_theta)
        out = _attn.attention(q, k, v, 1.0 / math.sqrt(self.dh), causal=True)
        if tp > 1:
            out = out.permute(1, 0, 2, 3).reshape(s, b, self.h * self.dh)
        else:
            out = out.reshape(b, s, self.h * self.dh)
        return self.project_out(out)


class LlamaMLP(DistributedModule):
    """``w_out(silu(gate) * up)`` with gate and up projections fused into one GEMM (interleaved per TP rank)."""

    def __init__(self, dim_model: int, dim_ff: int, dtype=None):
        super().__init__()
        if config["tp_size"] > 1:
            self.w_gate_up = ColumnParallelLinear(dim_model, 2 * dim_ff, bias=False, dtype=dtype)
            self.w_out = RowParallelLinear(dim_ff, dim_model, bias=False, dtype=dtype)
        else:
            self.w_gate_up = Linear(dim_model, 2 * dim_ff, bias=False, dtype=dtype)
            self.w_out = Linear(dim_ff, dim_model, bias=False, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.w_out(_ew.swiglu(self.w_gate_up(x)))


class LlamaBlock(DistributedModule):
    def __init__(self, dim_model, num_heads, num_kv_heads, dim_head, dim_ff, dtype=None, eps=1e-5):
        super().__init__()
        self.ln_attn = RMSNorm(dim_model, eps=eps, dtype=dtype)
        self.attn = LlamaAttention(dim_model, num_heads, num_kv_heads, dim_head, dtype=dtype)
        self.ln_ff = RMSNorm(dim_model, eps=eps, dtype=dtype)
        self.ff = LlamaMLP(dim_model, dim_ff, dtype=dtype)

    def forward(self, hidden: torch.Tensor) -> torch.Tensor:
        hidden = hidden + self.attn(self.ln_attn(hidden))
        return hidden + self.ff(self.ln_ff(hidden))


class Llama(DistributedModule):
    """``forward(input_ids (b, s)) -> logits`` ((b, s, vocab), or (s, b, vocab/tp) under tensor parallelism)."""

    def __init__(self, num_layers: int, vocab_size: int, dim_model: int, num_heads: int, dim_ff: int,
                 num_kv_heads: Optional[int] = None, dim_head: Optional[int] = None, dtype=None,
                 zero_level: int = 3, use_checkpoint: bool = True, init_std: float = 0.02):
        super().__init__()
        num_kv_heads = num_kv_heads or num_heads
        dim_head = dim_head or dim_model // num_heads
        tp = config["tp_size"]
        emb = VPEmbedding if tp > 1 else Embedding
        self.word_emb = emb(vocab_size, dim_model, dtype=dtype, init_std=init_std)
        self.lm_head = emb(vocab_size, dim_model, dtype=dtype, init_std=init_std)
        blocks = [Block(LlamaBlock(dim_model, num_heads, num_kv_heads, dim_head, dim_ff, dtype=dtype),
                        use_checkpoint=use_checkpoint, zero_level=zero_level,
                        mode="PIPE" if config["pipe_size"] > 1 else "BLOCK") for _ in range(num_layers)]
        if config["pipe_size"] > 1:
            from ..pipe_layer import PipelineTransformerBlockList

            self.transformers = PipelineTransformerBlockList(blocks)
        else:
            self.transformers = TransformerBlockList(blocks)
        self.layernorm = RMSNorm(dim_model, dtype=dtype)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        tp = config["tp_size"]
        if tp > 1:
            input = input.chunk(tp, dim=1)[config["tp_rank"]].t().contiguous()
        out = self.word_emb(input)
        out = self.transformers(out)
        out = self.layernorm(out)
        return self.lm_head(out, projection=True)
