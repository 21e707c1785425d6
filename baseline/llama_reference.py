"""Llama-shaped decoder built from the REFERENCE's public API (``bmtrain`` as installed under ``baseline/_ref``), for
the reference arm of ``bench.py --config llama13b``.

The reference ships only a GPT example, so the decoder is assembled here from its stock pieces: ``bmt.nn.
ColumnParallelLinear`` / ``RowParallelLinear`` / ``VPEmbedding`` inside ``bmt.Block`` + ``bmt.TransformerBlockList``
(ZeRO-3, activation checkpointing), ``bmt.loss.FusedCrossEntropy(parallel=True)``.  RMSNorm, rotary embedding and SwiGLU
are plain PyTorch ops and the attention core is ``F.scaled_dot_product_attention`` (PyTorch's own fused attention), i.e.
what a user of the reference would write today.  Activations between the tensor-parallel regions are sequence-first
``(s / tp, b, d)``, the layout the reference's column/row linears gather and scatter along dim 0.
Nothing of this repository's package is imported here.
"""
import math

import torch
import torch.nn.functional as F

import bmtrain as bmt


def _rms(x, w, eps=1e-5):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype) * w


def _rope(x, theta=10000.0):
    # x (b, h, s, d): rotate the pairs (x[..., :d/2], x[..., d/2:]) by absolute position
    s, d = x.shape[2], x.shape[3]
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=x.device, dtype=torch.float32) / d))
    ang = torch.outer(torch.arange(s, device=x.device, dtype=torch.float32), inv)
    cos, sin = ang.cos()[None, None].to(x.dtype), ang.sin()[None, None].to(x.dtype)
    x1, x2 = x[..., : d // 2], x[..., d // 2:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1)


class RefLlamaBlock(bmt.DistributedModule):
    def __init__(self, d, h, hk, dh, dff, dtype):
        super().__init__()
        tp = bmt.config["tp_size"]
        self.h, self.hk, self.dh, self.dff = h // tp, hk // tp, dh, dff // tp
        self.ln_attn = bmt.DistributedParameter(torch.ones(d, dtype=dtype))
        self.ln_ff = bmt.DistributedParameter(torch.ones(d, dtype=dtype))
        self.qkv = bmt.nn.ColumnParallelLinear(d, (h + 2 * hk) * dh, bias=False, dtype=dtype)
        self.out = bmt.nn.RowParallelLinear(h * dh, d, bias=False, dtype=dtype)
        self.gate_up = bmt.nn.ColumnParallelLinear(d, 2 * dff, bias=False, dtype=dtype)
        self.down = bmt.nn.RowParallelLinear(dff, d, bias=False, dtype=dtype)

    def forward(self, x):                                   # (s / tp, b, d)
        qkv = self.qkv(_rms(x, self.ln_attn))               # (s, b, (h + 2 hk) dh / tp)
        s, b = qkv.shape[0], qkv.shape[1]
        g = self.h // self.hk
        qkv = qkv.view(s, b, self.hk, g + 2, self.dh)
        q = qkv[:, :, :, :g].reshape(s, b, self.h, self.dh).permute(1, 2, 0, 3)
        k = qkv[:, :, :, g].permute(1, 2, 0, 3)
        v = qkv[:, :, :, g + 1].permute(1, 2, 0, 3)
        q, k = _rope(q), _rope(k)
        if g > 1:
            k, v = k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1)
        o = F.scaled_dot_product_attention(q, k, v, is_causal=True, scale=1.0 / math.sqrt(self.dh))
        o = o.permute(2, 0, 1, 3).reshape(s, b, self.h * self.dh)
        x = x + self.out(o)                                  # (s / tp, b, d)
        gu = self.gate_up(_rms(x, self.ln_ff))
        return x + self.down(F.silu(gu[..., : self.dff]) * gu[..., self.dff:])


class RefLlama(bmt.DistributedModule):
    def __init__(self, num_layers, vocab_size, dim_model, num_heads, dim_ff, num_kv_heads=None, dim_head=None, dtype=torch.bfloat16):
        super().__init__()
        hk = num_kv_heads or num_heads
        dh = dim_head or dim_model // num_heads
        self.word_emb = bmt.nn.VPEmbedding(vocab_size, dim_model, dtype=dtype, init_std=0.02)
        self.lm_head = bmt.nn.VPEmbedding(vocab_size, dim_model, dtype=dtype, init_std=0.02)
        self.transformers = bmt.TransformerBlockList(
            [bmt.Block(RefLlamaBlock(dim_model, num_heads, hk, dh, dim_ff, dtype)) for _ in range(num_layers)])
        self.layernorm = bmt.DistributedParameter(torch.ones(dim_model, dtype=dtype))

    def forward(self, ids):                                  # (b, s) -> (s, b, vocab / tp)
        tp = bmt.config["tp_size"]
        ids = ids.chunk(tp, dim=1)[bmt.config["topology"].tp_id].t().contiguous()
        x = self.word_emb(ids)
        x = self.transformers(x)
        x = _rms(x, self.layernorm)
        # VPEmbedding's own projection path reinterprets the gathered (tp, s / tp, b, d) tensor with a plain view, which is
        # only the sequence order for batch-first inputs of batch 1; gather explicitly and call the same operator
        x = bmt.distributed.all_gather(x, comm=bmt.config["tp_comm"]).flatten(0, 1)
        return bmt.nn.OpParallelLinear.apply(x, self.lm_head.weight, None, False, False, False, None, 1)
