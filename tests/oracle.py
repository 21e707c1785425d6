"""Plain-PyTorch fp32 models with the same parameter names as ``bmtrain_b200.models`` -- the numerical oracle."""
import math

import torch
import torch.nn as nn
import torch.nn.functional as F


class OracleBlock(nn.Module):
    def __init__(self, d, dh, h, dff, bias=True, activation="relu"):
        super().__init__()
        self.ln_attn = nn.LayerNorm(d)
        self.attn = nn.Module()
        self.attn.project_qkv = nn.Linear(d, 3 * h * dh, bias=bias)
        self.attn.project_out = nn.Linear(h * dh, d, bias=bias)
        self.ln_ff = nn.LayerNorm(d)
        self.ff = nn.Module()
        self.ff.w_in = nn.Linear(d, dff, bias=bias)
        self.ff.w_out = nn.Linear(dff, d, bias=bias)
        self.h, self.dh, self.activation = h, dh, activation

    def forward(self, hidden, mask):
        b, s, _ = hidden.shape
        x = self.ln_attn(hidden)
        qkv = self.attn.project_qkv(x).view(b, s, self.h, 3, self.dh)
        q, k, v = qkv[:, :, :, 0], qkv[:, :, :, 1], qkv[:, :, :, 2]
        score = torch.einsum("bqhd,bkhd->bhqk", q, k) / math.sqrt(self.dh)
        if mask is not None:
            score = score.masked_fill(~mask[:, None], float("-inf"))
        p = torch.softmax(score, dim=-1)
        if mask is not None:
            p = torch.where(mask[:, None], p, torch.zeros_like(p))
        p = torch.nan_to_num(p)
        o = torch.einsum("bhqk,bkhd->bqhd", p, v).reshape(b, s, self.h * self.dh)
        hidden = hidden + self.attn.project_out(o)
        x = self.ln_ff(hidden)
        x = self.ff.w_in(x)
        x = torch.relu(x) if self.activation == "relu" else F.gelu(x)
        return hidden + self.ff.w_out(x)


class OracleGPT(nn.Module):
    def __init__(self, num_layers, vocab, d, dh, h, dff, max_distance, bias=True, activation="relu"):
        super().__init__()
        self.word_emb = nn.Embedding(vocab, d)
        self.pos_emb = nn.Embedding(max_distance, d)
        self.transformers = nn.ModuleList([OracleBlock(d, dh, h, dff, bias, activation) for _ in range(num_layers)])
        self.layernorm = nn.LayerNorm(d)

    def forward(self, input, pos, mask):
        mask_2d = mask[:, None, :] & mask[:, :, None] & (pos[:, None, :] <= pos[:, :, None])
        out = self.pos_emb(pos) + self.word_emb(input)
        for blk in self.transformers:
            out = blk(out, mask_2d)
        out = self.layernorm(out)
        return F.linear(out, self.word_emb.weight)
