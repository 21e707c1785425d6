"""Cross-entropy kernels.

Forward is ONE pass over the logits (online softmax): per row it produces the
loss and the log-sum-exp; no softmax matrix is materialised.  Backward
recomputes ``exp(x - lse)`` from the logits and the saved log-sum-exp.
The reference materialises a full softmax (``csrc/cuda/cross_entropy.cu:9-121``,
three passes per row); the interface functions with its names are kept in
``bmtrain_b200/loss/_function.py``.

The same two kernels serve the vocab-parallel loss: ``row_stats`` returns the
local (max, sum-exp relative to that max, target logit) triple of a vocabulary
shard, the caller combines them over the tensor-parallel group, and
``ce_backward`` takes the global log-sum-exp and the shard's vocabulary offset.
"""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from . import _native

_DT = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def row_stats(logits: torch.Tensor, target: torch.Tensor, vocab_start: int = 0) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per row of ``logits`` (m, n): ``(max, sum_j exp(x_j - max), x[target - vocab_start] or 0 if outside the shard)``; all fp32."""
    m, n = logits.shape
    if not logits.is_cuda:
        x = logits.float()
        mx = x.max(dim=-1).values
        se = torch.exp(x - mx[:, None]).sum(dim=-1)
        local = target.long() - vocab_start
        inside = (local >= 0) & (local < n)
        tl = torch.where(inside, x.gather(1, local.clamp(0, n - 1)[:, None])[:, 0], torch.zeros_like(mx))
        return mx, se, tl
    assert logits.is_contiguous()
    target = target.to(torch.int64).contiguous()
    out = torch.empty(3, m, dtype=torch.float32, device=logits.device)
    _native.check(_native.cuda_lib().bmt_ce_row_stats(
        ctypes.c_int64(m), ctypes.c_int64(n), _native.ptr(logits), ctypes.c_int(_DT[logits.dtype]), _native.ptr(target),
        ctypes.c_int64(vocab_start), _native.ptr(out), _native.stream_handle()), "cross-entropy forward kernel")
    return out[0], out[1], out[2]


def ce_backward(logits: torch.Tensor, target: torch.Tensor, lse: torch.Tensor, grad_loss: torch.Tensor,
                vocab_start: int = 0, ignore_index: int = -100, inplace: bool = False) -> torch.Tensor:
    """``grad[i, j] = (exp(x[i,j] - lse[i]) - 1{j == target[i] - vocab_start}) * grad_loss[i]``; rows whose target is ``ignore_index`` give 0."""
    m, n = logits.shape
    if not logits.is_cuda:
        x = logits.float()
        g = torch.exp(x - lse[:, None].float())
        local = target.long() - vocab_start
        inside = (local >= 0) & (local < n)
        rows = torch.nonzero(inside, as_tuple=True)[0]
        g[rows, local[rows]] -= 1.0
        g = g * grad_loss.float()[:, None]
        g[target == ignore_index] = 0
        return g.to(logits.dtype)
    assert logits.is_contiguous()
    out = logits if inplace else torch.empty_like(logits)
    target = target.to(torch.int64).contiguous()
    _native.check(_native.cuda_lib().bmt_ce_backward(
        ctypes.c_int64(m), ctypes.c_int64(n), _native.ptr(logits), ctypes.c_int(_DT[logits.dtype]), _native.ptr(target),
        _native.ptr(lse.contiguous()), _native.ptr(grad_loss.float().contiguous()), ctypes.c_int64(vocab_start),
        ctypes.c_int64(ignore_index), _native.ptr(out), _native.stream_handle()), "cross-entropy backward kernel")
    return out
