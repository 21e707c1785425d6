"""Embedding gather / scatter-add kernels (the reference uses ``F.embedding``).

Index ``-1`` means "not in this shard": forward writes zeros, backward skips the row.
"""
from __future__ import annotations

import ctypes

import torch

from . import _native

_DT = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def embedding_forward(ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """``out[..., :] = weight[ids[...]]`` (zeros where ``ids < 0``)."""
    d = weight.shape[1]
    if not weight.is_cuda:
        safe = ids.clamp(min=0)
        out = weight[safe.reshape(-1)].view(*ids.shape, d)
        return out * (ids >= 0).unsqueeze(-1).to(out.dtype)
    ids64 = ids.to(torch.int64).contiguous()
    out = torch.empty(*ids.shape, d, dtype=weight.dtype, device=weight.device)
    _native.check(_native.cuda_lib().bmt_embedding_fwd(
        ctypes.c_int64(ids64.numel()), ctypes.c_int64(d), _native.ptr(ids64), _native.ptr(weight.contiguous()),
        ctypes.c_int(_DT[weight.dtype]), _native.ptr(out), _native.stream_handle()), "embedding forward kernel")
    return out


def embedding_backward(ids: torch.Tensor, grad: torch.Tensor, rows: int) -> torch.Tensor:
    """``grad_weight[ids[t]] += grad[t]`` accumulated in fp32, returned in ``grad``'s dtype."""
    d = grad.shape[-1]
    g2 = grad.reshape(-1, d)
    flat = ids.reshape(-1)
    if not grad.is_cuda:
        acc = torch.zeros(rows, d, dtype=torch.float32)
        keep = flat >= 0
        acc.index_add_(0, flat[keep], g2[keep].float())
        return acc.to(grad.dtype)
    acc = torch.zeros(rows, d, dtype=torch.float32, device=grad.device)
    ids64 = flat.to(torch.int64).contiguous()
    _native.check(_native.cuda_lib().bmt_embedding_bwd(
        ctypes.c_int64(ids64.numel()), ctypes.c_int64(d), _native.ptr(ids64), _native.ptr(g2.contiguous()),
        ctypes.c_int(_DT[grad.dtype]), _native.ptr(acc), _native.stream_handle()), "embedding backward kernel")
    return acc.to(grad.dtype)


class EmbeddingFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, weight):
        ctx.save_for_backward(ids)
        ctx.rows = weight.shape[0]
        return embedding_forward(ids, weight)

    @staticmethod
    def backward(ctx, grad):
        (ids,) = ctx.saved_tensors
        return None, embedding_backward(ids, grad.contiguous(), ctx.rows)


def embedding(ids: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    return EmbeddingFunction.apply(ids, weight)
