"""LayerNorm and RMSNorm, forward and backward (the reference calls ``F.layer_norm``:
``example/layers/layernorm.py:29``; RMSNorm is needed by the Llama-shaped models).

One row per warp-group, single pass: the row is held in registers, statistics
in fp32; backward produces dx and per-CTA partial dgamma/dbeta that a second
tiny kernel folds.  CPU tensors use the PyTorch definition.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _native

_DT = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


class LayerNormFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, eps, rms):
        shape = x.shape
        d = shape[-1]
        x2 = x.reshape(-1, d).contiguous()
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        stats = torch.empty(2, rows, dtype=torch.float32, device=x.device)  # mean, rstd
        _native.check(_native.cuda_lib().bmt_norm_fwd(
            ctypes.c_int64(rows), ctypes.c_int64(d), _native.ptr(x2), _native.ptr(weight), _native.ptr(bias),
            ctypes.c_float(eps), ctypes.c_int(1 if rms else 0), ctypes.c_int(_DT[x.dtype]),
            _native.ptr(y), _native.ptr(stats), _native.stream_handle()), "norm forward kernel")
        ctx.save_for_backward(x2, weight, stats)
        ctx.rms, ctx.has_bias, ctx.shape = rms, bias is not None, shape
        return y.view(shape)

    @staticmethod
    def backward(ctx, grad):
        x2, weight, stats = ctx.saved_tensors
        rows, d = x2.shape
        g2 = grad.reshape(-1, d).contiguous()
        dx = torch.empty_like(x2)
        nblk = min(rows, 296)
        partial = torch.empty(2, nblk, d, dtype=torch.float32, device=x2.device)
        dw = torch.empty(d, dtype=weight.dtype, device=x2.device)
        db = torch.empty(d, dtype=weight.dtype, device=x2.device) if ctx.has_bias else None
        _native.check(_native.cuda_lib().bmt_norm_bwd(
            ctypes.c_int64(rows), ctypes.c_int64(d), _native.ptr(x2), _native.ptr(g2), _native.ptr(weight),
            _native.ptr(stats), ctypes.c_int(1 if ctx.rms else 0), ctypes.c_int(_DT[x2.dtype]), ctypes.c_int(nblk),
            _native.ptr(dx), _native.ptr(partial), _native.ptr(dw), _native.ptr(db),
            _native.stream_handle()), "norm backward kernel")
        return dx.view(ctx.shape), dw, db, None, None


def layer_norm(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], eps: float = 1e-5) -> torch.Tensor:
    if not x.is_cuda:
        return torch.nn.functional.layer_norm(x, (x.shape[-1],), weight, bias, eps)
    return LayerNormFunction.apply(x, weight, bias, eps, False)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    if not x.is_cuda:
        xf = x.float()
        y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
        return (y * weight.float()).to(x.dtype)
    return LayerNormFunction.apply(x, weight, None, eps, True)
