"""Small fused elementwise operators: SwiGLU and rotary position embedding."""
from __future__ import annotations

import ctypes
from typing import Tuple

import torch

from . import _native

_DT = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


class SwiGLUFunction(torch.autograd.Function):
    """``silu(x[..., :f]) * x[..., f:]`` for the fused gate/up projection output ``x`` (..., 2f)."""

    @staticmethod
    def forward(ctx, x):
        f = x.shape[-1] // 2
        x2 = x.reshape(-1, 2 * f).contiguous()
        out = torch.empty(x2.shape[0], f, dtype=x.dtype, device=x.device)
        _native.check(_native.cuda_lib().bmt_swiglu_fwd(
            ctypes.c_int64(x2.shape[0]), ctypes.c_int64(f), _native.ptr(x2), ctypes.c_int(_DT[x.dtype]),
            _native.ptr(out), _native.stream_handle()), "swiglu forward kernel")
        ctx.save_for_backward(x2)
        ctx.shape = x.shape
        return out.view(*x.shape[:-1], f)

    @staticmethod
    def backward(ctx, grad):
        (x2,) = ctx.saved_tensors
        f = x2.shape[1] // 2
        g2 = grad.reshape(-1, f).contiguous()
        dx = torch.empty_like(x2)
        _native.check(_native.cuda_lib().bmt_swiglu_bwd(
            ctypes.c_int64(x2.shape[0]), ctypes.c_int64(f), _native.ptr(x2), _native.ptr(g2), ctypes.c_int(_DT[x2.dtype]),
            _native.ptr(dx), _native.stream_handle()), "swiglu backward kernel")
        return dx.view(ctx.shape)


def swiglu(x: torch.Tensor) -> torch.Tensor:
    if not x.is_cuda:
        f = x.shape[-1] // 2
        return torch.nn.functional.silu(x[..., :f]) * x[..., f:]
    return SwiGLUFunction.apply(x)


def _rope_tables(s: int, d: int, theta: float, device, offset: int = 0):
    inv = 1.0 / (theta ** (torch.arange(0, d, 2, device=device, dtype=torch.float32) / d))
    t = torch.arange(offset, offset + s, device=device, dtype=torch.float32)
    ang = torch.outer(t, inv)
    return ang.cos(), ang.sin()


def _rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, inverse: bool) -> torch.Tensor:
    # x (b, s, h, d); rotate pairs (x[..., :d/2], x[..., d/2:]) -- the "half rotation" convention
    d = x.shape[-1]
    x1, x2 = x[..., : d // 2].float(), x[..., d // 2:].float()
    c, s_ = cos[None, :, None, :], sin[None, :, None, :]
    if inverse:
        s_ = -s_
    return torch.cat([x1 * c - x2 * s_, x1 * s_ + x2 * c], dim=-1).to(x.dtype)


class RopeFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, theta):
        cos, sin = _rope_tables(q.shape[1], q.shape[-1], theta, q.device)
        ctx.save_for_backward(cos, sin)
        return _rope_apply(q, cos, sin, False), _rope_apply(k, cos, sin, False)

    @staticmethod
    def backward(ctx, gq, gk):
        cos, sin = ctx.saved_tensors
        return _rope_apply(gq, cos, sin, True), _rope_apply(gk, cos, sin, True), None


def rope(q: torch.Tensor, k: torch.Tensor, theta: float = 10000.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rotary embedding of ``q`` (b, s, h, d) and ``k`` (b, s, hk, d) by absolute position."""
    return RopeFunction.apply(q, k, theta)
