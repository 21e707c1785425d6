"""Small fused elementwise operators: SwiGLU and rotary position embedding.

The rotary embedding works on the packed projection ``(b, s, kv heads, g + 2, d)`` the Llama-shaped attention produces:
one kernel rotates the query and key heads and lays q, k, v out contiguously; its backward is one kernel as well
(``csrc/elementwise.cu``).  The eager PyTorch form below is the CPU definition and the numerical reference.
"""
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


_rope_cache = {}


def _rope_table(s: int, d: int, theta: float, device) -> torch.Tensor:
    """(s, d/2, 2) fp32 table of (cos, sin) of position x frequency, built once per shape and kept on the device."""
    key = (s, d, float(theta), str(device))
    tab = _rope_cache.get(key)
    if tab is None:
        cos, sin = _rope_tables(s, d, theta, device)
        tab = torch.stack([cos, sin], dim=-1).contiguous()
        if len(_rope_cache) > 16:
            _rope_cache.clear()
        _rope_cache[key] = tab
    return tab


class RopeQKVFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, packed, g, theta):
        b, s, hk, _, d = packed.shape
        q = torch.empty(b, s, hk * g, d, dtype=packed.dtype, device=packed.device)
        k = torch.empty(b, s, hk, d, dtype=packed.dtype, device=packed.device)
        v = torch.empty(b, s, hk, d, dtype=packed.dtype, device=packed.device)
        _native.check(_native.cuda_lib().bmt_rope_qkv(
            ctypes.c_int64(b), ctypes.c_int64(s), ctypes.c_int(hk), ctypes.c_int(g), ctypes.c_int(d), _native.ptr(packed),
            ctypes.c_int64(packed.stride(1)), ctypes.c_int64(packed.stride(0)), _native.ptr(q), _native.ptr(k), _native.ptr(v),
            _native.ptr(_rope_table(s, d, theta, packed.device)), ctypes.c_int64(0), ctypes.c_int(1), ctypes.c_int(_DT[packed.dtype]),
            _native.stream_handle()),
            "rotary embedding kernel")
        ctx.g, ctx.theta, ctx.shape = g, theta, packed.shape
        return q, k, v

    @staticmethod
    def backward(ctx, gq, gk, gv):
        b, s, hk, _, d = ctx.shape
        gq, gk, gv = gq.contiguous(), gk.contiguous(), gv.contiguous()
        out = torch.empty(ctx.shape, dtype=gq.dtype, device=gq.device)
        _native.check(_native.cuda_lib().bmt_rope_qkv(
            ctypes.c_int64(b), ctypes.c_int64(s), ctypes.c_int(hk), ctypes.c_int(ctx.g), ctypes.c_int(d), _native.ptr(out),
            ctypes.c_int64(out.stride(1)), ctypes.c_int64(out.stride(0)), _native.ptr(gq), _native.ptr(gk), _native.ptr(gv),
            _native.ptr(_rope_table(s, d, ctx.theta, gq.device)), ctypes.c_int64(0), ctypes.c_int(0), ctypes.c_int(_DT[gq.dtype]),
            _native.stream_handle()),
            "rotary embedding backward kernel")
        return out, None, None


def rope_qkv(packed: torch.Tensor, g: int, theta: float = 10000.0):
    """``packed`` (b, s, kv heads, g + 2, d) -> rotated ``q`` (b, s, kv heads * g, d), rotated ``k`` and ``v``
    (b, s, kv heads, d).  The token and batch dims of ``packed`` may be strided (a permuted view); the rest is contiguous."""
    b, s, hk, _, d = packed.shape
    ok = (packed.is_cuda and d % 16 == 0 and packed.dtype in (torch.float16, torch.bfloat16) and packed.stride(4) == 1
          and packed.stride(3) == d and packed.stride(2) == (g + 2) * d and packed.stride(0) % 8 == 0 and packed.stride(1) % 8 == 0)
    if not ok:
        q = packed[:, :, :, :g].reshape(b, s, hk * g, d)
        k, v = packed[:, :, :, g], packed[:, :, :, g + 1]
        q, k = rope(q, k, theta)
        return q, k, v
    return RopeQKVFunction.apply(packed, g, theta)
