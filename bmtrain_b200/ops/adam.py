"""Fused mixed-precision Adam steps.

GPU: one multi-tensor kernel launch updates a whole list of shards
(fp32 master, half parameter, first and second moment) -- replaces the
reference's one-launch-per-parameter kernels (``csrc/cuda/adam_cuda.cu:8-126``).
Host: AVX-512 / AVX2 Adam on a persistent thread pool
(reference: ``csrc/include/adam_cpu.hpp:15-557``).

Semantics (identical on every path):

* fp16 parameters keep ``exp_avg`` (fp16) and ``exp_avg_sq`` (fp32) in *loss-scaled* units,
  the gradient is never unscaled in memory:
  ``m' = b1 m' + (1-b1) g'``; ``v' = b2 v' + (1-b2) g'^2/s``;
  ``p -= lr * (m'/bc1) / (sqrt(v' s / bc2) + eps s) + lr wd p``.
* bf16 parameters and the host path unscale first (``g = g'/s``) and keep true-unit fp32 states.
* weight decay is decoupled (AdamW style) on all half-precision paths.
"""
from __future__ import annotations

import ctypes
import math
from typing import List, Optional, Sequence, Tuple

import torch

from . import _native

_MAX_TENSORS = 24  # tensors per launch (pointer table travels as a kernel argument)


class _AdamTable(ctypes.Structure):
    _fields_ = [
        ("p32", ctypes.c_void_p * _MAX_TENSORS),
        ("p16", ctypes.c_void_p * _MAX_TENSORS),
        ("g", ctypes.c_void_p * _MAX_TENSORS),
        ("m", ctypes.c_void_p * _MAX_TENSORS),
        ("v", ctypes.c_void_p * _MAX_TENSORS),
        ("n", ctypes.c_int64 * _MAX_TENSORS),
        ("count", ctypes.c_int32),
    ]


def _adam_half_torch(p32, p16, g, m, v, beta1, beta2, eps, lr, scale, wd, bc1, bc2):
    gf = g.float()
    if p16.dtype == torch.float16 and m.dtype == torch.float16:
        mf = beta1 * m.float() + (1 - beta1) * gf
        vf = beta2 * v + (1 - beta2) * gf * gf / scale
        upd = (mf / bc1) / (torch.sqrt(vf * scale / bc2) + eps * scale)
    else:
        gf = gf / scale
        mf = beta1 * m.float() + (1 - beta1) * gf
        vf = beta2 * v + (1 - beta2) * gf * gf
        upd = (mf / bc1) / (torch.sqrt(vf / bc2) + eps)
    p = p32 - lr * upd - lr * wd * p32
    p32.copy_(p)
    p16.copy_(p)
    m.copy_(mf)
    v.copy_(vf)


def adam_half_multi(entries: Sequence[Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]],
                    beta1: float, beta2: float, eps: float, lr: float, scale: float, weight_decay: float, step: int) -> None:
    """Update a list of ``(param_fp32, param_half, grad_half, exp_avg, exp_avg_sq)`` shards in place."""
    if not entries:
        return
    bc1 = 1.0 - math.pow(beta1, step)
    bc2 = 1.0 - math.pow(beta2, step)
    if not entries[0][0].is_cuda:
        for e in entries:
            _adam_half_torch(*e, beta1, beta2, eps, lr, scale, weight_decay, bc1, bc2)
        return
    lib = _native.cuda_lib()
    fp16 = entries[0][1].dtype == torch.float16
    if fp16 and entries[0][3].dtype == torch.float32:
        fn = lib.bmt_adam_fp16_f32state_multi  # offloaded-state layout: fp32 moments in true units
    else:
        fn = lib.bmt_adam_fp16_multi if fp16 else lib.bmt_adam_bf16_multi
    for i in range(0, len(entries), _MAX_TENSORS):
        chunk = entries[i:i + _MAX_TENSORS]
        table = _AdamTable()
        table.count = len(chunk)
        for j, (p32, p16, g, m, v) in enumerate(chunk):
            assert p16.dtype == entries[0][1].dtype and g.dtype == p16.dtype
            assert p32.is_contiguous() and p16.is_contiguous() and g.is_contiguous() and m.is_contiguous() and v.is_contiguous()
            table.p32[j], table.p16[j], table.g[j] = p32.data_ptr(), p16.data_ptr(), g.data_ptr()
            table.m[j], table.v[j], table.n[j] = m.data_ptr(), v.data_ptr(), p16.numel()
        _native.check(fn(ctypes.byref(table), ctypes.c_float(beta1), ctypes.c_float(beta2), ctypes.c_float(eps),
                         ctypes.c_float(lr), ctypes.c_float(scale), ctypes.c_float(weight_decay),
                         ctypes.c_float(bc1), ctypes.c_float(bc2), _native.stream_handle()), "adam multi-tensor kernel")


def adam_cpu(param_fp32: torch.Tensor, param_half: torch.Tensor, delta_info: Optional[torch.Tensor], grad_half: torch.Tensor,
             m_fp32: torch.Tensor, v_fp32: torch.Tensor, beta1: float, beta2: float, eps: float, lr: float,
             scale: float, weight_decay: float, step: int) -> None:
    """Host Adam: fp32 master/moments, half gradient in (loss-scaled), half parameter out.

    ``delta_info`` (4 floats: mean, variance, sum, sum of squares of the applied update) is filled when given.
    """
    for t in (param_fp32, param_half, grad_half, m_fp32, v_fp32):
        assert not t.is_cuda and t.is_contiguous()
    assert param_fp32.dtype == torch.float32 and m_fp32.dtype == torch.float32 and v_fp32.dtype == torch.float32
    assert param_half.dtype == grad_half.dtype and param_half.dtype in (torch.float16, torch.bfloat16)
    n = param_fp32.numel()
    assert param_half.numel() == n and grad_half.numel() == n and m_fp32.numel() == n and v_fp32.numel() == n
    bc1 = 1.0 - math.pow(beta1, step)
    bc2 = 1.0 - math.pow(beta2, step)
    lib = _native.cpu_lib()
    if lib is None:
        g = grad_half.float() / scale
        m_fp32.mul_(beta1).add_(g, alpha=1 - beta1)
        v_fp32.mul_(beta2).addcmul_(g, g, value=1 - beta2)
        upd = (m_fp32 / bc1) / (torch.sqrt(v_fp32 / bc2) + eps)
        new_p = param_fp32 - lr * upd - lr * weight_decay * param_fp32
        if delta_info is not None:
            d = new_p - param_fp32
            delta_info[0], delta_info[1] = d.mean(), d.var(unbiased=False)
            delta_info[2], delta_info[3] = d.sum(), (d * d).sum()
        param_fp32.copy_(new_p)
        param_half.copy_(new_p)
        return
    fn = lib.bmt_adam_cpu_fp16 if param_half.dtype == torch.float16 else lib.bmt_adam_cpu_bf16
    fn(ctypes.c_int64(n), _native.ptr(param_fp32), _native.ptr(param_half), _native.ptr(delta_info), _native.ptr(grad_half),
       _native.ptr(m_fp32), _native.ptr(v_fp32), ctypes.c_float(beta1), ctypes.c_float(beta2), ctypes.c_float(eps),
       ctypes.c_float(lr), ctypes.c_float(scale), ctypes.c_float(weight_decay), ctypes.c_float(bc1), ctypes.c_float(bc2))


def half_from_fp32(src: torch.Tensor, dst: torch.Tensor) -> None:
    """Host conversion fp32 -> fp16/bf16 (round to nearest even)."""
    assert not src.is_cuda and not dst.is_cuda and src.dtype == torch.float32 and src.numel() == dst.numel()
    lib = _native.cpu_lib()
    if lib is None or not (src.is_contiguous() and dst.is_contiguous()):
        dst.copy_(src)
        return
    fn = lib.bmt_fp16_from_fp32 if dst.dtype == torch.float16 else lib.bmt_bf16_from_fp32
    fn(ctypes.c_int64(src.numel()), _native.ptr(src), _native.ptr(dst))


fp16_from_fp32 = half_from_fp32
bf16_from_fp32 = half_from_fp32
