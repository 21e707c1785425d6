"""inf/nan detection and gradient norms over lists of tensors.

``has_inf_nan`` mirrors the reference API (``bmtrain/loss/_function.py:7-24`` over
``csrc/cuda/has_inf_nan.cu``): it ORs "some element is inf or nan" into a
one-byte flag.  ``multi_has_inf_nan`` scans a whole list of gradients in one
launch per <=24 tensors, ``multi_sq_norm`` accumulates the sum of squares
(fp32) of a list of tensors for gradient clipping.
"""
from __future__ import annotations

import ctypes
from typing import Sequence

import torch

from . import _native

_MAX = 24


class _PtrTable(ctypes.Structure):
    _fields_ = [("p", ctypes.c_void_p * _MAX), ("n", ctypes.c_int64 * _MAX), ("count", ctypes.c_int32)]


_DT = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def multi_has_inf_nan(tensors: Sequence[torch.Tensor], out_flag: torch.Tensor) -> None:
    """``out_flag`` (uint8 scalar tensor) |= any(isinf | isnan) over all ``tensors``."""
    tensors = [t for t in tensors if t is not None and t.numel() > 0]
    if not tensors:
        return
    if not tensors[0].is_cuda:
        for t in tensors:
            if not torch.isfinite(t.float()).all():
                out_flag.fill_(1)
        return
    lib = _native.cuda_lib()
    by_dtype = {}
    for t in tensors:
        assert t.is_contiguous()
        by_dtype.setdefault(t.dtype, []).append(t)
    for dtype, group in by_dtype.items():
        for i in range(0, len(group), _MAX):
            chunk = group[i:i + _MAX]
            tab = _PtrTable()
            tab.count = len(chunk)
            for j, t in enumerate(chunk):
                tab.p[j], tab.n[j] = t.data_ptr(), t.numel()
            _native.check(lib.bmt_has_inf_nan_multi(ctypes.byref(tab), ctypes.c_int(_DT[dtype]), _native.ptr(out_flag),
                                                    _native.stream_handle()), "has_inf_nan kernel")


def has_inf_nan(g: torch.Tensor, out: torch.Tensor) -> None:
    """Reference-compatible single-tensor form: ``out`` (uint8) is set to 1 if ``g`` holds inf or nan."""
    assert out.dtype == torch.uint8
    multi_has_inf_nan([g.contiguous()], out)


def multi_sq_norm(tensors: Sequence[torch.Tensor], out: torch.Tensor) -> None:
    """``out`` (fp32 scalar tensor) += sum over all tensors of sum(x^2), accumulated in fp32."""
    tensors = [t for t in tensors if t is not None and t.numel() > 0]
    if not tensors:
        return
    if not tensors[0].is_cuda:
        for t in tensors:
            out += t.float().pow(2).sum()
        return
    lib = _native.cuda_lib()
    by_dtype = {}
    for t in tensors:
        assert t.is_contiguous()
        by_dtype.setdefault(t.dtype, []).append(t)
    for dtype, group in by_dtype.items():
        for i in range(0, len(group), _MAX):
            chunk = group[i:i + _MAX]
            tab = _PtrTable()
            tab.count = len(chunk)
            for j, t in enumerate(chunk):
                tab.p[j], tab.n[j] = t.data_ptr(), t.numel()
            _native.check(lib.bmt_sq_norm_multi(ctypes.byref(tab), ctypes.c_int(_DT[dtype]), _native.ptr(out),
                                                _native.stream_handle()), "grad-norm kernel")


def multi_scale(tensors: Sequence[torch.Tensor], coef: torch.Tensor) -> None:
    """In-place ``t *= min(coef, 1)`` for every tensor; ``coef`` is a device scalar (no host sync)."""
    tensors = [t for t in tensors if t is not None and t.numel() > 0]
    if not tensors:
        return
    if not tensors[0].is_cuda:
        c = torch.clamp(coef.float(), max=1.0)
        for t in tensors:
            t.mul_(c.to(t.dtype))
        return
    lib = _native.cuda_lib()
    by_dtype = {}
    for t in tensors:
        if t.dtype not in _DT or not t.is_contiguous():
            # the kernel walks flat memory of the three training dtypes; anything else is scaled by torch
            t.mul_(torch.clamp(coef.float(), max=1.0).to(t.dtype))
            continue
        by_dtype.setdefault(t.dtype, []).append(t)
    for dtype, group in by_dtype.items():
        for i in range(0, len(group), _MAX):
            chunk = group[i:i + _MAX]
            tab = _PtrTable()
            tab.count = len(chunk)
            for j, t in enumerate(chunk):
                tab.p[j], tab.n[j] = t.data_ptr(), t.numel()
            _native.check(lib.bmt_scale_multi(ctypes.byref(tab), ctypes.c_int(_DT[dtype]), _native.ptr(coef),
                                              _native.stream_handle()), "grad-scale kernel")
