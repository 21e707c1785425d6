"""Loader of the in-tree native libraries.

Two shared objects are built next to this package (see ``bmtrain_b200/build.py``):

* ``_C.so``   -- the sm_100a CUDA kernels behind a plain C ABI (raw pointers + stream handle),
* ``_cpu.so`` -- host code: AVX-512/AVX2 Adam with a persistent thread pool, fp32 -> half converters.

On a machine with a GPU a missing ``_C.so`` is an error (no silent eager fallback); on CPU-only
machines the CUDA library is simply not loaded and ops use their plain-PyTorch definitions.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

_HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_cuda_lib: Optional[ctypes.CDLL] = None
_cpu_lib: Optional[ctypes.CDLL] = None
_cuda_err: Optional[str] = None
_cpu_tried = False
_cuda_tried = False


def cuda_lib() -> ctypes.CDLL:
    """The CUDA kernel library; raises if it has not been built."""
    global _cuda_lib, _cuda_tried, _cuda_err
    if not _cuda_tried:
        _cuda_tried = True
        path = os.path.join(_HERE, "_C.so")
        try:
            _cuda_lib = ctypes.CDLL(path)
        except OSError as exc:
            _cuda_err = str(exc)
    if _cuda_lib is None:
        raise RuntimeError(
            "bmtrain_b200/_C.so is missing or cannot be loaded (" + str(_cuda_err) + "); "
            "build it with `python -m bmtrain_b200.build` -- CUDA tensors have no PyTorch fallback path"
        )
    return _cuda_lib


def cpu_lib() -> Optional[ctypes.CDLL]:
    """The host library, or None when it has not been built (ops then use PyTorch on the CPU)."""
    global _cpu_lib, _cpu_tried
    if not _cpu_tried:
        _cpu_tried = True
        try:
            _cpu_lib = ctypes.CDLL(os.path.join(_HERE, "_cpu.so"))
        except OSError:
            _cpu_lib = None
    return _cpu_lib


def ptr(t: Optional[torch.Tensor]) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def stream_handle() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def check(status: int, what: str) -> None:
    if status != 0:
        raise RuntimeError(f"{what} failed with status {status}")
