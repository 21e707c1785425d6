"""Shared-memory transport for the CPU ranks of one host (``csrc/cpu_comm.cpp``).

gloo moves every collective through sockets and has no reduce-scatter; for the CPU runs of this package (plumbing
checks, host-side tests, the tiny CPU configuration) all ranks share one machine, so a mapped segment with a bounded
sense-reversing barrier does the same work with two memory copies per element.  Enabled with ``BMT_CPU_COMM=shm``;
the process group stays gloo for everything this transport does not cover (point-to-point messages, object broadcast,
exotic dtypes).  (The reference has no CPU path at all: ``bmtrain/parameter.py:46`` requires CUDA.)
"""
from __future__ import annotations

import ctypes
import os
import time
from typing import Optional

import torch
import torch.distributed as dist

from ..ops import _native

_DT = {torch.float32: 0, torch.float64: 1, torch.int32: 2, torch.int64: 3, torch.uint8: 4}
_OP = {"sum": 0, "max": 1, "min": 2, "prod": 3}
_SLOT_BYTES = 8 << 20


class ShmTransport:
    """Collectives of one communicator through a shared-memory segment.  Creation is collective."""

    def __init__(self, group, ranks, rank: int, timeout_s: float = 60.0):
        lib = _native.cpu_lib()
        if lib is None or not hasattr(lib, "bmt_shm_open"):
            raise RuntimeError("the CPU library was built without the shared-memory collectives")
        lib.bmt_shm_open.restype = ctypes.c_void_p
        name = [f"/bmt_{os.getpid()}_{time.time_ns() & 0xffffffffff:x}"] if rank == 0 else [None]
        dist.broadcast_object_list(name, src=ranks[0], group=group)
        self._lib = lib
        self.size, self.rank = len(ranks), rank
        self._h = lib.bmt_shm_open(name[0].encode(), ctypes.c_int(self.size), ctypes.c_int(rank), ctypes.c_uint64(_SLOT_BYTES),
                                   ctypes.c_double(timeout_s))
        ok = torch.tensor([1 if self._h else 0])
        dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
        if int(ok) == 0:
            self.close()
            raise RuntimeError("shared-memory segment could not be mapped on every rank")

    def close(self) -> None:
        if getattr(self, "_h", None):
            self._lib.bmt_shm_close(ctypes.c_void_p(self._h))
            self._h = None

    @staticmethod
    def supports(t: torch.Tensor, op: Optional[str] = None) -> bool:
        if t.is_cuda:
            return False
        if op is None:
            return True  # all-gather and broadcast move bytes
        return t.dtype in _DT and op in _OP

    def _check(self, rc: int, what: str) -> None:
        if rc == -2:
            raise RuntimeError(f"shared-memory {what}: a rank did not arrive within the time limit")
        if rc != 0:
            raise RuntimeError(f"shared-memory {what} failed with status {rc}")

    def all_reduce(self, t: torch.Tensor, op: str) -> None:
        assert t.is_contiguous()
        self._check(self._lib.bmt_shm_all_reduce(ctypes.c_void_p(self._h), ctypes.c_void_p(t.data_ptr()), ctypes.c_int64(t.numel()),
                                                 ctypes.c_int(_DT[t.dtype]), ctypes.c_int(_OP[op])), "all-reduce")

    def all_gather(self, out: torch.Tensor, inp: torch.Tensor) -> None:
        assert out.is_contiguous() and inp.is_contiguous() and out.dtype == inp.dtype
        self._check(self._lib.bmt_shm_all_gather(ctypes.c_void_p(self._h), ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(inp.data_ptr()),
                                                 ctypes.c_int64(inp.numel() * inp.element_size())), "all-gather")

    def reduce_scatter(self, out: torch.Tensor, inp: torch.Tensor, op: str) -> None:
        assert out.is_contiguous() and inp.is_contiguous() and out.dtype == inp.dtype
        self._check(self._lib.bmt_shm_reduce_scatter(ctypes.c_void_p(self._h), ctypes.c_void_p(out.data_ptr()), ctypes.c_void_p(inp.data_ptr()),
                                                     ctypes.c_int64(out.numel()), ctypes.c_int(_DT[inp.dtype]), ctypes.c_int(_OP[op])),
                    "reduce-scatter")

    def broadcast(self, t: torch.Tensor, root: int) -> None:
        assert t.is_contiguous()
        self._check(self._lib.bmt_shm_broadcast(ctypes.c_void_p(self._h), ctypes.c_void_p(t.data_ptr()),
                                                ctypes.c_int64(t.numel() * t.element_size()), ctypes.c_int(root)), "broadcast")

    def barrier(self) -> None:
        self._check(self._lib.bmt_shm_barrier(ctypes.c_void_p(self._h)), "barrier")
