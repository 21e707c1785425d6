"""Communicators on the library's own C++ NCCL wrapper (``csrc/nccl_comm.cpp`` -> ``_nccl.so``).

A :class:`NativeCommunicator` is a non-blocking NCCL communicator: creation and every call return at once, failures
are found by polling ``ncclCommGetAsyncError`` (optionally by a watchdog thread that aborts the communicator), and
``abort()`` releases kernels that wait for a peer that is gone.  Collectives run on the current CUDA stream with raw
device pointers, as the reference's binding does (``bmtrain/nccl/__init__.py:66-336``), whose communicators are
blocking and can neither be polled nor aborted.

The unique id travels through ``torch.distributed`` (an object broadcast over an existing group), which is only used
for this rendezvous.  The class offers the same methods as :class:`bmtrain_b200.comm.Communicator`, so the functions of
``bmtrain_b200.nccl`` and the micro-benchmarks take either.
"""
from __future__ import annotations

import ctypes
import os
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

from ..comm import DONE

_HERE = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_lib: Optional[ctypes.CDLL] = None
_tried = False

_DTYPE = {torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4, torch.float16: 6, torch.float32: 7,
          torch.float64: 8, torch.bfloat16: 9}
_OP = {"sum": 0, "prod": 1, "max": 2, "min": 3, "avg": 4}
IN_PROGRESS = 7   # ncclInProgress


def lib() -> Optional[ctypes.CDLL]:
    """The wrapper library, or None when it has not been built (no NCCL on the build machine)."""
    global _lib, _tried
    if not _tried:
        _tried = True
        try:
            _lib = ctypes.CDLL(os.path.join(_HERE, "_nccl.so"))
            _lib.bmt_nccl_error_string.restype = ctypes.c_char_p
            _lib.bmt_nccl_comm_init.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_double,
                                                ctypes.POINTER(ctypes.c_void_p)]
            _lib.bmt_nccl_wait_issued.argtypes = [ctypes.c_void_p, ctypes.c_double]
            for name in ("comm_count", "comm_rank", "async_error", "abort", "comm_destroy"):
                getattr(_lib, "bmt_nccl_" + name).argtypes = [ctypes.c_void_p]
            _lib.bmt_nccl_watchdog_start.argtypes = [ctypes.c_void_p, ctypes.c_int]
        except OSError:
            _lib = None
    return _lib


class NCCLError(RuntimeError):
    pass


def _check(code: int, what: str) -> None:
    if code != 0:
        text = lib().bmt_nccl_error_string(ctypes.c_int(code)).decode()
        raise NCCLError(f"{what}: {text} (code {code})")


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


class NativeCommunicator:
    """Non-blocking NCCL communicator over ``ranks`` (global ranks in group order) of an existing torch group."""

    def __init__(self, ranks: Sequence[int], my_global_rank: int, bootstrap_group=None, name: str = "native",
                 timeout_s: float = 120.0, watchdog_ms: int = 0):
        L = lib()
        if L is None:
            raise NCCLError("bmtrain_b200/_nccl.so has not been built")
        self.ranks: List[int] = list(ranks)
        self.name = name
        self.size = len(self.ranks)
        self.rank = self.ranks.index(my_global_rank)
        self.timeout_s = timeout_s
        self.group = None
        n = L.bmt_nccl_unique_id_size()
        uid = (ctypes.c_ubyte * n)()
        if self.rank == 0:
            _check(L.bmt_nccl_get_unique_id(uid), "ncclGetUniqueId")
        if self.size > 1:
            box = [bytes(uid)]
            dist.broadcast_object_list(box, src=self.ranks[0], group=bootstrap_group)
            uid = (ctypes.c_ubyte * n).from_buffer_copy(box[0])
        handle = ctypes.c_void_p()
        _check(L.bmt_nccl_comm_init(uid, self.size, self.rank, ctypes.c_double(timeout_s), ctypes.byref(handle)),
               f"creating communicator {name}")
        self._h = handle
        if watchdog_ms > 0:
            L.bmt_nccl_watchdog_start(self._h, watchdog_ms)

    # ---------------------------------------------------------------- state
    def async_error(self) -> int:
        """0 = healthy, ``IN_PROGRESS`` = calls still being issued, anything else = failed (negative: aborted / timed out)."""
        return int(lib().bmt_nccl_async_error(self._h))

    def check(self) -> None:
        code = self.async_error()
        if code not in (0, IN_PROGRESS):
            _check(code, f"communicator {self.name}")

    def abort(self) -> None:
        lib().bmt_nccl_abort(self._h)

    def destroy(self) -> None:
        if self._h is not None:
            lib().bmt_nccl_comm_destroy(self._h)
            self._h = None

    def _issued(self, code: int, what: str) -> None:
        _check(code, what)
        # a non-blocking communicator may still be enqueueing the call: wait (bounded) until it is on the stream
        _check(lib().bmt_nccl_wait_issued(self._h, ctypes.c_double(self.timeout_s)), what)

    def global_rank(self, group_rank: int) -> int:
        return self.ranks[group_rank]

    # ---------------------------------------------------------- collectives
    def all_reduce(self, t: torch.Tensor, op: str = "sum", async_op: bool = False):
        assert t.is_contiguous()
        self._issued(lib().bmt_nccl_all_reduce(self._h, _ptr(t), _ptr(t), ctypes.c_int64(t.numel()), _DTYPE[t.dtype], _OP[op],
                                               _stream()), "all_reduce")
        return DONE

    def all_gather_into(self, out: torch.Tensor, inp: torch.Tensor, async_op: bool = False):
        assert out.numel() == inp.numel() * self.size and out.is_contiguous()
        inp = inp.contiguous()
        self._issued(lib().bmt_nccl_all_gather(self._h, _ptr(inp), _ptr(out), ctypes.c_int64(inp.numel()), _DTYPE[inp.dtype],
                                               _stream()), "all_gather")
        return DONE

    def reduce_scatter_into(self, out: torch.Tensor, inp: torch.Tensor, op: str = "sum", async_op: bool = False):
        assert inp.numel() == out.numel() * self.size and out.is_contiguous()
        inp = inp.contiguous()
        self._issued(lib().bmt_nccl_reduce_scatter(self._h, _ptr(inp), _ptr(out), ctypes.c_int64(out.numel()), _DTYPE[inp.dtype],
                                                   _OP[op], _stream()), "reduce_scatter")
        return DONE

    def broadcast(self, t: torch.Tensor, root: int = 0, async_op: bool = False):
        assert t.is_contiguous()
        self._issued(lib().bmt_nccl_broadcast(self._h, _ptr(t), _ptr(t), ctypes.c_int64(t.numel()), _DTYPE[t.dtype], root, _stream()),
                     "broadcast")
        return DONE

    def reduce(self, t: torch.Tensor, op: str = "sum", root: int = 0):
        assert t.is_contiguous()
        self._issued(lib().bmt_nccl_reduce(self._h, _ptr(t), _ptr(t), ctypes.c_int64(t.numel()), _DTYPE[t.dtype], _OP[op], root,
                                           _stream()), "reduce")
        return DONE

    def send(self, t: torch.Tensor, peer: int):
        t = t.contiguous()
        self._issued(lib().bmt_nccl_send(self._h, _ptr(t), ctypes.c_int64(t.numel()), _DTYPE[t.dtype], peer, _stream()), "send")
        return DONE

    def recv(self, t: torch.Tensor, peer: int):
        assert t.is_contiguous()
        self._issued(lib().bmt_nccl_recv(self._h, _ptr(t), ctypes.c_int64(t.numel()), _DTYPE[t.dtype], peer, _stream()), "recv")
        return DONE

    def barrier(self) -> None:
        flag = torch.zeros(1, device="cuda")
        self.all_reduce(flag)
        torch.cuda.current_stream().synchronize()

    def __repr__(self) -> str:  # pragma: no cover
        return f"NativeCommunicator({self.name}, rank {self.rank}/{self.size})"


def from_communicator(comm, watchdog_ms: int = 0) -> NativeCommunicator:
    """A native communicator over the same ranks as a :class:`bmtrain_b200.comm.Communicator` (collective call)."""
    from ..global_var import config

    return NativeCommunicator(comm.ranks, config["rank"], bootstrap_group=comm.group, name=comm.name + "/native",
                              watchdog_ms=watchdog_ms)
