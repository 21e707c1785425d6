"""Peer-memory (NVLink) runtime: symmetric buffers, flag rows and the fused gradient reduce-scatter.

One :class:`PeerRuntime` exists per communicator whose ranks sit in one NVLink / NVSwitch domain.  It owns

* symmetric buffers -- every rank allocates the same size, the CUDA IPC handles are exchanged through the
  communicator's process group and every rank maps all peers' buffers (``csrc/symm.cu``),
* a symmetric flag buffer: row ``s`` holds one 32-bit counter per rank; rank ``r`` publishes "reached epoch e on
  row s" by storing ``e`` into slot ``r`` of that row on every peer,
* a device status word that kernels set when a bounded wait runs out (:meth:`PeerRuntime.check`).

Creation is collective: every rank of the communicator has to construct buffers in the same order.
(The reference has nothing comparable; its collectives are NCCL calls on torch storages.)
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..comm import Communicator
from ..global_var import config
from ..ops import _native

_FLAG_ROWS = 256
_runtimes: Dict[int, Optional["PeerRuntime"]] = {}


class _CudaArray:
    """Adapter exposing raw device memory through ``__cuda_array_interface__``."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
        self._owner = owner


class SymmetricBuffer:
    """``nbytes`` of device memory on every rank of ``comm``; ``ptrs[j]`` is rank j's buffer as seen from this process."""

    def __init__(self, comm: Communicator, nbytes: int):
        lib = _native.cuda_lib()
        self.comm, self.nbytes = comm, int(nbytes)
        self.local_ptr = 0
        self.ptrs: List[int] = []
        self._opened: List[int] = []
        # Every step that can fail on one rank alone (allocation, export, import) is followed by an agreement before the
        # next collective, so that a failing rank never leaves the others blocked inside a collective it will not join.
        local = ctypes.c_void_p()
        handle = (ctypes.c_ubyte * lib.bmt_ipc_handle_size())()
        ok = lib.bmt_symm_alloc(ctypes.c_int64(self.nbytes), ctypes.byref(local)) == 0
        if ok:
            self.local_ptr = local.value
            ok = lib.bmt_ipc_get_handle(ctypes.c_void_p(self.local_ptr), handle) == 0
        if not self._all_ok(ok):
            self.close()
            raise RuntimeError(f"symmetric allocation of {self.nbytes} bytes failed on a rank of communicator {comm.name}")
        gathered: List = [None] * comm.size
        dist.all_gather_object(gathered, bytes(handle), group=comm.group)
        ok = True
        for j, raw in enumerate(gathered):
            if j == comm.rank:
                self.ptrs.append(self.local_ptr)
                continue
            buf = (ctypes.c_ubyte * len(raw)).from_buffer_copy(raw)
            out = ctypes.c_void_p()
            if lib.bmt_ipc_open_handle(buf, ctypes.byref(out)) != 0:
                ok = False
                break
            self.ptrs.append(out.value)
            self._opened.append(out.value)
        if not self._all_ok(ok):
            self.close()
            raise RuntimeError(f"mapping a peer's buffer failed on a rank of communicator {comm.name}")
        self._bytes = torch.as_tensor(_CudaArray(self.local_ptr, self.nbytes, self), device=config["device"])

    def _all_ok(self, ok: bool) -> bool:
        flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=config["device"])
        self.comm.all_reduce(flag, "min")
        return int(flag.item()) == 1

    def tensor(self, dtype: torch.dtype, numel: int, byte_offset: int = 0) -> torch.Tensor:
        """A tensor that aliases the local buffer."""
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        return self._bytes[byte_offset:byte_offset + nbytes].view(dtype)

    def ptr_table(self, byte_offset: int = 0):
        return (ctypes.c_void_p * self.comm.size)(*[p + byte_offset for p in self.ptrs])

    def close(self) -> None:
        lib = _native.cuda_lib()
        for p in self._opened:
            lib.bmt_ipc_close(ctypes.c_void_p(p))
        self._opened = []
        if self.local_ptr:
            self._bytes = None
            lib.bmt_symm_free(ctypes.c_void_p(self.local_ptr))
            self.local_ptr = 0


class MulticastBuffer:
    """Symmetric buffer backed by CUDA virtual-memory allocations that are also bound to an NVSwitch multicast object:
    ``ptrs[j]`` is rank j's copy as seen from this process, ``mc_ptr`` the multicast address (a ``multimem`` load from it
    returns the sum over all copies, a ``multimem`` store writes all of them).  Allocation, handle exchange and multicast
    binding are done by ``torch.distributed._symmetric_memory`` over the communicator's process group; the kernels that
    use the addresses are this library's.  Same interface as :class:`SymmetricBuffer`."""

    def __init__(self, comm: Communicator, nbytes: int):
        import torch.distributed._symmetric_memory as symm_mem

        self.comm, self.nbytes = comm, int(nbytes)
        self._bytes = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=config["device"])
        self._handle = symm_mem.rendezvous(self._bytes, comm.group)
        self.ptrs: List[int] = [int(p) for p in self._handle.buffer_ptrs]
        self.local_ptr = self.ptrs[comm.rank]
        self.mc_ptr = int(self._handle.multicast_ptr or 0)

    def tensor(self, dtype: torch.dtype, numel: int, byte_offset: int = 0) -> torch.Tensor:
        nbytes = numel * torch.empty((), dtype=dtype).element_size()
        return self._bytes[byte_offset:byte_offset + nbytes].view(dtype)

    def ptr_table(self, byte_offset: int = 0):
        return (ctypes.c_void_p * self.comm.size)(*[p + byte_offset for p in self.ptrs])

    def close(self) -> None:
        self._handle = None
        self._bytes = None
        self.local_ptr = 0


def nvls_wanted() -> bool:
    """``BMT_NVLS=1``: gradient staging buffers are multicast-bound and the fused reduce-scatter sums inside the switch."""
    return os.environ.get("BMT_NVLS", "0") == "1"


class StreamWork:
    """Handle whose ``wait()`` makes the current stream wait for an event (same contract as a c10d work object)."""

    def __init__(self, event: torch.cuda.Event):
        self.event = event

    def wait(self) -> None:
        torch.cuda.current_stream().wait_event(self.event)


class PeerRuntime:
    """Flags, status word and gradient staging slots of one communicator."""

    def __init__(self, comm: Communicator):
        self.comm = comm
        dev = config["device"]
        self.flags = SymmetricBuffer(comm, _FLAG_ROWS * comm.size * 4)
        self.flag_ptrs = self.flags.ptr_table()
        self.flag_table_dev = torch.tensor(list(self.flags.ptrs), dtype=torch.int64, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.overflow = torch.zeros(1, dtype=torch.uint8, device=dev)
        self.epochs: Dict[int, int] = {}
        self.rows: Dict[Tuple, int] = {}
        self.slots: Dict[Tuple, SymmetricBuffer] = {}
        self._counters: Dict[Tuple, torch.Tensor] = {}
        self.cache: Dict[Tuple, object] = {}
        self._multicast_ok = nvls_wanted()
        self.timeout_s = float(os.environ.get("BMT_PEER_TIMEOUT", "10"))
        self.stream = torch.cuda.Stream(priority=-1)

    # ----------------------------------------------------------------- bookkeeping
    def row(self, key: Tuple) -> int:
        if key not in self.rows:
            if len(self.rows) >= _FLAG_ROWS:
                raise RuntimeError("out of flag rows")
            self.rows[key] = len(self.rows)
        return self.rows[key]

    def next_epoch(self, row: int) -> int:
        self.epochs[row] = self.epochs.get(row, 0) + 1
        return self.epochs[row]

    def slot(self, key: Tuple, nbytes: int, multicast: bool = False) -> SymmetricBuffer:
        """Symmetric staging buffer for ``key`` (allocated collectively on first use, regrown when too small).
        ``multicast``: bind it to an NVSwitch multicast object when the platform offers one (see MulticastBuffer)."""
        buf = self.slots.get(key)
        if buf is None or buf.nbytes < nbytes:
            if buf is not None:
                torch.cuda.synchronize()
                self.comm.barrier()
                buf.close()
            buf = None
            if multicast and self._multicast_ok:
                try:
                    buf = MulticastBuffer(self.comm, nbytes)
                    good = 1 if buf.mc_ptr else 0
                    why = "the platform reports no multicast support"
                except Exception as exc:
                    good, why = 0, f"{type(exc).__name__}: {exc}"
                if not good and self.comm.rank == 0:
                    import sys

                    print(f"bmtrain_b200: multicast-bound buffers are not used on {self.comm.name} ({why})", file=sys.stderr)
                flag = torch.tensor([good], dtype=torch.int32, device=config["device"])
                self.comm.all_reduce(flag, "min")
                if int(flag.item()) == 0:   # some rank cannot: everybody uses plain peer memory for this and later slots
                    self._multicast_ok = False
                    buf = None
            if buf is None:
                buf = SymmetricBuffer(self.comm, nbytes)
            self.slots[key] = buf
        return buf

    def check(self) -> None:
        """Raise if a kernel's bounded wait on a peer ran out (reads the device status word: host sync)."""
        code = int(self.status.item())
        if code != 0:
            self.status.zero_()
            raise RuntimeError(f"peer wait timed out on communicator {self.comm.name} (code {code:#x}): "
                               "a rank did not reach the matching step within the time limit")

    # -------------------------------------------------------------------- kernels
    def signal_wait(self, row: int, epoch: int, signal: bool, wait: bool) -> None:
        lib = _native.cuda_lib()
        _native.check(lib.bmt_symm_signal_wait(
            ctypes.c_void_p(self.flag_table_dev.data_ptr()), ctypes.c_int(self.comm.size), ctypes.c_int(self.comm.rank),
            ctypes.c_int(row), ctypes.c_uint(epoch), ctypes.c_int(int(signal)), ctypes.c_int(int(wait)),
            _native.ptr(self.status), ctypes.c_double(self.timeout_s), _native.stream_handle()), "peer signal/wait kernel")

    def push_ranges(self, dst: SymmetricBuffer, ranges, free_row: int, done_row: int, epoch: int, key: Tuple) -> None:
        """Push-style all-gather on the current stream: ``ranges`` = [(src_ptr, dst_byte_offset, nbytes), ...] (at most 16)
        are written to the same offsets of ``dst`` on every rank once that rank published "free" for ``epoch``; when this
        rank's data is delivered everywhere it publishes ``epoch`` on ``done_row``."""
        lib = _native.cuda_lib()
        n = len(ranges)
        assert n <= 16
        grid = 96
        ckey = key + ("push_counter", n)
        if ckey not in self._counters:
            self._counters[ckey] = torch.zeros(1, dtype=torch.int32, device=config["device"])
        src = (ctypes.c_void_p * max(n, 1))(*[r[0] for r in ranges])
        off = (ctypes.c_int64 * max(n, 1))(*[r[1] for r in ranges])
        nb = (ctypes.c_int64 * max(n, 1))(*[r[2] for r in ranges])
        _native.check(lib.bmt_push_ranges(
            src, off, nb, ctypes.c_int(n), dst.ptr_table(), self.flag_ptrs, ctypes.c_int(self.comm.size), ctypes.c_int(self.comm.rank),
            ctypes.c_int(free_row), ctypes.c_int(done_row), ctypes.c_uint(epoch), _native.ptr(self._counters[ckey]),
            _native.ptr(self.status), ctypes.c_double(self.timeout_s), ctypes.c_int(grid), _native.stream_handle()),
            "push all-gather kernel")

    def reduce_scatter(self, full: SymmetricBuffer, row: int, part: int, out: torch.Tensor, accumulate: bool,
                       scale: float = 1.0, acc32: Optional[torch.Tensor] = None, sqsum: Optional[torch.Tensor] = None) -> None:
        """``out`` (+)= scale * sum over ranks of their ``full`` buffer, restricted to this rank's partition.

        Runs on the current stream; the kernel itself tells the peers that this rank's buffer is complete and
        waits (bounded) for theirs, adds in fp32 in rank order, and ORs inf/nan into ``self.overflow``.
        ``acc32``: fp32 copy of the partition gradient; accumulation then goes through it and ``out`` is its rounding.
        ``sqsum``: one fp32 element that receives += the sum of squares of the values written.
        """
        lib = _native.cuda_lib()
        epoch = self.next_epoch(row)
        dt = {torch.float16: 0, torch.bfloat16: 1}[out.dtype]
        if no_spin():
            # other kernels that wait for other ranks run next to this one (tensor-parallel kernels of the same step): the
            # cross-rank hand-shake is done by one CTA, the reduction kernel itself then never waits
            self.signal_wait(row, epoch, signal=True, wait=True)
            epoch = 0
        mc = getattr(full, "mc_ptr", 0)
        if acc32 is not None or sqsum is not None:
            _native.check(lib.bmt_fused_reduce_scatter_ex(
                full.ptr_table(), ctypes.c_void_p(mc) if mc else None, self.flag_ptrs, ctypes.c_int(self.comm.size),
                ctypes.c_int(self.comm.rank), ctypes.c_int(row), ctypes.c_uint(epoch), ctypes.c_int64(part), _native.ptr(out),
                ctypes.c_int(int(accumulate)), ctypes.c_float(scale), ctypes.c_int(dt),
                _native.ptr(acc32) if acc32 is not None else None, _native.ptr(sqsum) if sqsum is not None else None,
                _native.ptr(self.overflow), _native.ptr(self.status), ctypes.c_double(self.timeout_s), _native.stream_handle()),
                "fused reduce-scatter kernel with fp32 accumulator / sum of squares")
            return
        if mc:
            _native.check(lib.bmt_fused_reduce_scatter_mc(
                ctypes.c_void_p(mc), self.flag_ptrs, ctypes.c_int(self.comm.size), ctypes.c_int(self.comm.rank), ctypes.c_int(row),
                ctypes.c_uint(epoch), ctypes.c_int64(part), _native.ptr(out), ctypes.c_int(int(accumulate)), ctypes.c_float(scale),
                ctypes.c_int(dt), _native.ptr(self.overflow), _native.ptr(self.status), ctypes.c_double(self.timeout_s),
                _native.stream_handle()), "fused reduce-scatter kernel (multimem)")
            return
        _native.check(lib.bmt_fused_reduce_scatter(
            full.ptr_table(), self.flag_ptrs, ctypes.c_int(self.comm.size), ctypes.c_int(self.comm.rank), ctypes.c_int(row),
            ctypes.c_uint(epoch), ctypes.c_int64(part), _native.ptr(out), ctypes.c_int(int(accumulate)), ctypes.c_float(scale),
            ctypes.c_int(dt), _native.ptr(self.overflow), _native.ptr(self.status), ctypes.c_double(self.timeout_s),
            _native.stream_handle()), "fused reduce-scatter kernel")


def no_spin() -> bool:
    """Whether kernels of more than one parallel dimension wait for other ranks during a step (tensor parallel x ZeRO).
    Then no large grid may hold its SMs while it waits: a kernel of one dimension could keep the kernel another rank is
    waiting for from being scheduled.  Waits are given to one-CTA kernels and the fused GEMM -> reduce-scatter runs as
    separate deliver / wait / sum launches.  ``BMT_NO_SPIN=0/1`` overrides."""
    env = os.environ.get("BMT_NO_SPIN")
    if env is not None:
        return env == "1"
    return config.get("tp_size", 1) > 1 and config.get("tp_zero_size", 1) > 1


def _same_node(comm: Communicator) -> bool:
    return config["local_size"] == config["world_size"]


def peer_runtime(comm: Communicator) -> Optional[PeerRuntime]:
    """The runtime of ``comm``, created on first use (collective); None when peer memory cannot be used."""
    from ..comm import _LOCAL_ONLY

    if _LOCAL_ONLY[0]:
        return None   # timing without inter-rank traffic: the peer-memory kernels are part of that traffic
    key = id(comm)
    if key in _runtimes:
        return _runtimes[key]
    ok = (config["device"] is not None and config["device"].type == "cuda" and 2 <= comm.size <= 8 and _same_node(comm)
          and os.environ.get("BMT_PEER", "1") != "0")
    rt = None
    if ok:
        try:
            rt = PeerRuntime(comm)
        except RuntimeError:  # IPC / peer mapping not available; the buffer constructor made every rank raise together
            rt = None
    _runtimes[key] = rt
    return rt


def peer_runtime_ready(comm: Communicator) -> bool:
    return peer_runtime(comm) is not None


def reset() -> None:
    """Forget every runtime (process-group teardown)."""
    for rt in _runtimes.values():
        if rt is not None:
            for buf in rt.slots.values():
                buf.close()
            rt.flags.close()
    _runtimes.clear()
    try:
        from ..optim import optim_manager

        optim_manager._status_host.clear()
    except Exception:
        pass
