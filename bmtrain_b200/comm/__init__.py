"""Communicator: one object per parallel group.

The reference drives NCCL through its own pybind wrappers
(``csrc/include/nccl.hpp:8-188``, ``bmtrain/nccl/__init__.py``).  Here a
communicator wraps a ``torch.distributed`` process group -- ``nccl`` when the
ranks own B200s (NVLink 5 / NVSwitch underneath), ``gloo`` when the job runs on
CPUs (unit tests, plumbing checks) -- and adds the pieces NCCL-only code never
needed: size-1 short circuits, reductions gloo lacks (reduce-scatter, avg,
half-precision sums) and asynchronous handles the ZeRO scheduler uses for
prefetch/overlap.

All tensor arguments are ordinary ``torch.Tensor`` objects; collectives that
run asynchronously return a handle with ``wait()``.
"""
from __future__ import annotations

from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

_REDUCE_OPS = {
    "sum": dist.ReduceOp.SUM,
    "prod": dist.ReduceOp.PRODUCT,
    "max": dist.ReduceOp.MAX,
    "min": dist.ReduceOp.MIN,
}


class _Done:
    """Handle of an operation that already completed."""

    def wait(self) -> None:  # noqa: D401
        return None

    def is_completed(self) -> bool:
        return True


class _Chain:
    """Handle that runs a continuation after the wrapped work finished."""

    def __init__(self, work, then=None):
        self._work = work
        self._then = then

    def wait(self) -> None:
        if self._work is not None:
            self._work.wait()
            self._work = None
        if self._then is not None:
            fn, self._then = self._then, None
            fn()


DONE = _Done()

# Measurement aid: while set, all-gather and reduce-scatter only move this rank's own piece (no traffic between ranks).
# A training step timed this way against the same step with real collectives gives the communication time that
# computation does not hide.  Values are wrong in this mode; it is for timing only (see `local_collectives`).
_LOCAL_ONLY = [False]


class local_collectives:
    """``with local_collectives(): ...`` -- run a region with rank-local stand-ins for all-gather / reduce-scatter."""

    def __enter__(self):
        self._old, _LOCAL_ONLY[0] = _LOCAL_ONLY[0], True

    def __exit__(self, *exc):
        _LOCAL_ONLY[0] = self._old


class Communicator:
    """A group of ranks that communicate with each other.

    ``ranks`` lists the global ranks of the members in group order; the index
    of this process in that list is its group rank.
    """

    def __init__(self, group: Optional[dist.ProcessGroup], ranks: Sequence[int], my_global_rank: int, name: str = "world"):
        self.group = group
        self.ranks: List[int] = list(ranks)
        self.name = name
        self.size = len(self.ranks)
        self.rank = self.ranks.index(my_global_rank)
        self._gloo = group is not None and dist.get_backend(group) == "gloo"
        self._shm = None          # shared-memory transport of CPU ranks (created on first use when BMT_CPU_COMM=shm)
        self._shm_tried = False

    # ------------------------------------------------------------------ helpers
    def global_rank(self, group_rank: int) -> int:
        return self.ranks[group_rank]

    def __repr__(self) -> str:  # pragma: no cover
        return f"Communicator({self.name}, rank {self.rank}/{self.size})"

    def _needs_upcast(self, t: torch.Tensor) -> bool:
        return self._gloo and t.dtype in (torch.float16, torch.bfloat16)

    def _shm_for(self, t: torch.Tensor, op=None):
        """The shared-memory transport when it is enabled and can carry ``t`` (see ``comm/shm.py``), else None.  The first
        call creates it collectively, so every rank of the group has to reach its first CPU collective together (which
        collectives are anyway)."""
        if not self._gloo or t.is_cuda:
            return None
        if not self._shm_tried:
            import os

            self._shm_tried = True
            from ..global_var import config

            if os.environ.get("BMT_CPU_COMM", "gloo") == "shm" and config.get("local_size") == config.get("world_size"):
                from .shm import ShmTransport

                self._shm = ShmTransport(self.group, self.ranks, self.rank)
        if self._shm is None:
            return None
        from .shm import ShmTransport

        return self._shm if ShmTransport.supports(t, op) else None

    # -------------------------------------------------------------- collectives
    def all_gather_into(self, out: torch.Tensor, inp: torch.Tensor, async_op: bool = False):
        """``out`` (size * inp.numel()) <- concatenation of every rank's ``inp``."""
        assert out.numel() == inp.numel() * self.size, "all_gather: output size mismatch"
        if self.size == 1:
            out.view(-1).copy_(inp.reshape(-1))
            return DONE
        if _LOCAL_ONLY[0]:
            out.view(self.size, -1)[self.rank].copy_(inp.reshape(-1))
            return DONE
        inp = inp.contiguous()
        shm = self._shm_for(inp)
        if shm is not None and out.is_contiguous() and out.dtype == inp.dtype:
            shm.all_gather(out, inp)
            return DONE
        work = dist.all_gather_into_tensor(out.view(-1), inp.view(-1), group=self.group, async_op=async_op)
        return work if async_op else DONE

    def reduce_scatter_into(self, out: torch.Tensor, inp: torch.Tensor, op: str = "sum", async_op: bool = False):
        """``out`` <- this rank's 1/size slice of the element-wise reduction of ``inp``."""
        assert inp.numel() == out.numel() * self.size, "reduce_scatter: input size mismatch"
        avg = op == "avg"
        if self.size == 1:
            out.view(-1).copy_(inp.reshape(-1))
            return DONE
        if _LOCAL_ONLY[0]:
            out.view(-1).copy_(inp.reshape(self.size, -1)[self.rank])
            return DONE
        if self._gloo:
            # gloo has no reduce-scatter: all-reduce a (fp32 for half types) copy, keep own slice
            tmp = inp.reshape(-1).to(torch.float32 if self._needs_upcast(inp) else inp.dtype, copy=True)
            n = out.numel()
            shm = self._shm_for(tmp, "sum" if avg else op)
            if shm is not None:
                piece = torch.empty(n, dtype=tmp.dtype)
                shm.reduce_scatter(piece, tmp, "sum" if avg else op)
            else:
                dist.all_reduce(tmp, op=_REDUCE_OPS["sum" if avg else op], group=self.group)
                piece = tmp[self.rank * n:(self.rank + 1) * n]
            if avg:
                piece = piece / self.size
            out.view(-1).copy_(piece)
            return DONE
        rop = dist.ReduceOp.AVG if avg else _REDUCE_OPS[op]
        work = dist.reduce_scatter_tensor(out.view(-1), inp.contiguous().view(-1), op=rop, group=self.group, async_op=async_op)
        return work if async_op else DONE

    def all_reduce(self, t: torch.Tensor, op: str = "sum", async_op: bool = False):
        """In-place all-reduce of ``t``."""
        if self.size == 1:
            return DONE
        avg = op == "avg"
        if self._gloo:
            if self._needs_upcast(t) or not t.is_contiguous():
                tmp = t.to(torch.float32).contiguous()
                shm = self._shm_for(tmp, "sum" if avg else op)
                if shm is not None:
                    shm.all_reduce(tmp, "sum" if avg else op)
                else:
                    dist.all_reduce(tmp, op=_REDUCE_OPS["sum" if avg else op], group=self.group)
                if avg:
                    tmp /= self.size
                t.copy_(tmp)
            else:
                shm = self._shm_for(t, "sum" if avg else op)
                if shm is not None:
                    shm.all_reduce(t, "sum" if avg else op)
                else:
                    dist.all_reduce(t, op=_REDUCE_OPS["sum" if avg else op], group=self.group)
                if avg:
                    if t.is_floating_point():
                        t /= self.size
                    else:
                        t.copy_(t // self.size)
            return DONE
        rop = dist.ReduceOp.AVG if avg else _REDUCE_OPS[op]
        work = dist.all_reduce(t, op=rop, group=self.group, async_op=async_op)
        return work if async_op else DONE

    def broadcast(self, t: torch.Tensor, root: int = 0, async_op: bool = False):
        """Broadcast ``t`` from group rank ``root``."""
        if self.size == 1:
            return DONE
        if not t.is_contiguous():
            tmp = t.contiguous()
            dist.broadcast(tmp, src=self.ranks[root], group=self.group)
            t.copy_(tmp)
            return DONE
        shm = self._shm_for(t)
        if shm is not None:
            shm.broadcast(t, root)
            return DONE
        work = dist.broadcast(t, src=self.ranks[root], group=self.group, async_op=async_op)
        return work if async_op else DONE

    def reduce(self, t: torch.Tensor, op: str = "sum", root: int = 0):
        if self.size == 1:
            return DONE
        dist.reduce(t, dst=self.ranks[root], op=_REDUCE_OPS[op], group=self.group)
        return DONE

    def send(self, t: torch.Tensor, peer: int):
        """Asynchronous send to group rank ``peer``; returns a handle."""
        return dist.isend(t.contiguous(), dst=self.ranks[peer], group=self.group)

    def recv(self, t: torch.Tensor, peer: int):
        """Asynchronous receive from group rank ``peer``; returns a handle."""
        return dist.irecv(t, src=self.ranks[peer], group=self.group)

    def barrier(self) -> None:
        if self.size == 1:
            return
        flag = torch.zeros(1, device=_device_of(self))
        dist.all_reduce(flag, group=self.group)
        if flag.is_cuda:
            torch.cuda.current_stream().synchronize()


def _device_of(comm: Communicator) -> torch.device:
    from ..global_var import config

    return config["device"] if config.get("device") is not None else torch.device("cpu")
