"""Tensor-level communication calls with the reference's names.

The reference exposes NCCL on torch storages (``bmtrain/nccl/__init__.py:7-336``):
``allReduce(src, dst, op, comm)``, ``allGather``, ``reduceScatter``,
``broadcast``, ``reduce``, ``send``, ``recv``, ``groupStart/groupEnd`` and the
communicator helpers.  ``bmtrain_b200.nccl.native.NativeCommunicator`` is the
library's own C++ NCCL binding (non-blocking communicators with error polling
and abort); every function below takes one of those as well.  Here the same functions accept tensors (or anything
with ``.view(-1)``; a typed storage is wrapped) and run on a
:class:`~bmtrain_b200.comm.Communicator`, i.e. on NCCL over NVLink when the
ranks own GPUs and on gloo otherwise.
"""
from __future__ import annotations

import os
from typing import List

import torch
import torch.distributed as dist

from ..comm import Communicator
from ..global_var import config
from .enums import REDUCE_OPS

NCCLCommunicator = Communicator


def _t(x) -> torch.Tensor:
    if isinstance(x, torch.Tensor):
        return x
    if isinstance(x, (torch.TypedStorage,)):
        return torch.tensor([], dtype=x.dtype, device=x.device).set_(x)
    raise TypeError(f"expected a tensor or typed storage, got {type(x)}")


def dtype2nccl(dtype: torch.dtype) -> int:
    """NCCL's ``ncclDataType_t`` number of a torch dtype (reference: ``bmtrain/nccl/__init__.py:29-47``).  The numbers are
    the public ones of ``nccl.h``; nothing in this package needs them, the process groups take torch dtypes."""
    table = {torch.int8: 0, torch.uint8: 1, torch.int32: 2, torch.int64: 4, torch.float16: 6, torch.float32: 7,
             torch.float64: 8, torch.bfloat16: 9}
    if dtype not in table:
        raise TypeError(f"Unsupport dtype {dtype}")
    return table[dtype]


def op2nccl(op: str) -> int:
    """NCCL's ``ncclRedOp_t`` number of a reduction name (reference: ``bmtrain/nccl/__init__.py:49-59``)."""
    table = {"sum": 0, "prod": 1, "max": 2, "min": 3, "avg": 4}
    if op not in table:
        raise ValueError(f"Unsupport op {op}")
    return table[op]


def getUniqueId() -> bytes:
    """An opaque id for a new communicator (random token; the rendezvous is torch.distributed's)."""
    return os.urandom(16)


def commInitRank(unique_id: bytes, world_size: int, rank: int) -> Communicator:
    """Create a communicator over ``world_size`` consecutive-id members.

    Every process of the job must call this (it creates a process group), and
    members are identified by publishing ``(unique_id, rank)`` through an
    all-gather over the world.
    """
    world: Communicator = config["comm"]
    mine = [int.from_bytes(unique_id[:7], "little"), rank, world_size]
    gathered: List = [None] * world.size
    if world.size > 1:
        dist.all_gather_object(gathered, mine)
    else:
        gathered = [mine]
    groups = {}
    for g_rank, (uid, r, n) in enumerate(gathered):
        groups.setdefault(uid, {})[r] = g_rank
    result = None
    for uid in sorted(groups):
        members = [groups[uid][r] for r in sorted(groups[uid])]
        pg = dist.new_group(ranks=members) if len(members) > 1 else None
        if config["rank"] in members:
            result = Communicator(pg, members, config["rank"], name=f"user{uid & 0xffff}")
    return result


def commDestroy(comm: Communicator) -> None:
    if comm.group is not None and comm.group is not dist.group.WORLD:
        dist.destroy_process_group(comm.group)
        comm.group = None


def commCount(comm: Communicator) -> int:
    return comm.size


def commRank(comm: Communicator) -> int:
    return comm.rank


def allReduce(src, dst, op: str, comm: Communicator) -> None:
    assert op in REDUCE_OPS
    src, dst = _t(src), _t(dst)
    if dst.data_ptr() != src.data_ptr():
        dst.view(-1).copy_(src.view(-1))
    comm.all_reduce(dst, op)


def allGather(src, dst, comm: Communicator) -> None:
    comm.all_gather_into(_t(dst), _t(src))


def reduceScatter(src, dst, op: str, comm: Communicator) -> None:
    assert op in REDUCE_OPS
    comm.reduce_scatter_into(_t(dst), _t(src), op)


def broadcast(src, dst, root: int, comm: Communicator) -> None:
    src, dst = _t(src), _t(dst)
    if comm.rank == root and dst.data_ptr() != src.data_ptr():
        dst.view(-1).copy_(src.view(-1))
    comm.broadcast(dst, root)


def reduce(src, dst, op: str, root: int, comm: Communicator) -> None:
    src, dst = _t(src), _t(dst)
    if dst.data_ptr() != src.data_ptr():
        dst.view(-1).copy_(src.view(-1))
    comm.reduce(dst, op, root)


_pending: List = []
_group_depth = 0


def send(src, peer: int, comm: Communicator) -> None:
    work = comm.send(_t(src), peer)
    if _group_depth:
        _pending.append(work)
    else:
        work.wait()


def recv(dst, peer: int, comm: Communicator) -> None:
    work = comm.recv(_t(dst), peer)
    if _group_depth:
        _pending.append(work)
    else:
        work.wait()


def groupStart() -> None:
    """Open a group: point-to-point calls inside are posted together and completed by groupEnd."""
    global _group_depth
    _group_depth += 1


def groupEnd() -> None:
    global _group_depth
    _group_depth -= 1
    if _group_depth == 0:
        while _pending:
            _pending.pop(0).wait()
