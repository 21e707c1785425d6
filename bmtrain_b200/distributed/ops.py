"""Autograd-aware collectives on tensors.

Same call signatures and gradient rules as the reference
(``bmtrain/distributed/ops.py:21-220``):

* ``all_gather(x)`` stacks the ranks on a new leading dim; backward keeps the own slice.
* ``reduce_scatter(x, op)`` scatters dim 0; backward all-gathers (``avg`` divides).
* ``all_reduce(x, op)`` with gradients for sum / avg / max / min / prod.
* ``broadcast(src, root)``; backward sums the gradients onto the root.
* ``send_activations`` / ``recv_activations`` for pipeline stages.  Shapes are
  sent once per (peer, tag) and cached afterwards, so the steady state has no
  metadata message and no host synchronisation.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch

from ..comm import Communicator
from ..global_var import config

_DTYPES = [torch.float16, torch.bfloat16, torch.float32, torch.float64, torch.int8, torch.int16,
           torch.int32, torch.int64, torch.uint8, torch.bool]


def _comm(comm: Optional[Communicator]) -> Communicator:
    if not config["initialized"]:
        raise RuntimeError("BMTrain is not initialized")
    return comm if comm is not None else config["comm"]


class OpBroadcast(torch.autograd.Function):
    @staticmethod
    def forward(ctx, src, root, comm):
        ctx.comm, ctx.root = comm, root
        out = src.detach().clone().contiguous()
        comm.broadcast(out, root)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        g = grad_output.contiguous().clone()
        ctx.comm.all_reduce(g, "sum")
        return g, None, None


def broadcast(src: torch.Tensor, root: int, comm: Optional[Communicator] = None) -> torch.Tensor:
    return OpBroadcast.apply(src, root, _comm(comm))


class OpAllGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        x = x.contiguous()
        out = torch.empty((comm.size,) + tuple(x.shape), dtype=x.dtype, device=x.device)
        comm.all_gather_into(out, x)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        return grad_output[ctx.comm.rank], None


def all_gather(x: torch.Tensor, comm: Optional[Communicator] = None) -> torch.Tensor:
    """Gather ``x`` from every rank: result shape ``(group_size, *x.shape)``."""
    return OpAllGather.apply(x, _comm(comm))


class OpReduceScatter(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, op, comm):
        ctx.comm, ctx.op = comm, op
        x = x.contiguous()
        assert x.shape[0] % comm.size == 0, "reduce_scatter: dim 0 must be divisible by the group size"
        out = torch.empty((x.shape[0] // comm.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        comm.reduce_scatter_into(out, x, op)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        comm = ctx.comm
        g = grad_output.contiguous()
        out = torch.empty((comm.size,) + tuple(g.shape), dtype=g.dtype, device=g.device)
        comm.all_gather_into(out, g)
        out = out.flatten(0, 1)
        if ctx.op == "sum":
            return out, None, None
        if ctx.op == "avg":
            return out / comm.size, None, None
        raise RuntimeError(f"reduce_scatter: backward of '{ctx.op}' is not defined")


def reduce_scatter(x: torch.Tensor, op: str = "sum", comm: Optional[Communicator] = None) -> torch.Tensor:
    """Reduce over the ranks and keep this rank's slice of dim 0."""
    return OpReduceScatter.apply(x, op, _comm(comm))


class OpAllReduce(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, op, comm):
        ctx.comm, ctx.op = comm, op
        out = x.detach().clone().contiguous()
        comm.all_reduce(out, op)
        if op in ("max", "min"):
            ctx.save_for_backward(x != out)
        elif op == "prod":
            ctx.save_for_backward(out / x)
        return out

    @staticmethod
    def backward(ctx, grad_output):
        op, comm = ctx.op, ctx.comm
        if op == "sum":
            return grad_output, None, None
        if op == "avg":
            return grad_output / comm.size, None, None
        if op in ("max", "min"):
            return grad_output.masked_fill(ctx.saved_tensors[0], 0), None, None
        return grad_output * ctx.saved_tensors[0], None, None


def all_reduce(x: torch.Tensor, op: str = "sum", comm: Optional[Communicator] = None) -> torch.Tensor:
    """All-reduce with ``op`` in sum / prod / max / min / avg."""
    assert op in ("sum", "prod", "max", "min", "avg")
    return OpAllReduce.apply(x, op, _comm(comm))


# ---------------------------------------------------------------- pipeline p2p
_shape_cache: Dict[Tuple[int, int, str], Tuple[Tuple[int, ...], torch.dtype]] = {}
_META_LEN = 16


def reset_shape_cache() -> None:
    _shape_cache.clear()


def send_meta(x: torch.Tensor, next_rank: int, comm: Communicator) -> None:
    """Send the header of ``x`` (number of dimensions, dtype index, shape) to group rank ``next_rank``
    (reference: ``bmtrain/distributed/ops.py:21-30``)."""
    meta = torch.zeros(_META_LEN, dtype=torch.int64)
    meta[0] = x.dim()
    meta[1] = _DTYPES.index(x.dtype)
    for i, s in enumerate(x.shape):
        meta[2 + i] = s
    comm.send(meta.to(x.device), next_rank).wait()


def recv_meta(prev_rank: int, comm: Communicator):
    """Receive a header sent by :func:`send_meta`; returns ``(dtype, shape)`` (reference: ``bmtrain/distributed/ops.py:32-45``).
    Reading the header is a host sync; the pipeline avoids it after the first transfer by caching shapes."""
    meta = torch.zeros(_META_LEN, dtype=torch.int64, device=config["device"])
    comm.recv(meta, prev_rank).wait()
    m = meta.tolist()
    return _DTYPES[m[1]], list(m[2:2 + m[0]])


def send_activations(hidden_state: torch.Tensor, next_rank: int, comm: Communicator, tag: str = "act", static: bool = False):
    """Send a tensor to group rank ``next_rank``.

    With ``static=True`` the shape/dtype header is only exchanged the first
    time a (peer, tag) pair is used; later transfers of the same tag reuse it.
    """
    hidden_state = hidden_state.contiguous()
    key = (id(comm), next_rank, "s" + tag)
    desc = (tuple(hidden_state.shape), hidden_state.dtype)
    if not static or _shape_cache.get(key) != desc:
        send_meta(hidden_state, next_rank, comm)
        if static:
            _shape_cache[key] = desc
    work = comm.send(hidden_state, next_rank)
    return work


def recv_activations(prev_rank: int, comm: Communicator, tag: str = "act", static: bool = False) -> torch.Tensor:
    """Receive a tensor sent with :func:`send_activations` from group rank ``prev_rank``."""
    dev = config["device"]
    key = (id(comm), prev_rank, "r" + tag)
    desc = _shape_cache.get(key) if static else None
    if desc is None:
        dtype, shape = recv_meta(prev_rank, comm)
        desc = (tuple(shape), dtype)
        if static:
            _shape_cache[key] = desc
    out = torch.empty(desc[0], dtype=desc[1], device=dev)
    comm.recv(out, prev_rank).wait()
    return out
