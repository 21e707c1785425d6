"""Sharded parameters.

``DistributedParameter`` is an ``nn.Parameter`` that is created from a *full*
tensor but only keeps this rank's contiguous 1-D slice of it; the full value is
rebuilt on demand with an all-gather over the ZeRO group (the orthogonal
``tp_zero`` group for tensor-parallel parameters).  Same contract as the
reference's ``bmtrain/parameter.py:9-206``; unlike the reference the slice
lives on whatever device the runtime was initialised on (a B200, or the CPU in
host-only runs).
"""
from __future__ import annotations

from typing import Callable, Iterable, Optional

import torch

from .comm import Communicator
from .global_var import config


def _zero_comm_for(tp_mode: bool) -> Communicator:
    return config["tp_zero_comm"] if (tp_mode and config["tp_zero_comm"] is not None) else config["zero_comm"]


class DistributedParameter(torch.nn.Parameter):
    """A parameter partitioned over the ranks of its ZeRO group.

    Args:
        data: the full (per tensor-parallel rank) value; may live on any device, including ``meta``.
        requires_grad: as for ``nn.Parameter``.
        init_method: ``f(tensor)`` used by :func:`init_parameters` to fill the full tensor.
        group: optimizer group name, see :func:`grouped_parameters`.
        tp_mode: the tensor is one tensor-parallel shard of a larger one.
        tp_split_dim: dimension along which the larger tensor was split (``-1``: replicated).
    """

    _original_shape: torch.Size
    _start_partition: int
    _end_partition: int
    _init_method: Optional[Callable]
    _in_block: bool
    _group: Optional[str]

    def __new__(cls, data: torch.Tensor, requires_grad: bool = True,
                init_method: Optional[Callable] = None, group: Optional[str] = None,
                tp_mode: bool = False, tp_split_dim: int = -1):
        if not config["initialized"]:
            raise RuntimeError("BMTrain is not initialized")
        comm = _zero_comm_for(tp_mode)
        n = data.numel()
        per = (n + comm.size - 1) // comm.size
        start = min(per * comm.rank, n)
        end = min(per * (comm.rank + 1), n)
        dev = config["device"]
        if data.is_meta:
            local = torch.empty(end - start, dtype=data.dtype, device=dev)
        else:
            local = data.detach().reshape(-1)[start:end].to(dev, copy=True)

        ret = torch.Tensor._make_subclass(cls, local, requires_grad)
        ret._original_shape = data.size()
        ret._start_partition = start
        ret._end_partition = end
        ret._init_method = init_method
        ret._in_block = False
        ret._group = group if not tp_mode else "tp"
        ret._tp_mode = tp_mode
        ret._zero_comm = comm
        ret._tp_split_dim = tp_split_dim
        if tp_mode and tp_split_dim >= 0:
            shape = list(data.size())
            shape[tp_split_dim] *= config["tp_size"]
            ret._tp_original_shape = torch.Size(shape)
        else:
            ret._tp_original_shape = data.size()
        return ret

    # nn.Parameter defines __deepcopy__/__reduce_ex__ that would drop the extra attributes
    def __deepcopy__(self, memo):
        raise RuntimeError("DistributedParameter cannot be deep-copied; build the module again instead")

    def __repr__(self):  # pragma: no cover
        return f"DistributedParameter(shard {tuple(self.shape)} of {tuple(self._original_shape)}, dtype={self.dtype})"

    @property
    def group(self) -> Optional[str]:
        """Name of the optimizer group this parameter belongs to."""
        return self._group

    # ------------------------------------------------------------------ gathers
    def gather(self) -> torch.Tensor:
        """Full value over the ZeRO group (a new tensor; use :meth:`gather_all` to also undo TP)."""
        if self._in_block:
            raise RuntimeError("parameters inside a Block are gathered by the Block")
        return OpAllGather.apply(self).detach()

    def gather_all(self) -> torch.Tensor:
        """Full value with the tensor-parallel split undone as well."""
        return self.tp_gather(self.gather())

    def tp_gather(self, zero_param: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Concatenate the tensor-parallel shards of ``zero_param`` (default: :meth:`gather`)."""
        full = zero_param if zero_param is not None else self.gather()
        if config["tp_size"] > 1 and self._tp_mode and self._tp_split_dim >= 0:
            comm: Communicator = config["tp_comm"]
            full = full.contiguous()
            out = torch.empty((comm.size,) + tuple(full.shape), dtype=full.dtype, device=full.device)
            comm.all_gather_into(out, full)
            return torch.cat(list(out.unbind(0)), dim=self._tp_split_dim)
        return full

    def _copy_data(self, data: torch.Tensor) -> None:
        """Overwrite the local shard from a full tensor."""
        self.data.copy_(data.reshape(-1)[self._start_partition:self._end_partition])


def gather_flat_shard(local: torch.Tensor, numel: int, comm: Communicator) -> torch.Tensor:
    """All-gather equal-capacity 1-D shards (the last ones may be short or empty) into ``numel`` elements."""
    per = (numel + comm.size - 1) // comm.size
    if local.numel() != per:
        padded = torch.zeros(per, dtype=local.dtype, device=local.device)
        padded[: local.numel()].copy_(local)
    else:
        padded = local.contiguous()
    out = torch.empty(per * comm.size, dtype=local.dtype, device=local.device)
    comm.all_gather_into(out, padded)
    return out[:numel]


class OpAllGather(torch.autograd.Function):
    """Full value of a stand-alone sharded parameter; backward reduce-scatters the gradient onto the shards."""

    @staticmethod
    def forward(ctx, value: DistributedParameter):
        assert isinstance(value, DistributedParameter)
        ctx.comm = value._zero_comm
        ctx.numel = value._original_shape.numel()
        ctx.bounds = (value._start_partition, value._end_partition)
        hook = getattr(value, "_bmt_pending_update", None)
        if hook is not None:
            hook(True)   # an asynchronous optimizer step is still rewriting this shard
        full = gather_flat_shard(value.data, ctx.numel, ctx.comm)
        return full.view(value._original_shape)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        comm: Communicator = ctx.comm
        per = (ctx.numel + comm.size - 1) // comm.size
        flat = grad_output.reshape(-1)
        if flat.numel() != per * comm.size:
            padded = torch.zeros(per * comm.size, dtype=flat.dtype, device=flat.device)
            padded[: flat.numel()].copy_(flat)
            flat = padded
        out = torch.empty(per, dtype=flat.dtype, device=flat.device)
        comm.reduce_scatter_into(out, flat, "sum")
        start, end = ctx.bounds
        return out[: end - start]


class ParameterInitializer:
    """``ParameterInitializer(f, *args, **kw)(t)`` calls ``f(t, *args, **kw)``."""

    def __init__(self, func: Callable, *args, **kwargs) -> None:
        self.func = func
        self._args = args
        self._kwargs = kwargs

    def __call__(self, param: torch.Tensor):
        self.func(param, *self._args, **self._kwargs)
