"""Checkpoint I/O with the reference's file layout (``bmtrain/store.py:15-325``).

``save`` gathers every parameter to its full shape (ZeRO partitions and
tensor-parallel shards re-assembled) and rank 0 writes ONE ordinary
``torch.save`` file keyed by the plain module names -- a file a vanilla
``torch.nn`` model can load.  ``load`` has rank 0 read the file; tensors
travel to the other ranks by broadcast on demand and every rank keeps its own
slice only.
"""
from __future__ import annotations

import io
import pickle
import threading
from collections import OrderedDict
from typing import Any, Dict, List, Mapping

import torch

from .block_layer import Block, TransformerBlockList, drain_pending
from .global_var import config
from .synchronize import synchronize

_DTYPE_TABLE = [torch.float16, torch.bfloat16, torch.float32, torch.float64, torch.int8, torch.int16,
                torch.int32, torch.int64, torch.uint8, torch.bool]


# -------------------------------------------------------------------- objects
def _to_bytes_tensor(obj: Any) -> torch.Tensor:
    data = pickle.dumps(obj)
    return torch.frombuffer(bytearray(data), dtype=torch.uint8).to(config["device"])


def allgather_objects(obj: Any) -> List[Any]:
    """Gather one picklable object from every rank."""
    comm = config["comm"]
    if comm.size == 1:
        return [obj]
    dev = config["device"]
    payload = _to_bytes_tensor(obj)
    sizes = torch.zeros(comm.size, dtype=torch.int64, device=dev)
    mine = torch.tensor([payload.numel()], dtype=torch.int64, device=dev)
    comm.all_gather_into(sizes, mine)
    cap = int(sizes.max().item())
    padded = torch.zeros(cap, dtype=torch.uint8, device=dev)
    padded[: payload.numel()] = payload
    out = torch.empty(comm.size * cap, dtype=torch.uint8, device=dev)
    comm.all_gather_into(out, padded)
    out = out.view(comm.size, cap).cpu()
    return [pickle.loads(out[i, : int(sizes[i])].numpy().tobytes()) for i in range(comm.size)]


def broadcast_object(obj: Any, comm=None, src: int = 0) -> Any:
    """Broadcast a picklable object from group rank ``src``."""
    comm = comm if comm is not None else config["comm"]
    if comm.size == 1:
        return obj
    dev = config["device"]
    if comm.rank == src:
        payload = _to_bytes_tensor(obj)
        size = torch.tensor([payload.numel()], dtype=torch.int64, device=dev)
    else:
        size = torch.zeros(1, dtype=torch.int64, device=dev)
    comm.broadcast(size, src)
    if comm.rank != src:
        payload = torch.empty(int(size.item()), dtype=torch.uint8, device=dev)
    comm.broadcast(payload, src)
    return obj if comm.rank == src else pickle.loads(payload.cpu().numpy().tobytes())


# ----------------------------------------------------------------------- save
def _save_to_state_dict(model: torch.nn.Module, rank: int, destination, prefix: str):
    if isinstance(model, Block):
        if rank != 0:
            destination = OrderedDict()  # throw-away: every rank takes part in the gathers
        model.state_dict(destination=destination, prefix=prefix, keep_vars=False)
        return
    if rank != 0:
        destination = OrderedDict()
    model._save_to_state_dict(destination, prefix, False)


def _save_to_local_rank0(model: torch.nn.Module, destination=None, prefix: str = ""):
    if destination is None:
        destination = OrderedDict()
    local_metadata = dict(version=getattr(model, "_version", 1))
    if hasattr(destination, "_metadata"):
        destination._metadata[prefix[:-1]] = local_metadata
    _save_to_state_dict(model, config["local_rank"], destination, prefix)
    for name, module in model._modules.items():
        if module is not None:
            _save_to_local_rank0(module, destination, prefix + name + ".")
    return destination


def _save_to_rank0(model: torch.nn.Module, destination=None, prefix: str = ""):
    """Walk the module tree; rank 0 collects full tensors, the others only take part in the collectives."""
    if destination is None:
        destination = OrderedDict()
        destination._metadata = OrderedDict()
    destination._metadata[prefix[:-1]] = dict(version=getattr(model, "_version", 1))
    if not isinstance(model, Block) and hasattr(model, "_pipeline_save"):
        model._pipeline_save(destination, prefix)
        return destination
    _save_to_state_dict(model, config["rank"], destination, prefix)
    if isinstance(model, Block):
        return destination
    for name, module in model._modules.items():
        if module is not None:
            _save_to_rank0(module, destination, prefix + name + ".")
    return destination


def _save_to_infer_model(model: torch.nn.Module, infer_model, destination=None, prefix: str = ""):
    """Stream the gathered parameters layer by layer into an external inference model (rank 0 only)."""
    config["save_param_to_cpu"] = False
    try:
        if destination is None:
            destination = OrderedDict()
            destination._metadata = OrderedDict()
        _save_to_state_dict(model, config["rank"], destination, prefix)
        if isinstance(model, Block):
            if config["rank"] == 0:
                infer_model.load_layer_state_dict(destination)
            return
        for name, module in model._modules.items():
            if module is None:
                continue
            if isinstance(module, TransformerBlockList):
                for local_name, local_module in module._modules.items():
                    local_state = OrderedDict()
                    _save_to_state_dict(local_module, config["rank"], local_state, prefix + name + "." + local_name + ".")
                    if config["rank"] == 0:
                        infer_model.load_layer_state_dict(local_state)
            else:
                _save_to_infer_model(module, infer_model, destination, prefix + name + ".")
        if config["rank"] == 0 and prefix == "":
            infer_model.load_layer_state_dict(destination)
    finally:
        config["save_param_to_cpu"] = True


def async_save_to_file(state_dict, file_path: str) -> None:
    torch.save(state_dict, file_path)
    config["finish_save"] = True


def save(model: torch.nn.Module, file_name: str, non_blocking: bool = False, save_gradient: bool = False) -> None:
    """Save the full model to ``file_name`` (written by rank 0).

    With ``non_blocking=True`` the file is written by a background thread; a
    second save joins the previous writer first.
    """
    drain_pending()
    if config["device"].type == "cuda":
        torch.cuda.synchronize()
    state_dict = _save_to_rank0(model)
    if config["rank"] == 0:
        if non_blocking:
            prev = config.get("save_thread")
            if prev is not None:
                prev.join()
            config["finish_save"] = False
            config["save_thread"] = threading.Thread(target=async_save_to_file, args=(state_dict, file_name))
            config["save_thread"].start()
        else:
            torch.save(state_dict, file_name)
    synchronize()


# ----------------------------------------------------------------------- load
class DistributedTensorWrapper:
    """Stand-in for a tensor that only rank 0 holds; ``broadcast()`` materialises it everywhere."""

    def __init__(self, tensor, shape=None):
        self._dtype = tensor.dtype
        self._device = tensor.device
        self.shape = torch.Size(shape if shape is not None else tensor.shape)
        self.tensor = tensor

    def broadcast(self) -> torch.Tensor:
        dev = config["device"]
        if config["rank"] == 0:
            t = self.tensor.to(dev).contiguous()
        else:
            t = torch.empty(self.shape, dtype=self._dtype, device=dev)
        config["comm"].broadcast(t, 0)
        return t

    def copy(self):
        return self.tensor

    def size(self):
        return self.shape

    def __getattribute__(self, name):
        if name in ("tensor", "shape", "broadcast", "copy", "size", "_dtype", "_device", "__class__", "dtype"):
            if name == "dtype":
                return object.__getattribute__(self, "_dtype")
            return object.__getattribute__(self, name)
        return getattr(object.__getattribute__(self, "tensor"), name)


class DistributedStateDictWrapper(Mapping):
    """A state dict that exists on rank 0 and is mirrored lazily on the other ranks."""

    def __init__(self, state_dict: Dict) -> None:
        self._state_dict = state_dict
        self._metadata = broadcast_object(getattr(state_dict, "_metadata", None))

    def __getitem__(self, key: str):
        dev = config["device"]
        header = torch.zeros(32, dtype=torch.int64, device=dev)
        if config["rank"] == 0:
            t = self._state_dict[key]
            vals = [t.dim(), _DTYPE_TABLE.index(t.dtype)] + list(t.shape)
            header[: len(vals)] = torch.tensor(vals, dtype=torch.int64)
        config["comm"].broadcast(header, 0)
        h = header.tolist()
        shape, dtype = h[2:2 + h[0]], _DTYPE_TABLE[h[1]]
        if config["rank"] == 0:
            return DistributedTensorWrapper(self._state_dict[key], shape=shape)
        return DistributedTensorWrapper(torch.tensor([], dtype=dtype), shape=shape)

    def copy(self):
        return self

    def __len__(self):
        return broadcast_object(len(self._state_dict))

    def __contains__(self, key: str):
        return broadcast_object(key in self._state_dict)

    def keys(self):
        return broadcast_object(list(self._state_dict.keys()))

    def __iter__(self):
        return iter(self.keys())


def load(model: torch.nn.Module, file_name: str, strict: bool = True):
    """Load a checkpoint written by :func:`save` (or by plain ``torch.save`` of a state dict).

    Only rank 0 opens the file.
    """
    if config["rank"] == 0:
        state_dict = DistributedStateDictWrapper(torch.load(file_name, map_location="cpu"))
    else:
        state_dict = DistributedStateDictWrapper({})
    ret = model.load_state_dict(state_dict, strict=strict)
    if config["device"].type == "cuda":
        torch.cuda.synchronize()
    return ret
