"""Convert an ordinary torch model in place (behaviour of reference ``bmtrain/wrapper.py:6-54``).

The conversion is two flat passes over the module tree instead of a recursive
dispatch:

1. every plain module gets its parameters replaced by
   :class:`DistributedParameter`, its buffers moved to the runtime device and
   its class re-based on :class:`DistributedModule` (so that sharded
   parameters read as full tensors inside ``forward``);
2. every ``nn.ModuleList`` is replaced by a :class:`TransformerBlockList`
   holding one :class:`Block` per entry.  The block list still supports
   ``len``, iteration and indexing, so a model that loops over its layers
   keeps working, and checkpoint keys (``layers.<i>.…``) do not change; the
   blocks are linked, which is what lets each one prefetch its neighbour's
   parameters.

Subtrees that are already distributed (a ``Block``, a block list, a
``DistributedModule``) are left untouched.
"""
from typing import List

import torch

from .block_layer import Block, TransformerBlockList
from .global_var import config
from .layer import DistributedModule
from .parameter import DistributedParameter

_FINISHED = (Block, TransformerBlockList, DistributedModule)


def _plain_modules(root: torch.nn.Module) -> List[torch.nn.Module]:
    """All modules under ``root`` (parents before children) that still need converting."""
    found, todo = [], [root]
    while todo:
        mod = todo.pop()
        found.append(mod)
        todo.extend(c for c in mod._modules.values() if c is not None and not isinstance(c, _FINISHED))
    return found


def _shard_tensors(mod: torch.nn.Module) -> None:
    for name, p in mod._parameters.items():
        if p is not None and not isinstance(p, DistributedParameter):
            mod._parameters[name] = DistributedParameter(p, requires_grad=p.requires_grad)
    for name, buf in mod._buffers.items():
        if buf is not None:
            mod._buffers[name] = buf.to(config["device"])


def _rebase(mod: torch.nn.Module) -> None:
    cls = mod.__class__
    if issubclass(DistributedModule, cls):
        # a bare nn.Module used as a container: DistributedModule already is one
        mod.__class__ = DistributedModule
    else:
        mod.__class__ = type("Distributed" + cls.__name__, (cls, DistributedModule), {})


def _as_block_list(entries: torch.nn.ModuleList) -> TransformerBlockList:
    return TransformerBlockList([m for m in entries if m is not None])


def BMTrainModelWrapper(model: torch.nn.Module) -> torch.nn.Module:
    """Shard ``model`` in place and return it (a bare ``nn.ModuleList`` comes back as a ``TransformerBlockList``)."""
    if isinstance(model, _FINISHED):
        return model
    modules = _plain_modules(model)
    for mod in modules:
        _shard_tensors(mod)
        _rebase(mod)
    # deepest lists first, so that an entry is complete before it is frozen into a block
    for mod in reversed(modules):
        for name, child in mod._modules.items():
            if isinstance(child, torch.nn.ModuleList) and not isinstance(child, TransformerBlockList):
                mod._modules[name] = _as_block_list(child)
    if isinstance(model, torch.nn.ModuleList):
        return _as_block_list(model)
    return model


# historical entry points of the reference module
model_wrapper_dispatch = BMTrainModelWrapper
make_distributed = BMTrainModelWrapper
