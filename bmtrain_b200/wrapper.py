"""Convert an ordinary torch model in place (reference: ``bmtrain/wrapper.py:6-54``).

Parameters become :class:`DistributedParameter`, buffers move to the runtime
device, every ``nn.ModuleList`` becomes a :class:`TransformerBlockList` of
:class:`Block` and module classes are re-based on :class:`DistributedModule`
so that sharded parameters read as full tensors.
"""
import torch

from .block_layer import Block, TransformerBlockList
from .global_var import config
from .layer import DistributedModule
from .parameter import DistributedParameter


def make_distributed(model: torch.nn.Module) -> torch.nn.Module:
    for kw in list(model._parameters.keys()):
        if model._parameters[kw] is not None and not isinstance(model._parameters[kw], DistributedParameter):
            model._parameters[kw] = DistributedParameter(
                model._parameters[kw], requires_grad=model._parameters[kw].requires_grad
            )
    for kw in list(model._buffers.keys()):
        if model._buffers[kw] is not None:
            model._buffers[kw] = model._buffers[kw].to(config["device"])
    is_module_list = isinstance(model, torch.nn.ModuleList)
    pre_module = None
    for kw in list(model._modules.keys()):
        if model._modules[kw] is None:
            continue
        if is_module_list:
            if not isinstance(model._modules[kw], Block):
                model._modules[kw] = Block(model_wrapper_dispatch(model._modules[kw]))
            if pre_module is not None:
                model._modules[kw].set_pre_module(pre_module)
            pre_module = model._modules[kw]
        else:
            model._modules[kw] = model_wrapper_dispatch(model._modules[kw])
    if not isinstance(model, DistributedModule):
        model.__class__ = type("Distributed" + model.__class__.__name__, (model.__class__, DistributedModule), {})
    return model


def model_wrapper_dispatch(model: torch.nn.Module) -> torch.nn.Module:
    if isinstance(model, TransformerBlockList):
        return model
    if isinstance(model, DistributedModule):
        return model
    if isinstance(model, Block):
        return model
    return make_distributed(model)


def BMTrainModelWrapper(model: torch.nn.Module) -> torch.nn.Module:
    """Shard ``model`` in place and return it."""
    return model_wrapper_dispatch(model)
