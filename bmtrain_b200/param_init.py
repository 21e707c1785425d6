"""Parameter initialisation and optimizer grouping (reference: ``bmtrain/param_init.py:8-105``)."""
from __future__ import annotations

from typing import Dict, Generator, Iterable, List, Optional, Tuple

import torch

from .block_layer import Block
from .global_var import config
from .parameter import DistributedParameter
from .utils import tp_split_tensor


def init_distributed_parameter(params: Iterable[torch.nn.Parameter]) -> None:
    """Initialise stand-alone distributed parameters.

    The ``init_method`` runs on a full-size temporary on every rank (same seed
    everywhere, hence the same values as a single-process run); each rank keeps
    its slice.
    """
    dev = config["device"]
    for param in params:
        if not isinstance(param, DistributedParameter) or param._init_method is None:
            continue
        with torch.no_grad():
            tmp = torch.empty(param._tp_original_shape, dtype=param.dtype, device=dev)
            param._init_method(tmp)
            if param._tp_mode and param._tp_split_dim >= 0:
                tmp = tp_split_tensor(tmp, param._tp_split_dim)
            param._copy_data(tmp)
            del tmp


def iterate_parameters(model: torch.nn.Module):
    for _, val in model._parameters.items():
        if hasattr(val, "_in_block") and val._in_block:
            return []
        yield val


def init_parameters(model: torch.nn.Module) -> None:
    """Initialise every parameter of ``model`` with its ``init_method``."""
    modules = model.named_modules()
    for _, module in modules:
        if isinstance(module, Block):
            module.init_parameters()
        else:
            init_distributed_parameter(iterate_parameters(module))
    if config["device"].type == "cuda":
        torch.cuda.current_stream().synchronize()


def grouped_parameters(model: torch.nn.Module) -> Generator[Tuple[Optional[str], List[torch.nn.Parameter]], None, None]:
    """``(group name, [parameters])`` pairs.  Blocks contribute their flat partitions."""
    ret: Dict[Optional[str], List[torch.nn.Parameter]] = {}
    for module in model.modules():
        if isinstance(module, Block):
            for kw, params in module.grouped_parameters():
                ret.setdefault(kw, []).extend(params)
        else:
            for param in module._parameters.values():
                if param is None:
                    continue
                group = param.group if isinstance(param, DistributedParameter) else None
                ret.setdefault(group, []).append(param)
    yield from ret.items()
