"""Parameter / gradient statistics of a sharded model (reference: ``bmtrain/inspect/model.py:10-246``).

``inspect_model(model, glob)`` returns, for every parameter whose dotted name
matches ``glob``, a dict with name, full shape, std, mean, max, min and the
std / mean of its gradient (0.0 when there is none).  Sharded values are
gathered over their ZeRO group first; pipeline lists report the layers of all
stages on every rank.
"""
from __future__ import annotations

import fnmatch
from typing import Dict, List

import torch

from ..block_layer import Block, drain_pending
from ..global_var import config
from ..parameter import DistributedParameter, gather_flat_shard


def _stats(name: str, p: torch.Tensor, g) -> Dict:
    p = p.float()
    out = {"name": name, "shape": tuple(p.shape), "std": p.std().item(), "mean": p.mean().item(),
           "max": p.max().item(), "min": p.min().item(), "grad_std": 0.0, "grad_mean": 0.0}
    if g is not None:
        g = g.float()
        out["grad_std"], out["grad_mean"] = g.std().item(), g.mean().item()
    return out


def _gather_value(value: torch.Tensor, partition_size: int, origin_size) -> torch.Tensor:
    """Full tensor of shape ``origin_size`` from every rank's flat shard ``value`` (shards shorter than
    ``partition_size`` are zero padded first; reference: ``bmtrain/inspect/model.py:10-33``)."""
    comm = config["comm"]
    shard = torch.zeros(partition_size, dtype=value.dtype, device=value.device)
    shard[:value.numel()] = value.reshape(-1)
    full = torch.empty(partition_size * comm.size, dtype=value.dtype, device=value.device)
    comm.all_gather_into(full, shard)
    numel = 1
    for s in tuple(origin_size):
        numel *= s
    return full[:numel].view(tuple(origin_size))


def inspect_block(model: Block, param_name: str, prefix: str = "") -> List[Dict]:
    if not any(fnmatch.fnmatch(prefix + s.name, param_name) for s in model._slots):
        return []
    ret = []
    for b in model._buckets.values():
        full = torch.empty(b.total, dtype=b.dtype, device=b.storage.device)
        b.comm.all_gather_into(full, b.storage.data)
        full_grad = None
        if b.storage.grad is not None:
            full_grad = torch.empty(b.total, dtype=b.dtype, device=b.storage.device)
            b.comm.all_gather_into(full_grad, b.storage.grad.contiguous())
        for s in b.slots:
            name = prefix + s.name
            if not fnmatch.fnmatch(name, param_name):
                continue
            p = full[s.offset:s.offset + s.numel].view(s.shape)
            g = full_grad[s.offset:s.offset + s.numel].view(s.shape) if full_grad is not None else None
            ret.append(_stats(name, p, g))
    order = {prefix + s.name: i for i, s in enumerate(model._slots)}
    ret.sort(key=lambda r: order[r["name"]])
    return ret


def inspect_pipeline_transformer_block_list(pipe_model, param_name: str, prefix: str = "") -> List[Dict]:
    """Every stage inspects its own layers; results are exchanged over the pipeline group."""
    from ..store import broadcast_object

    ret = []
    for idx in range(len(pipe_model)):
        stage = pipe_model.get_stage_by_layer_id(idx)
        local = None
        if stage == pipe_model.stage_id:
            local = inspect_block(pipe_model[idx], param_name, prefix + str(idx) + ".")
        ret.extend(broadcast_object(local, config["pipe_comm"], src=stage))
    return ret


@torch.no_grad()
def inspect_model(model: torch.nn.Module, param_name: str, prefix: str = "") -> List[Dict]:
    """Statistics of the parameters of ``model`` whose name matches the glob ``param_name``."""
    from ..pipe_layer import PipelineTransformerBlockList

    drain_pending()
    if isinstance(model, PipelineTransformerBlockList):
        return inspect_pipeline_transformer_block_list(model, param_name, prefix)
    if isinstance(model, Block):
        return inspect_block(model, param_name, prefix)
    ret = []
    for name, param in model._parameters.items():
        if param is None or not fnmatch.fnmatch(prefix + name, param_name):
            continue
        if isinstance(param, DistributedParameter):
            n = param._original_shape.numel()
            p = gather_flat_shard(param.data, n, param._zero_comm).view(param._original_shape)
            g = None
            if param.grad is not None:
                g = gather_flat_shard(param.grad.data, n, param._zero_comm).view(param._original_shape)
        else:
            p, g = param.data, (param.grad.data if param.grad is not None else None)
        ret.append(_stats(prefix + name, p, g))
    for name, module in model._modules.items():
        if module is not None:
            ret.extend(inspect_model(module, param_name, prefix + name + "."))
    return ret
