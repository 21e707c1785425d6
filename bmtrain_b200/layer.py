"""``DistributedModule``: an ``nn.Module`` whose sharded parameters read as full tensors.

Contract of the reference's ``bmtrain/layer.py:7-143``:

* reading ``self.weight`` of a stand-alone ``DistributedParameter`` returns the
  gathered tensor (autograd-aware: backward reduce-scatters the gradient);
  parameters managed by a ``Block`` are returned as they are, because the Block
  has already put the full value behind them;
* ``state_dict`` holds *full* tensors (ZeRO and tensor-parallel shards
  re-assembled), ``load_state_dict`` takes full tensors and keeps the own slice.
"""
from __future__ import annotations

import itertools

import torch

from .global_var import config
from .parameter import DistributedParameter, OpAllGather
from .utils import tp_split_tensor


class DistributedModule(torch.nn.Module):
    """Base class of modules that own :class:`DistributedParameter` objects."""

    def __getattr__(self, name: str):
        params = self.__dict__.get("_parameters")
        if params is not None and name in params:
            p = params[name]
            if isinstance(p, DistributedParameter) and not p._in_block:
                return OpAllGather.apply(p)
            return p
        return super().__getattr__(name)

    # ------------------------------------------------------------- state dict
    def _save_to_state_dict(self, destination, prefix, keep_vars):
        for name, param in self._parameters.items():
            if param is None:
                continue
            if isinstance(param, DistributedParameter):
                if param._in_block:
                    # the enclosing Block gathered the value: ``param.data`` is the full tensor
                    full = param.tp_gather(param.data).detach()
                else:
                    full = param.gather_all().detach()
                destination[prefix + name] = full.cpu() if config["save_param_to_cpu"] else full.clone()
            else:
                destination[prefix + name] = param if keep_vars else param.detach()
        for name, buf in self._buffers.items():
            if buf is not None and name not in self._non_persistent_buffers_set:
                destination[prefix + name] = buf if keep_vars else buf.detach()

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict,
                              missing_keys, unexpected_keys, error_msgs):
        from .store import DistributedTensorWrapper

        for hook in self._load_state_dict_pre_hooks.values():
            hook(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)

        persistent_buffers = {k: v for k, v in self._buffers.items() if k not in self._non_persistent_buffers_set}
        local_state = {k: v for k, v in itertools.chain(self._parameters.items(), persistent_buffers.items()) if v is not None}

        for name, param in local_state.items():
            key = prefix + name
            if key not in state_dict:
                if strict:
                    missing_keys.append(key)
                continue
            value = state_dict[key]
            is_dist = isinstance(param, DistributedParameter)
            expect_shape = param._tp_original_shape if is_dist else param.shape
            if tuple(value.shape) != tuple(expect_shape) and not (len(expect_shape) == 0 and tuple(value.shape) == (1,)):
                error_msgs.append(
                    f"size mismatch for {key}: copying a param with shape {tuple(value.shape)} from checkpoint, "
                    f"the shape in current model is {tuple(expect_shape)}."
                )
                continue
            if isinstance(value, DistributedTensorWrapper):
                value = value.broadcast()
            try:
                with torch.no_grad():
                    if is_dist:
                        if param._tp_mode and param._tp_split_dim >= 0:
                            value = tp_split_tensor(value, param._tp_split_dim)
                        if param._in_block:
                            param._block_owner()._load_param(param, value)
                        else:
                            param._copy_data(value.to(param.dtype))
                    else:
                        param.copy_(value)
            except Exception as ex:  # pragma: no cover - mirrors torch's error style
                error_msgs.append(f"While copying the parameter named \"{key}\": {ex.args}")

        if strict:
            for key in state_dict.keys():
                if key.startswith(prefix):
                    input_name = key[len(prefix):].split(".", 1)[0]
                    if input_name not in self._modules and input_name not in local_state:
                        unexpected_keys.append(key)
