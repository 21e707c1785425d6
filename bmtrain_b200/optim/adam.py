"""GPU mixed-precision Adam (reference: ``bmtrain/optim/adam.py:14-252``).

State per parameter: ``step``, ``exp_avg`` (fp16 for fp16 parameters -- kept in
loss-scaled units -- else fp32), ``exp_avg_sq`` (fp32) and, for half
parameters, the fp32 master copy ``_param_fp32``.  All half-precision shards of
a parameter group are updated by ONE multi-tensor kernel launch; fp32
parameters use torch's functional Adam (coupled L2 decay, as in the reference).
"""
from __future__ import annotations

from collections import defaultdict
from copy import deepcopy
from itertools import chain

import torch

from ..ops import adam as _adam
from ._distributed import state_dict_gather


def _partition_bounds(p):
    owner = getattr(p, "_bmt_bounds", None)
    if owner is not None:
        return owner
    if getattr(p, "_start_partition", None) is not None:
        # stand-alone parameters and parameters inside a block alike: the local slice of the flattened full tensor
        return (p._start_partition, p._end_partition)
    return None


def _zero_grad(optimizer, set_to_none: bool) -> None:
    """``zero_grad`` that does not touch memory for parameters owned by a ZeRO block.

    A block's reduce-scatter produces a fresh partition gradient every step, so its old gradient is simply dropped
    (the next reduction then writes instead of accumulating) -- no zero-fill kernel per parameter and no read-modify-
    write in the reduction.  Other parameters are zeroed (or set to None) as ``torch.optim.Optimizer.zero_grad`` does."""
    for group in optimizer.param_groups:
        for p in group["params"]:
            if p.grad is None:
                continue
            if getattr(p, "_bmt_bucket", None) is not None:
                p.grad = None
            elif getattr(p, "_in_block", False):
                p.grad = None
                bucket, _ = p._block_owner()._slot_of[id(p)]
                bucket.storage.grad = None
            elif set_to_none:
                p.grad = None
            else:
                p.grad.detach_()
                p.grad.requires_grad_(False)
                p.grad.zero_()


class AdamOptimizer(torch.optim.Optimizer):
    """Adam for fp32 / fp16 / bf16 parameters living on the device."""

    _bmtrain_optimizer = True

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0, hold_steps=0):
        if not 0.0 <= lr:
            raise ValueError(f"Invalid learning rate: {lr}")
        if not 0.0 <= eps:
            raise ValueError(f"Invalid epsilon value: {eps}")
        if not 0.0 <= betas[0] < 1.0:
            raise ValueError(f"Invalid beta parameter at index 0: {betas[0]}")
        if not 0.0 <= betas[1] < 1.0:
            raise ValueError(f"Invalid beta parameter at index 1: {betas[1]}")
        if not 0.0 <= weight_decay:
            raise ValueError(f"Invalid weight_decay value: {weight_decay}")
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self._hold_steps = hold_steps

    def _on_justify_scale(self, old_scale, new_scale):
        """fp16 moments are stored in loss-scaled units: rescale them with the loss scale."""
        delta = new_scale / old_scale
        for group in self.param_groups:
            for p in group["params"]:
                state = self.state.get(p)
                if state and p.dtype == torch.float16:
                    state["exp_avg"] *= delta
                    state["exp_avg_sq"] *= delta

    def _init_state(self, p):
        state = self.state[p]
        state["step"] = 0
        m_dtype = torch.float16 if p.dtype == torch.float16 else torch.float32
        state["exp_avg"] = torch.zeros(p.size(), dtype=m_dtype, device=p.device)
        state["exp_avg_sq"] = torch.zeros(p.size(), dtype=torch.float32, device=p.device)
        if p.dtype != torch.float32:
            state["_param_fp32"] = p.detach().to(torch.float32)
        return state

    @torch.no_grad()
    def step(self, closure=None, scale=1):
        from ..block_layer import params_changed

        params_changed()
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            batches = defaultdict(list)  # (dtype, step) -> entries for one launch
            for p in group["params"]:
                if p.grad is None or not p.requires_grad:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("Adam does not support sparse gradients, please consider SparseAdam instead")
                if p.dtype not in (torch.float32, torch.float16, torch.bfloat16):
                    raise RuntimeError("Adam only supports fp32, fp16 and bf16 gradients")
                state = self.state[p]
                if len(state) == 0:
                    state = self._init_state(p)
                grad = -p.grad if group.get("maximize", False) else p.grad
                if p.dtype == torch.float32:
                    lr = 0.0 if state["step"] < self._hold_steps else group["lr"]
                    torch.optim._functional.adam(
                        [p], [grad / scale], [state["exp_avg"]], [state["exp_avg_sq"]], [],
                        [torch.tensor(float(state["step"]))],
                        amsgrad=False, beta1=group["betas"][0], beta2=group["betas"][1], lr=lr,
                        weight_decay=group["weight_decay"], eps=group["eps"], maximize=False,
                    )
                    state["step"] += 1
                else:
                    state["step"] += 1
                    if p.numel() == 0:
                        continue
                    batches[(p.dtype, state["step"])].append(
                        (state["_param_fp32"], p.data, grad.contiguous(), state["exp_avg"], state["exp_avg_sq"]))
            for (dtype, step), entries in batches.items():
                lr = 0.0 if step < self._hold_steps else group["lr"]
                _adam.adam_half_multi(entries, group["betas"][0], group["betas"][1], group["eps"], lr, scale,
                                      group["weight_decay"], step)
        return loss

    def get_avg_delta(self):
        raise NotImplementedError("get delta info is not supported in Adam optimizer , try bmt.optim.AdamOffloadOptimizer")

    def get_var_delta(self):
        raise NotImplementedError("get delta info is not supported in Adam optimizer , try bmt.optim.AdamOffloadOptimizer")

    # ------------------------------------------------------------ state dict
    def state_dict(self, gather: bool = False) -> dict:
        """Per-rank state by default; ``gather=True`` returns whole (layout independent) tensors."""
        sd = super().state_dict()
        if gather:
            sd = deepcopy(sd)
            params = list(chain.from_iterable(g["params"] for g in self.param_groups))
            comms = {i: getattr(p, "_zero_comm", None) or getattr(p, "_bmt_comm", None) for i, p in enumerate(params)}
            comms = {k: v for k, v in comms.items() if v is not None}
            sd = state_dict_gather(sd, comms)
            sd["is_whole"] = True
        else:
            sd["is_whole"] = False
        return sd

    def load_state_dict(self, state_dict: dict) -> None:
        state_dict = deepcopy(state_dict)
        groups = self.param_groups
        saved_groups = state_dict["param_groups"]
        if len(groups) != len(saved_groups):
            raise ValueError("loaded state dict has a different number of parameter groups")
        if any(len(g["params"]) != len(s["params"]) for g, s in zip(groups, saved_groups)):
            raise ValueError("loaded state dict contains a parameter group that doesn't match the size of optimizer's group")
        id_map = dict(zip(chain.from_iterable(g["params"] for g in saved_groups),
                          chain.from_iterable(g["params"] for g in groups)))
        is_whole = state_dict.get("is_whole", False)
        state = defaultdict(dict)
        for k, v in state_dict["state"].items():
            if k not in id_map:
                state[k] = v
                continue
            param = id_map[k]
            if is_whole:
                bounds = _partition_bounds(param)
                if bounds is not None:
                    for key in ("_param_fp32", "exp_avg", "exp_avg_sq"):
                        if key in v:
                            v[key] = v[key][bounds[0]:bounds[1]]
            if param.dtype != torch.float32 and "_param_fp32" not in v:
                v["_param_fp32"] = param.detach().to(torch.float32)
            m_dtype = torch.float16 if param.dtype == torch.float16 else torch.float32
            for name, dtype in (("exp_avg", m_dtype), ("exp_avg_sq", torch.float32), ("_param_fp32", torch.float32)):
                if name in v:
                    v[name] = v[name].to(param.device).to(dtype).reshape(param.shape).contiguous()
            state[param] = v
        param_groups = []
        for g, ng in zip(groups, saved_groups):
            ng["params"] = g["params"]
            param_groups.append(ng)
        self.__setstate__({"state": state, "param_groups": param_groups})

    def zero_grad(self, set_to_none: bool = False):
        _zero_grad(self, set_to_none)
