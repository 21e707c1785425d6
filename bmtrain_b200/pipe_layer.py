"""Pipeline-parallel block list (GPipe schedule; reference: ``bmtrain/pipe_layer.py:17-314``).

Ranks are split into ``pipe_size`` stages of consecutive ranks; the layers are
split as evenly as possible with the earlier stages taking the remainder.  A
call works on the batch of the whole pipeline group:

1. every rank all-gathers its input batch over the pipeline group, the group
   batch is cut into ``micros`` micro-batches;
2. for each micro-batch a stage receives the activation of the previous stage
   (stage 0 uses the gathered input), runs its layers and sends the result on;
3. the last stage's outputs are broadcast and every rank keeps the slice that
   belongs to its own samples, so embedding / head / loss run data parallel.

Stage-to-stage transfers are NCCL point-to-point messages with cached shapes
(one header the first time a shape is seen, none afterwards, no host sync in
steady state); sends are asynchronous and overlap the next micro-batch.
Inside a stage the blocks use ZeRO-2 over the stage's ranks: parameters are
gathered at the first micro-batch and kept until the last backward
micro-batch, gradients are reduced once per step.
"""
from __future__ import annotations

from collections import OrderedDict
from typing import Dict, Iterable, Iterator, List, Union

import torch

from . import block_layer as _bl
from . import debug
from .block_layer import Block, _block_wrapper
from .distributed.ops import recv_activations, send_activations
from .global_var import config

_inflight: List = []


def _gather_stack(t: torch.Tensor, comm) -> torch.Tensor:
    t = t.contiguous()
    out = torch.empty((comm.size,) + tuple(t.shape), dtype=t.dtype, device=t.device)
    comm.all_gather_into(out, t)
    return out


def _reap_sends() -> None:
    while _inflight:
        _inflight.pop(0).wait()


_bl._extra_drains.append(_reap_sends)


class PipePreFunction(torch.autograd.Function):
    """Gather the pipeline group's inputs and cut them into micro-batches."""

    @staticmethod
    def forward(ctx, hidden_state, *args):
        comm = config["pipe_comm"]
        *args, batch_related = args
        micros = config["micros"]
        gathered = _gather_stack(hidden_state, comm).requires_grad_()
        batch = hidden_state.shape[0]
        per_micro: List[List] = [[] for _ in range(micros)]
        requires, rule = [], []
        for arg in args:
            if torch.is_tensor(arg):
                everyone = _gather_stack(arg, comm)
                if arg.dim() == hidden_state.dim() and arg.shape[0] == batch:
                    rule.append(True)
                    pieces = [p.requires_grad_(arg.requires_grad) for p in everyone.flatten(0, 1).chunk(micros, dim=0)]
                else:
                    rule.append(False)
                    pieces = [everyone[0].requires_grad_(arg.requires_grad) for _ in range(micros)]
                requires.append(arg.requires_grad)
            else:
                rule.append(False)
                pieces = [arg] * micros
                requires.append(False)
            for i in range(micros):
                per_micro[i].append(pieces[i])
        ctx.requires, ctx.per_micro = requires, per_micro
        ctx.batch_related = [i in batch_related for i in range(len(args))] if len(batch_related) else rule
        return gathered, per_micro

    @staticmethod
    def backward(ctx, grads, _unused):
        comm, topo, micros = config["pipe_comm"], config["topology"], config["micros"]
        grads = grads.contiguous().clone()
        comm.broadcast(grads, 0)
        arg_grads = []
        for idx, req in enumerate(ctx.requires):
            if not req:
                arg_grads.append(None)
                continue
            g = torch.cat([ctx.per_micro[m][idx].grad for m in range(micros)], dim=0).contiguous()
            comm.all_reduce(g, "sum")
            if ctx.batch_related[idx]:
                arg_grads.append(g.chunk(topo.stages)[topo.stage_id])
            else:
                arg_grads.append(g.chunk(micros)[0])
        return (grads[topo.stage_id],) + tuple(arg_grads) + (None,)


class PipePostFunction(torch.autograd.Function):
    """Broadcast the last stage's outputs; every rank keeps its own samples."""

    @staticmethod
    def forward(ctx, last_hidden, hidden_states=None, forward_stage_ranges=None, backward_stage_ranges=None,
                last_hidden_shape=None, return_hidden_states=False):
        comm, topo = config["pipe_comm"], config["topology"]
        ctx.return_hidden_states = return_hidden_states
        last = last_hidden.detach().clone().contiguous()
        comm.broadcast(last, topo.stages - 1)
        output = last.chunk(topo.stages, dim=0)[topo.stage_id].clone().requires_grad_()
        if not return_hidden_states:
            return output
        ctx.backward_stage_ranges = backward_stage_ranges
        middles = []
        for stage in range(topo.stages):
            if stage == topo.stage_id:
                mid = hidden_states.detach().clone().contiguous()
            else:
                mid = torch.zeros((forward_stage_ranges[stage],) + tuple(last_hidden_shape),
                                  device=hidden_states.device, dtype=hidden_states.dtype)
            comm.broadcast(mid, stage)
            middles.append(mid.chunk(topo.stages, dim=1)[topo.stage_id].clone())
        return output, torch.cat(middles, dim=0).requires_grad_()

    @staticmethod
    def backward(ctx, grads, grad_middle=None):
        comm, topo = config["pipe_comm"], config["topology"]
        grad_list = _gather_stack(grads, comm).flatten(0, 1)
        if not ctx.return_hidden_states:
            return grad_list
        mine = None
        for stage in range(topo.stages):
            rng = ctx.backward_stage_ranges[stage]
            part = grad_middle[rng.start:rng.stop].transpose(0, 1).contiguous()
            part = _gather_stack(part, comm).flatten(0, 1).transpose(0, 1)
            if stage == topo.stage_id:
                mine = part
        return grad_list, mine, None, None, None, None


class StagePreFunction(torch.autograd.Function):
    """Entry of a stage: take the activation from the previous stage; backward sends the gradient back."""

    @staticmethod
    def forward(ctx, input, stage_id):
        ctx.stage_id = stage_id
        if stage_id == 0:
            return input
        out = recv_activations(stage_id - 1, config["pipe_comm"], tag="fwd", static=True)
        return out.requires_grad_()

    @staticmethod
    def backward(ctx, grad):
        if ctx.stage_id != 0:
            _inflight.append(send_activations(grad.contiguous(), ctx.stage_id - 1, config["pipe_comm"], tag="bwd", static=True))
        return grad, None


class StagePostFunction(torch.autograd.Function):
    """Exit of a stage: hand the activation to the next stage; backward receives its gradient."""

    @staticmethod
    def forward(ctx, outputs, stage_id):
        ctx.stage_id = stage_id
        ctx.is_last = stage_id == config["pipe_size"] - 1
        if not ctx.is_last:
            _inflight.append(send_activations(outputs.detach(), stage_id + 1, config["pipe_comm"], tag="fwd", static=True))
        return outputs.view_as(outputs)

    @staticmethod
    def backward(ctx, grad):
        if not ctx.is_last:
            return recv_activations(ctx.stage_id + 1, config["pipe_comm"], tag="bwd", static=True), None
        return grad, None


class PipelineTransformerBlockList(torch.nn.Module):
    """``TransformerBlockList`` whose layers are spread over the pipeline stages."""

    _modules: Dict[str, Block]

    def __init__(self, modules: Iterable[torch.nn.Module], num_hidden: int = 1) -> None:
        super().__init__()
        self.num_hidden = num_hidden
        topo = config["topology"]
        self.stages = topo.stages
        self.stage_id = topo.stage_id
        self.pipe_idx = topo.pipe_idx
        module_dict: dict = {}
        for idx, module in enumerate(modules):
            module = _block_wrapper(module, module_dict, "PIPE")
            module._zero_level = 2  # parameters stay gathered across the micro-batches of a step
            self.add_module(str(idx), module)
        self.layer_ids = self.get_range_by_stage_id(self.stage_id)
        pre = None
        for layer_id in self.layer_ids:
            module = self._modules[str(layer_id)]
            module.set_pre_module(pre)
            pre = module
            module._is_first_layer = module._is_last_layer = False
        if len(self.layer_ids):
            self._modules[str(self.layer_ids[0])]._is_first_layer = True
            self._modules[str(self.layer_ids[-1])]._is_last_layer = True

    def __len__(self) -> int:
        return len(self._modules)

    def __iter__(self) -> Iterator[Block]:
        return iter(self._modules.values())

    def __getitem__(self, index: Union[int, str]) -> Block:
        return self._modules[str(index)]

    def forward(self, hidden_state, *args, batch_related=[], return_hidden_states: bool = False):
        self.return_hidden_states = return_hidden_states
        micros = config["micros"]
        if not hidden_state.requires_grad and torch.is_grad_enabled():
            hidden_state = hidden_state.detach().requires_grad_()
        gathered, args_list = PipePreFunction.apply(hidden_state, *args, batch_related)
        micro_inputs = gathered.flatten(0, 1).chunk(micros, dim=0)
        outputs, hidden_states = [], []
        recording = debug.get("_inspect_tensor", False)
        if recording:
            # tensors recorded inside the stages are put together across micro-batches and stages when the inspector is
            # read: a marker tells it (on every rank of the pipeline group, with or without records) where a pass begins
            segment = debug.get("_inspect_pipe_segments", 0) + 1
            debug.set("_inspect_pipe_segments", segment)
            where = {"segment": segment, "stage_id": self.stage_id, "stages": self.stages, "micros": micros}
            debug.append("_inspect_hidden_states", {"pipe_marker": dict(where)})
        for micro_idx, (x, arg) in enumerate(zip(micro_inputs, args_list)):
            seen = []
            if recording:
                debug.set("_inspect_pipe", dict(where, micro=micro_idx))
            x = StagePreFunction.apply(x, self.stage_id)
            for layer_id in self.layer_ids:
                block = self._modules[str(layer_id)]
                block._micro_idx = micro_idx
                if return_hidden_states:
                    seen.append(x)
                x = block(x, *arg)
            x = StagePostFunction.apply(x, self.stage_id)
            outputs.append(x)
            if return_hidden_states:
                hidden_states.append(torch.stack(seen, dim=0))
        if recording:
            debug.set("_inspect_pipe", None)
        _reap_sends()
        last_hidden = torch.cat(outputs, dim=0)
        if not return_hidden_states:
            return PipePostFunction.apply(last_hidden)
        stacked = torch.cat(hidden_states, dim=1)
        fwd_ranges = [self.get_part_len_by_stage_id(s) for s in range(self.stages)]
        bwd_ranges = [self.get_range_by_stage_id(s) for s in range(self.stages)]
        return PipePostFunction.apply(last_hidden, stacked, fwd_ranges, bwd_ranges, last_hidden.shape, True)

    # --------------------------------------------------------- layer partition
    def get_part_len_by_stage_id(self, stage_id: int) -> int:
        return len(self) // self.stages + (1 if stage_id < len(self) % self.stages else 0)

    def get_range_by_stage_id(self, stage_id: int) -> range:
        start = sum(self.get_part_len_by_stage_id(s) for s in range(stage_id))
        return range(start, start + self.get_part_len_by_stage_id(stage_id))

    def get_stage_by_layer_id(self, layer_id: int) -> int:
        for stage in range(self.stages):
            if layer_id in self.get_range_by_stage_id(stage):
                return stage
        raise IndexError(layer_id)

    # --------------------------------------------------------------- state dict
    def _pipeline_save(self, destination, prefix: str) -> None:
        """Collect every layer's full state on global rank 0 (stage leaders send their layers)."""
        for name, module in self._modules.items():
            idx = int(name)
            layer_prefix = prefix + name + "."
            owner_stage = self.get_stage_by_layer_id(idx)
            keys = [layer_prefix + n for n, _ in module._module.named_parameters()]
            keys += [layer_prefix + n for n, _ in module._module.named_buffers()]
            if idx in self.layer_ids:
                dst = OrderedDict()
                module.state_dict(destination=dst, prefix=layer_prefix, keep_vars=False)
                if config["topology"].pp_zero_id == 0:
                    if config["rank"] == 0:
                        destination.update(dst)
                    else:
                        for key in keys:
                            send_activations(dst[key].to(config["device"]), 0, config["pipe_comm"]).wait()
            if config["rank"] == 0 and idx not in self.layer_ids:
                for key in keys:
                    destination[key] = recv_activations(owner_stage, config["pipe_comm"]).cpu()

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        self._pipeline_save(destination, prefix)
