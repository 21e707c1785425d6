"""Loss scaling and multi-optimizer stepping (reference: ``bmtrain/optim/optim_manager.py:9-226``).

State machine: ``backward`` multiplies the loss by ``loss_scale / grad_scale``
(``grad_scale`` defaults to the ZeRO group size, which turns the summing
gradient reduce-scatter into a mean).  ``step`` first looks for inf/nan in all
half-precision gradients (one multi-tensor scan, one max all-reduce, one host
read); on overflow the scale shrinks, gradients are zeroed and nothing is
stepped; otherwise every optimizer steps with the current scale, schedulers
advance, and after ``loss_scale_steps`` clean steps the scale grows.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..block_layer import drain_pending, fused_sq_norms, grads_modified, params_changed
from ..global_var import config
from ..lr_scheduler.warmup import WarmupLRScheduler
from ..ops import infnan
from ..utils import print_rank


def found_overflow(param_groups) -> bool:
    """True when any half-precision gradient of ``param_groups``, on any rank, holds inf or nan (one host read)."""
    dev = config["device"]
    flag = torch.zeros(1, dtype=torch.uint8, device=dev)
    grads = [p.grad for group in param_groups for p in group["params"]
             if p.grad is not None and p.dtype != torch.float32]
    infnan.multi_has_inf_nan([g if g.is_contiguous() else g.contiguous() for g in grads], flag)
    if dev.type == "cuda":
        # gradients reduced by the fused NVLink kernel were checked there
        from ..parallel import symm

        for rt in symm._runtimes.values():
            if rt is not None:
                flag |= rt.overflow
                rt.overflow.zero_()
    if config["comm"].size > 1:
        f32 = flag.to(torch.int32)
        config["comm"].all_reduce(f32, "max")
        flag = f32
    return int(flag.item()) > 0


def check_overflow(param_groups) -> None:
    """Reference-compatible form (``bmtrain/optim/optim_manager.py:9-21``): raises ``OverflowError`` on inf/nan."""
    if found_overflow(param_groups):
        raise OverflowError("Gradient overflow")


_status_host = {}


def check_peer_status() -> None:
    """Raise when a peer-memory kernel of an earlier step gave up waiting for another rank (its bounded wait ran out).

    The status words are copied to pinned host memory without synchronising; the copy started by the previous call is the
    one that is looked at, so a failure surfaces one step late instead of costing a host sync per step."""
    if config["device"] is None or config["device"].type != "cuda":
        return
    from ..parallel import symm

    for key, rt in symm._runtimes.items():
        if rt is None:
            continue
        slot = _status_host.get(key)
        if slot is None:
            # one pinned word per runtime, allocated once (pinning memory is far too slow to do per step)
            slot = _status_host[key] = [torch.zeros(1, dtype=torch.int32).pin_memory(), None]
        host, event = slot
        if event is not None:
            if not event.query():
                continue  # the previous copy has not landed yet: look again next step
            if int(host[0]) != 0:
                slot[1] = None
                rt.check()
        host.copy_(rt.status, non_blocking=True)
        event = torch.cuda.Event()
        event.record()
        slot[1] = event


def grad_rescale(param_groups, scale) -> None:
    for group in param_groups:
        for p in group["params"]:
            if p.grad is not None and p.requires_grad:
                p.grad /= scale


class LossScaler:
    """Dynamic loss scale: ``scale`` shrinks by ``factor`` after a step with inf/nan gradients (never below ``floor``)
    and grows by ``factor`` after ``interval`` clean steps in a row (never above ``ceiling``).  ``on_change(old, new)``
    is called before every change so that state kept in scaled units can follow."""

    def __init__(self, scale, factor, interval, floor, ceiling, on_change):
        self.enabled = scale is not None
        self.scale = scale if self.enabled else 1
        self.factor = factor if factor > 1 else 1 / factor
        self.interval, self.floor, self.ceiling = interval, floor, ceiling
        self.clean_steps = 0
        self._on_change = on_change

    def set(self, value) -> None:
        self._on_change(self.scale, value)
        self.scale = value
        self.clean_steps = 0

    def overflowed(self) -> None:
        if self.scale > self.floor:
            self.set(self.scale / self.factor)

    def stepped(self) -> None:
        self.clean_steps += 1
        if self.clean_steps >= self.interval and self.scale < self.ceiling:
            self.set(self.scale * self.factor)


class OptimManager:
    """Drives several optimizers (+ schedulers) under one dynamic loss scale."""

    def __init__(self, loss_scale: Optional[float] = None, loss_scale_factor: float = 2, loss_scale_steps: int = 1024,
                 min_loss_scale=1, max_loss_scale=float("inf"), grad_scale: Optional[int] = None):
        self.optimizers = []
        self.lr_schedulers = []
        self._scaler = LossScaler(loss_scale, loss_scale_factor, loss_scale_steps, min_loss_scale, max_loss_scale,
                                  self._rescale_optimizer_state)
        self.grad_scale = config["zero_size"] if grad_scale is None else grad_scale

    # the scaler's fields under the names the reference exposes (read and written by user code and checkpoints)
    loss_scale = property(lambda self: self._scaler.scale, lambda self, v: setattr(self._scaler, "scale", v))
    loss_scale_enabled = property(lambda self: self._scaler.enabled, lambda self, v: setattr(self._scaler, "enabled", v))
    steps_since_last_scale = property(lambda self: self._scaler.clean_steps,
                                      lambda self, v: setattr(self._scaler, "clean_steps", v))
    loss_scale_factor = property(lambda self: self._scaler.factor)
    loss_scale_steps = property(lambda self: self._scaler.interval)
    min_loss_scale = property(lambda self: self._scaler.floor)
    max_loss_scale = property(lambda self: self._scaler.ceiling)

    def _rescale_optimizer_state(self, old, new) -> None:
        with torch.no_grad():
            for optimizer in self.optimizers:
                hook = getattr(optimizer, "_on_justify_scale", None)
                if hook is not None:
                    hook(old, new)

    def _justify_scale(self, scale) -> None:
        self._scaler.set(scale)

    def add_optimizer(self, optimizer: torch.optim.Optimizer, lr_scheduler: Optional[WarmupLRScheduler] = None):
        self.optimizers.append(optimizer)
        self.lr_schedulers.append(lr_scheduler)

    def scale_loss(self, loss: torch.Tensor) -> torch.Tensor:
        return loss * (self.loss_scale / self.grad_scale)

    def backward(self, loss: torch.Tensor):
        """Backward of the scaled loss; returns once all gradient reductions are queued behind it."""
        # with gradient accumulation many backward passes separate two optimizer steps: a kernel that gave up waiting for
        # another rank is reported here too (one pass late, without a host sync)
        check_peer_status()
        for optimizer in self.optimizers:
            announce = getattr(optimizer, "_expect_step", None)
            if announce is not None:
                announce(self.loss_scale)   # lets an offloading optimizer start on finished gradients during backward
        self.scale_loss(loss).backward()
        drain_pending()

    def zero_grad(self):
        for optimizer in self.optimizers:
            optimizer.zero_grad(set_to_none=False)

    def step(self):
        drain_pending()
        check_peer_status()
        scaler = self._scaler
        if scaler.enabled and any(found_overflow(opt.param_groups) for opt in self.optimizers):
            shrunk = scaler.scale / scaler.factor if scaler.scale > scaler.floor else scaler.scale
            print_rank("Gradient overflow, change scale from %lf to %lf" % (scaler.scale, shrunk))
            scaler.overflowed()
            with torch.no_grad():
                self.zero_grad()
            return  # nothing is stepped, schedulers do not advance
        params_changed()
        for optimizer, lr_scheduler in zip(self.optimizers, self.lr_schedulers):
            if getattr(optimizer, "_bmtrain_optimizer", False):
                optimizer.step(scale=scaler.scale)
            else:
                if scaler.enabled:
                    grad_rescale(optimizer.param_groups, scaler.scale)
                optimizer.step()
            if lr_scheduler is not None:
                lr_scheduler.step()
        if scaler.enabled:
            scaler.stepped()

    def clip_grad_norm(self, param_groups, max_norm, norm_type=2, eps=1e-6):
        """Clip the global gradient norm (computed on the still loss-scaled gradients); returns the unscaled norm."""
        drain_pending()
        scale = self.loss_scale
        dev = config["device"]
        parameters = [p for group in param_groups for p in group["params"]]
        grads = [p.grad.data for p in parameters if p.grad is not None]
        if norm_type == "inf":
            total = torch.zeros(1, dtype=torch.float32, device=dev)
            for g in grads:
                if g.numel():
                    total = torch.maximum(total, g.abs().max().float().reshape(1))
            config["comm"].all_reduce(total, "max")
            total_norm = total[0]
        else:
            norm_type = float(norm_type)
            total = torch.zeros(1, dtype=torch.float32, device=dev)
            if norm_type == 2.0:
                # buckets whose gradients came out of the fused reduce-scatter kernel bring their sum of squares along; only
                # the remaining gradients are read again
                known, parts = fused_sq_norms(parameters)
                rest = [p.grad.data for p in parameters if p.grad is not None and id(p) not in known]
                infnan.multi_sq_norm([g if g.is_contiguous() else g.contiguous() for g in rest], total)
                for part in parts:
                    total += part
            else:
                for g in grads:
                    total += g.float().norm(norm_type) ** norm_type
            config["comm"].all_reduce(total, "sum")
            total_norm = total[0] ** (1.0 / norm_type)
        clip_coef = float(max_norm * scale) / (total_norm + eps)
        infnan.multi_scale(grads, clip_coef.reshape(1))
        grads_modified()
        for optimizer in self.optimizers:
            if hasattr(optimizer, "_invalidate_staged"):
                optimizer._invalidate_staged()
        return total_norm / scale

    def state_dict(self, gather_opt: bool = False) -> dict:
        def opt_state(opt):
            try:
                return opt.state_dict(gather_opt)
            except TypeError:
                return opt.state_dict()

        return {
            "optimizers": [opt_state(opt) for opt in self.optimizers],
            "lr_schedulers": [lrs.state_dict() if lrs else None for lrs in self.lr_schedulers],
            "loss_scale": self.loss_scale,
            "loss_scale_enabled": self.loss_scale_enabled,
        }

    def load_state_dict(self, state_dict: dict) -> None:
        assert len(self.optimizers) == len(state_dict["optimizers"])
        assert len(self.lr_schedulers) == len(state_dict["lr_schedulers"])
        for opt, opt_st in zip(self.optimizers, state_dict["optimizers"]):
            opt.load_state_dict(opt_st)
        for lrs, lrs_st in zip(self.lr_schedulers, state_dict["lr_schedulers"]):
            if lrs is not None and lrs_st is not None:
                lrs.load_state_dict(lrs_st)
        self.loss_scale = state_dict["loss_scale"]
        self.loss_scale_enabled = state_dict["loss_scale_enabled"]
