"""Learning-rate schedules with linear warm-up (reference: ``bmtrain/lr_scheduler/*.py``).

A schedule is a pure function of the iteration number; ``step()`` advances the
counter and writes the new rate into every parameter group of the optimizer.
"""
from __future__ import annotations

import torch


class WarmupLRScheduler:
    """Base: ``lr = warmup(n)`` for ``n < warmup_iter`` else ``decay(n)``."""

    _STATE = ("start_lr", "warmup_iter", "end_iter", "num_iter")

    def __init__(self, optimizer: torch.optim.Optimizer, start_lr, warmup_iter, end_iter, num_iter=0) -> None:
        self.optimizer = optimizer
        self.start_lr, self.warmup_iter, self.end_iter = start_lr, warmup_iter, end_iter
        self.num_iter = num_iter
        self._current_lr = None
        self.step(num_iter)

    # the two pieces a concrete schedule defines
    def get_lr_warmup(self, num_iter) -> float:
        return self.start_lr * num_iter / self.warmup_iter

    def get_lr_decay(self, num_iter) -> float:
        raise NotImplementedError

    def get_lr(self) -> float:
        if self.num_iter < 0:
            raise ValueError("iteration number must be non-negative")
        piece = self.get_lr_warmup if self.num_iter < self.warmup_iter else self.get_lr_decay
        return piece(self.num_iter)

    @property
    def current_lr(self):
        return self._current_lr

    def step(self, num_iter=None) -> None:
        self.num_iter = self.num_iter + 1 if num_iter is None else num_iter
        self._current_lr = self.get_lr()
        for group in self.optimizer.param_groups:
            group["lr"] = self._current_lr

    def state_dict(self):
        return {k: getattr(self, k) for k in self._STATE}

    def load_state_dict(self, state_dict) -> None:
        for k in self._STATE:
            setattr(self, k, state_dict[k])
        self.step(self.num_iter)
