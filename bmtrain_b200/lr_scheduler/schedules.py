"""Concrete decay rules: constant, Noam, linear, cosine and exponential."""
import math

from .warmup import WarmupLRScheduler


class NoDecay(WarmupLRScheduler):
    """Constant ``start_lr`` after warm-up."""

    def get_lr_decay(self, num_iter) -> float:
        return self.start_lr


class Noam(WarmupLRScheduler):
    """``start_lr * n / warmup^1.5`` during warm-up, then ``start_lr / sqrt(n)``."""

    def get_lr_warmup(self, num_iter) -> float:
        return self.start_lr * num_iter / (self.warmup_iter * math.sqrt(self.warmup_iter))

    def get_lr_decay(self, num_iter) -> float:
        return self.start_lr / math.sqrt(num_iter)


class Linear(WarmupLRScheduler):
    """Straight line from ``start_lr`` at the end of warm-up to 0 at ``end_iter``."""

    def get_lr_decay(self, num_iter) -> float:
        remaining = (self.end_iter - num_iter) / (self.end_iter - self.warmup_iter)
        return max(0.0, self.start_lr * remaining)


class Cosine(WarmupLRScheduler):
    """Half cosine from ``start_lr`` to 0 between ``warmup_iter`` and ``end_iter``."""

    def get_lr_decay(self, num_iter) -> float:
        span = max(1, self.end_iter - self.warmup_iter)
        progress = (num_iter - self.warmup_iter) / span
        return max(0.0, 0.5 * self.start_lr * (1.0 + math.cos(math.pi * progress)))


class Exponential(WarmupLRScheduler):
    """``start_lr * gamma^(n - warmup_iter)`` after warm-up."""

    def __init__(self, optimizer, start_lr, warmup_iter, end_iter, num_iter=0, gamma=0.95) -> None:
        self.gamma = gamma
        super().__init__(optimizer, start_lr, warmup_iter, end_iter, num_iter)

    def get_lr_decay(self, num_iter) -> float:
        return max(0.0, self.start_lr * self.gamma ** (num_iter - self.warmup_iter))
