"""Small helpers: printing on selected ranks, memory report, rounding, TP splitting, EMA recorder.

Counterpart of the reference's ``bmtrain/utils.py:12-184``.
"""
from __future__ import annotations

import sys
from typing import Any, Dict

import torch

from ..global_var import config

ALIGN = 4
ROW_WIDTH = 60


def check_torch_version(version_str: str) -> int:
    """>0 when the running torch is newer than ``version_str``, 0 when equal, <0 when older."""
    def parse(v):
        return [int("".join(ch for ch in p if ch.isdigit()) or 0) for p in v.split("+")[0].split(".")[:3]]
    cur, ref = parse(torch.__version__), parse(version_str)
    cur += [0] * (3 - len(cur))
    ref += [0] * (3 - len(ref))
    return (cur > ref) - (cur < ref)


def load_nccl_pypi() -> None:
    """Kept for API parity: NCCL ships inside torch, nothing has to be preloaded."""
    return None


def round_up(x: int, d: int) -> int:
    return (x + d - 1) // d * d


def print_dict(title: str, content: Dict[str, Any], file=sys.stdout) -> None:
    max_kw = max((len(k) for k in content), default=0)
    max_kw = round_up(max_kw + 3, 4)
    raw = f"{title}".center(ROW_WIDTH, "=")
    print(raw, file=file)
    for kw, val in content.items():
        print(f"{kw} :".ljust(max_kw) + f" {val}", file=file)
    print("", file=file, flush=True)


def print_block(title: str, content: str, file=sys.stdout) -> None:
    print(f" {title} ".center(ROW_WIDTH, "="), file=file)
    print(content, file=file)
    print("", file=file, flush=True)


def print_rank(*args, rank: int = 0, **kwargs) -> None:
    """``print`` on one rank only."""
    if config["rank"] == rank:
        print(*args, **kwargs)
        sys.stdout.flush()


def see_memory(message: str, detail: bool = False) -> None:
    """Report allocated / peak device memory on rank 0 and reset the peak counter."""
    print_rank(message)
    if config.get("device") is not None and config["device"].type == "cuda":
        if detail:
            print_rank(torch.cuda.memory_summary())
        else:
            gib = 1024 ** 3
            print_rank(
                f"         {round(torch.cuda.memory_allocated() / gib, 2)}GB "
                f"{round(torch.cuda.max_memory_allocated() / gib, 2)}GB"
            )
        torch.cuda.reset_peak_memory_stats()
    else:
        print_rank("         (no device memory on CPU runs)")


def tp_split_tensor(tensor: torch.Tensor, split_dim: int) -> torch.Tensor:
    """This rank's tensor-parallel slice of ``tensor`` along ``split_dim`` (contiguous copy)."""
    tp = config["tp_size"]
    if tp == 1:
        return tensor
    size = tensor.shape[split_dim]
    assert size % tp == 0, "tensor-parallel dimension must divide evenly"
    return tensor.narrow(split_dim, config["tp_rank"] * (size // tp), size // tp).contiguous()


class AverageRecorder:
    """Exponential moving average with start-up bias correction."""

    def __init__(self, alpha: float = 0.9, start_value: float = 0):
        self._value = start_value
        self.alpha = alpha
        self._steps = 0

    def record(self, v: float) -> None:
        self._value = self._value * self.alpha + v * (1 - self.alpha)
        self._steps += 1

    @property
    def value(self) -> float:
        if self._steps <= 0:
            return self._value
        return self._value / (1 - pow(self.alpha, self._steps))


from .profiling import StepTimer  # noqa: E402  (needs the helpers above)
