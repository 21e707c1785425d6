"""Process-global runtime state.

One dictionary (``config``) holds everything ``init_distributed`` sets up:
ranks, sizes, the device, the side streams and the communicators of every
parallel group.  Mirrors the role of the reference's ``bmtrain/global_var.py:1-35``.
"""
from typing import Any, Dict


class ConfigMap(dict):
    """dict with attribute access; unknown keys raise KeyError like a dict."""

    def __getattr__(self, name: str) -> Any:
        try:
            return self[name]
        except KeyError as exc:  # pragma: no cover - trivial
            raise AttributeError(name) from exc


config: Dict[str, Any] = ConfigMap(
    initialized=False,
    rank=0,
    world_size=1,
    local_rank=0,
    local_size=1,
    pipe_size=1,
    pipe_enabled=False,
    tp_size=1,
    tp_rank=0,
    zero_rank=0,
    tp_zero_rank=0,
    zero_size=1,
    tp_zero_size=1,
    micros=1,
    save_param_to_cpu=True,
    device=None,
    backend=None,
)


def rank() -> int:
    """Global rank of this process."""
    return config["rank"]


def world_size() -> int:
    """Number of processes in the job."""
    return config["world_size"]
