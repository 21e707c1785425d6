"""Step timer with named phases, NVTX ranges and max-over-ranks reduction.

The reference times its example loop with ``time.time`` and an EMA (``example/train.py:75,114-129``); there is no
device timing and no cross-rank view.  ``StepTimer`` brackets phases with CUDA events on the current stream (wall clock
on CPU runs), pushes an NVTX range of the same name so the phases show up in timeline tools, and reports each phase as
the maximum over the ranks of a communicator, which is the figure a synchronous data-parallel step is bound by.

    timer = bmt.utils.StepTimer()
    with timer.phase("forward"):
        loss = model(...)
    with timer.phase("backward"):
        optim_manager.backward(loss)
    with timer.phase("optimizer"):
        optim_manager.step()
    print(timer.finish_step())      # {"forward": ms, "backward": ms, "optimizer": ms, "total": ms}
"""
from __future__ import annotations

import time
from contextlib import contextmanager
from typing import Dict, List, Optional, Tuple

import torch

from ..global_var import config


class StepTimer:
    def __init__(self, comm=None, nvtx: bool = True):
        self._comm = comm
        self._nvtx = nvtx
        self._open: List[Tuple[str, object, object]] = []
        self._history: Dict[str, List[float]] = {}

    def _cuda(self) -> bool:
        dev = config.get("device") if hasattr(config, "get") else None
        return dev is not None and dev.type == "cuda"

    @contextmanager
    def phase(self, name: str):
        cuda = self._cuda()
        if cuda:
            if self._nvtx:
                torch.cuda.nvtx.range_push(name)
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
        else:
            start, end = time.perf_counter(), None
        try:
            yield
        finally:
            if cuda:
                end.record()
                if self._nvtx:
                    torch.cuda.nvtx.range_pop()
            else:
                end = time.perf_counter()
            self._open.append((name, start, end))

    def finish_step(self, reduce: bool = True) -> Dict[str, float]:
        """Milliseconds per phase of the step that just ended (phases of the same name add up) and their total; with
        ``reduce`` the maximum over the ranks of the communicator (default: all ranks).  Synchronises the device."""
        cuda = self._cuda()
        if cuda:
            torch.cuda.synchronize()
        out: Dict[str, float] = {}
        for name, start, end in self._open:
            ms = start.elapsed_time(end) if cuda else (end - start) * 1e3
            out[name] = out.get(name, 0.0) + ms
        self._open = []
        out["total"] = sum(out.values())
        comm = self._comm or (config["comm"] if config.get("initialized") else None)
        if reduce and comm is not None and comm.size > 1:
            names = sorted(out)
            t = torch.tensor([out[n] for n in names], dtype=torch.float32, device=config["device"])
            comm.all_reduce(t, "max")
            out = {n: float(v) for n, v in zip(names, t.tolist())}
        for n, v in out.items():
            self._history.setdefault(n, []).append(v)
        return out

    def averages(self, skip: int = 0) -> Dict[str, float]:
        """Mean of every phase over the finished steps, leaving out the first ``skip`` (warm-up)."""
        return {n: sum(v[skip:]) / max(len(v[skip:]), 1) for n, v in self._history.items()}
