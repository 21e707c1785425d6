"""Bandwidth sweeps for all-gather, reduce-scatter and paired send/recv.

The reference prints one un-warmed shot per size (``bmtrain/benchmark/all_gather.py:21`` etc.).
Here each size is warmed up, timed with CUDA events over several iterations and
reported as the maximum over ranks; on CPU runs wall-clock time is used.
"""
from __future__ import annotations

import time
from typing import List, Tuple

import torch

from ..global_var import config
from ..utils import print_rank

SIZES = [2 ** p for p in range(10, 31, 2)]


def _timeit(fn, iters: int = 5, warmup: int = 2) -> float:
    dev = config["device"]
    for _ in range(warmup):
        fn()
    if dev.type == "cuda":
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(iters):
            fn()
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end) / iters
    else:
        t0 = time.perf_counter()
        for _ in range(iters):
            fn()
        ms = (time.perf_counter() - t0) * 1e3 / iters
    t = torch.tensor([ms], dtype=torch.float32, device=dev)
    config["comm"].all_reduce(t, "max")
    return float(t.item())


def all_gather(sizes=None) -> List[Tuple[int, float, float]]:
    """(bytes gathered per rank, ms, GB/s received) for each size."""
    comm, dev, out = config["comm"], config["device"], []
    for nbytes in sizes or SIZES:
        n = nbytes // 2 // comm.size
        if n == 0:
            continue
        src = torch.empty(n, dtype=torch.float16, device=dev)
        dst = torch.empty(n * comm.size, dtype=torch.float16, device=dev)
        ms = _timeit(lambda: comm.all_gather_into(dst, src))
        bw = (comm.size - 1) * n * 2 / ms / 1e6
        print_rank(f"all_gather    {nbytes:>12d} B  {ms:9.3f} ms  {bw:9.2f} GB/s")
        out.append((nbytes, ms, bw))
    return out


def reduce_scatter(sizes=None) -> List[Tuple[int, float, float]]:
    comm, dev, out = config["comm"], config["device"], []
    for nbytes in sizes or SIZES:
        n = nbytes // 2 // comm.size
        if n == 0:
            continue
        src = torch.zeros(n * comm.size, dtype=torch.float16, device=dev)
        dst = torch.empty(n, dtype=torch.float16, device=dev)
        ms = _timeit(lambda: comm.reduce_scatter_into(dst, src, "avg"))
        bw = (comm.size - 1) * n * 2 / ms / 1e6
        print_rank(f"reduce_scatter {nbytes:>11d} B  {ms:9.3f} ms  {bw:9.2f} GB/s")
        out.append((nbytes, ms, bw))
    return out


def send_recv(sizes=None) -> List[Tuple[int, float, float]]:
    """Ranks pair up (2i <-> 2i+1): even ranks send, odd ranks receive."""
    comm, dev, out = config["comm"], config["device"], []
    if comm.size < 2:
        print_rank("send_recv needs at least two ranks")
        return out
    for nbytes in sizes or SIZES:
        n = nbytes // 2
        buf = torch.empty(n, dtype=torch.float16, device=dev)

        def once():
            peer = comm.rank ^ 1
            if peer >= comm.size:
                return
            (comm.send if comm.rank % 2 == 0 else comm.recv)(buf, peer).wait()

        ms = _timeit(once)
        bw = n * 2 / ms / 1e6
        print_rank(f"send_recv     {nbytes:>12d} B  {ms:9.3f} ms  {bw:9.2f} GB/s")
        out.append((nbytes, ms, bw))
    return out
