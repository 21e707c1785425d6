"""Helpers to run a test body on several ranks (one process per rank, gloo on CPU or nccl on GPUs)."""
import importlib
import os
import socket
import sys
import traceback

import torch.multiprocessing as mp


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, module, fn, kwargs, init_kwargs, device, errq):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), LOCAL_WORLD_SIZE=str(world),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), BMT_QUIET="1")
    here = os.path.dirname(os.path.abspath(__file__))
    sys.path.insert(0, here)
    sys.path.insert(0, os.path.dirname(here))
    try:
        import torch

        torch.set_num_threads(1)
        import bmtrain_b200 as bmt

        bmt.init_distributed(seed=0, device=device, **init_kwargs)
        torch.set_num_threads(1)
        getattr(importlib.import_module(module), fn)(**kwargs)
        bmt.synchronize()
        bmt.shutdown()
    except Exception:
        errq.put((rank, traceback.format_exc()))
        raise


def run_distributed(module: str, fn: str, world: int, device: str = "cpu", init_kwargs=None, timeout: int = 240, **kwargs):
    """Run ``module.fn(**kwargs)`` on ``world`` ranks; raises with the first rank's traceback on failure."""
    ctx = mp.get_context("spawn")
    errq = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, module, fn, kwargs, init_kwargs or {}, device, errq))
             for r in range(world)]
    for p in procs:
        p.start()
    failed = False
    for p in procs:
        p.join(timeout)
        if p.is_alive():
            failed = True
    if failed:
        for p in procs:
            if p.is_alive():
                p.kill()
    errors = []
    while not errq.empty():
        errors.append(errq.get())
    if errors or failed or any(p.exitcode != 0 for p in procs):
        msg = "\n".join(f"[rank {r}]\n{tb}" for r, tb in errors) or "a rank timed out or crashed"
        raise AssertionError(f"distributed run of {module}.{fn} failed:\n{msg}")
