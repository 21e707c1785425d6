"""Barriers and tiny result helpers (reference: ``bmtrain/synchronize.py:8-73``)."""
import torch

from . import distributed
from .global_var import config


def synchronize() -> None:
    """Block the host until every rank reached this point and all queued device work is done."""
    if not config["initialized"]:
        raise RuntimeError("call init_distributed() first")
    from .optim.adam_offload import finish_all_updates

    finish_all_updates()   # optimizer steps still being applied by the offload worker
    config["comm"].barrier()
    if config["device"].type == "cuda":
        torch.cuda.synchronize()


def wait_loader() -> None:
    """Wait for outstanding parameter prefetches.

    The reference uses this as a per-block host throttle
    (``bmtrain/synchronize.py:21-29``).  The block scheduler here tracks its
    transfers with device-side handles, so this only drains what is pending.
    """
    from .block_layer import drain_pending

    drain_pending()


def sum_loss(loss: torch.Tensor, comm=None) -> torch.Tensor:
    """Average of ``loss`` over the ranks (the name is historical: it is a mean)."""
    comm = comm if comm is not None else config["comm"]
    return distributed.all_reduce(loss, "avg", comm)


def gather_result(result: torch.Tensor) -> torch.Tensor:
    """Concatenate ``result`` from all ranks along dim 0 (returned on the input's device)."""
    comm = config["comm"]
    result = result.contiguous()
    out = torch.empty((comm.size,) + tuple(result.shape), dtype=result.dtype, device=result.device)
    comm.all_gather_into(out, result)
    return out.flatten(0, 1) if result.dim() > 0 else out
