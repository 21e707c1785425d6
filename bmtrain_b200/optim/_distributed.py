"""Gather per-rank optimizer state into whole tensors (reference: ``bmtrain/optim/_distributed.py:5-40``)."""
import torch

from ..global_var import config


def _gather_flat(t: torch.Tensor, comm) -> torch.Tensor:
    """Concatenate 1-D shards of possibly different length from every rank of ``comm`` (returned on the CPU)."""
    dev = config["device"]
    n = torch.tensor([t.numel()], dtype=torch.int64, device=dev)
    sizes = torch.zeros(comm.size, dtype=torch.int64, device=dev)
    comm.all_gather_into(sizes, n)
    sizes = sizes.tolist()
    cap = max(sizes)
    padded = torch.zeros(cap, dtype=t.dtype, device=dev)
    padded[: t.numel()] = t.reshape(-1).to(dev)
    out = torch.empty(cap * comm.size, dtype=t.dtype, device=dev)
    comm.all_gather_into(out, padded)
    out = out.view(comm.size, cap)
    return torch.cat([out[i, : sizes[i]] for i in range(comm.size)]).cpu()


def state_dict_gather(state_dict: dict, comms=None) -> dict:
    """Replace every tensor state by its concatenation over the parameter's ZeRO group.

    ``comms`` maps state keys to communicators (default: the world group).
    """
    for k, v in state_dict["state"].items():
        comm = (comms or {}).get(k, config["zero_comm"])
        for name in list(v.keys()):
            if torch.is_tensor(v[name]) and v[name].dim() > 0:
                v[name] = _gather_flat(v[name], comm)
    return state_dict
