"""Recording of intermediate tensors and their gradients (reference: ``bmtrain/inspect/tensor.py:11-383``).

Inside ``with inspect_tensor() as inspector:`` every ``record_tensor(x, name)``
call keeps ``x`` (and asks autograd to keep its gradient).  After the block,
``inspector.get_summary()`` reduces min / max / mean / std (and gradient mean /
std) over all ranks.  While recording is on, blocks run without activation
recomputation so that each tensor is seen exactly once and keeps its gradient.

Tensors recorded inside a ``PipelineTransformerBlockList`` exist once per micro-batch and only on the stage that owns
the layer.  When the context is left, the micro-batch pieces are joined along the batch dimension and every stage
hands its records to the other stages of its pipeline group, so that every rank lists every layer, in layer order,
and holds its own share of the batch of each record (reference: ``bmtrain/inspect/tensor.py:28-175``).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .. import debug
from ..global_var import config


class InspectTensor:
    """Result object of an ``inspect_tensor()`` context."""

    def __init__(self) -> None:
        self.summary: List[Dict] = []
        self._raw: List[Dict] = []

    def _set_summary(self, records: List[Dict]) -> None:
        self._raw = records
        self.summary = []
        seen: Dict[str, int] = {}
        flat: List[Dict] = []
        i = 0
        while i < len(records):
            marker = records[i].get("pipe_marker")
            if marker is None:
                flat.append(records[i])
                i += 1
                continue
            j = i + 1
            while j < len(records) and (records[j].get("inside_pipe") or {}).get("segment") == marker["segment"]:
                j += 1
            flat.extend(_exchange_pipeline_records(records[i + 1:j], marker))
            i = j
        for item in flat:
            prefix = f"{item['group']}." if item["group"] is not None else ""
            base = prefix + item["name"]
            idx = seen.get(base, 0)
            seen[base] = idx + 1
            entry = dict(item)
            entry["summary_name"] = f"{prefix}{idx}.{item['name']}"
            entry["name"] = entry["summary_name"]
            self.summary.append(entry)

    def get_summary(self) -> List[Dict]:
        """Cross-rank statistics of every recorded tensor (call it after leaving the context)."""
        comm = config["comm"]
        ret = []
        for item in self.summary:
            x = item["tensor"]
            has_grad = item["requires_grad"] and x.grad is not None
            vals = [x.float().mean(), x.float().var()]
            if has_grad:
                vals += [x.grad.float().mean(), x.grad.float().var()]
            info = torch.stack(vals).float()
            comm.all_reduce(info, "sum")
            info = (info / comm.size).tolist()
            ext = torch.stack([x.float().max(), -x.float().min()])
            comm.all_reduce(ext, "max")
            ext = ext.tolist()
            ret.append({
                "name": item["summary_name"],
                "min": -ext[1], "max": ext[0], "mean": info[0], "std": math.sqrt(max(info[1], 0.0)),
                "shape": (item["shape"][0] * config["world_size"],) + tuple(item["shape"][1:]),
                "grad_mean": info[2] if has_grad else None,
                "grad_std": math.sqrt(max(info[3], 0.0)) if has_grad else None,
            })
        return ret

    def get_tensor(self, name: str, group: Optional[str] = None, index: Optional[int] = None) -> Optional[torch.Tensor]:
        """The recorded tensor called ``name`` (``index`` selects among repeated recordings; default the first)."""
        prefix = f"{group}." if group is not None else ""
        wanted = [f"{prefix}{name}", f"{prefix}0.{name}"] if index is None else [f"{prefix}{index}.{name}"]
        for item in self.summary:
            if item["summary_name"] in wanted:
                return item["tensor"]
        return None


def _exchange_pipeline_records(local: List[Dict], where: Dict) -> List[Dict]:
    """Records of one pass through a pipeline: join the micro-batches of this stage, then let every stage in turn
    broadcast its records over the pipeline group.  Returns the records of all stages in stage order; each tensor (and
    gradient) is cut down to this rank's share of the batch."""
    comm = config["pipe_comm"]
    stages, me, micros = where["stages"], where["stage_id"], where["micros"]
    per_micro: List[List[Dict]] = [[] for _ in range(micros)]
    for rec in local:
        per_micro[rec["inside_pipe"]["micro"]].append(rec)
    count = len(per_micro[0])
    assert all(len(m) == count for m in per_micro), "every micro-batch has to record the same tensors"
    mine = []
    for k in range(count):
        pieces = [per_micro[m][k] for m in range(micros)]
        first = pieces[0]
        tensor = torch.cat([p["tensor"].detach() for p in pieces], dim=0).contiguous()
        grads = [p["tensor"].grad for p in pieces]
        grad = torch.cat(grads, dim=0).contiguous() if first["requires_grad"] and all(g is not None for g in grads) else None
        mine.append({"name": first["name"], "group": first["group"], "requires_grad": first["requires_grad"], "tensor": tensor,
                     "grad": grad})
    from ..store import broadcast_object

    out: List[Dict] = []
    dev = config["device"]
    for stage in range(stages):
        if stage == me:
            meta = [{"name": r["name"], "group": r["group"], "requires_grad": r["requires_grad"], "shape": tuple(r["tensor"].shape),
                     "dtype": r["tensor"].dtype, "has_grad": r["grad"] is not None} for r in mine]
            broadcast_object(meta, comm, src=stage)
        else:
            meta = broadcast_object(None, comm, src=stage)
        for k, info in enumerate(meta):
            if stage == me:
                tensor, grad = mine[k]["tensor"], mine[k]["grad"]
            else:
                tensor = torch.empty(info["shape"], dtype=info["dtype"], device=dev)
                grad = torch.empty(info["shape"], dtype=info["dtype"], device=dev) if info["has_grad"] else None
            if comm.size > 1:
                comm.broadcast(tensor, stage)
                if grad is not None:
                    comm.broadcast(grad, stage)
            share = tensor.chunk(stages, dim=0)[me].clone()
            if info["has_grad"]:
                share.requires_grad_()
                share.grad = grad.chunk(stages, dim=0)[me].clone()
            out.append({"name": info["name"], "group": info["group"], "shape": tuple(share.shape), "tensor": share,
                        "requires_grad": info["requires_grad"], "min": None, "max": None, "mean": None, "std": None,
                        "grad_mean": None, "grad_std": None, "inside_pipe": {"stage_id": stage}})
    return out


class InspectTensorManager:
    def __init__(self) -> None:
        self._inspector: Optional[InspectTensor] = None

    def __enter__(self) -> InspectTensor:
        if debug.get("_inspect_tensor", False):
            raise RuntimeError("InspectTensorManager is already in use")
        debug.set("_inspect_tensor", True)
        debug.set("_inspect_hidden_states", [])
        self._inspector = InspectTensor()
        return self._inspector

    def __exit__(self, *args):
        debug.set("_inspect_tensor", False)
        self._inspector._set_summary(debug.get("_inspect_hidden_states", []))
        self._inspector = None
        debug.set("_inspect_hidden_states", [])


def inspect_tensor() -> InspectTensorManager:
    """Context manager that turns ``record_tensor`` on; run forward *and* backward inside it."""
    return InspectTensorManager()


def record_tensor(x: torch.Tensor, name: str, group: Optional[str] = None) -> None:
    """Remember ``x`` under ``name`` for the active ``inspect_tensor()`` context (no-op otherwise)."""
    if isinstance(x, torch.nn.Parameter):
        raise RuntimeError("Cannot inspect Parameter")
    if not debug.get("_inspect_tensor", False):
        return
    if x.requires_grad:
        x.retain_grad()
    debug.append("_inspect_hidden_states", {
        "name": name, "group": group, "shape": tuple(x.shape), "tensor": x, "requires_grad": x.requires_grad,
        "min": None, "max": None, "mean": None, "std": None, "grad_mean": None, "grad_std": None,
        "inside_pipe": debug.get("_inspect_pipe"),   # set while a pipeline stage runs its layers on a micro-batch
    })
