"""Process bring-up: rendezvous, device binding, streams, parallel groups.

Same call and the same group arithmetic as the reference
(``bmtrain/init.py:14-258``): ``init_distributed(init_method, seed, pipe_size,
num_micro_batches, tp_size)`` fills the global ``config``.  The plumbing is
``torch.distributed`` -- NCCL (NVLink 5 / NVSwitch) when the process owns a
GPU, gloo on CPU-only hosts so that every host-side code path can be tested
without hardware.
"""
from __future__ import annotations

import datetime
import os
import random
from typing import Optional

import torch
import torch.distributed as dist

from .comm import Communicator
from .global_var import config


class Topology:
    """Group ids / group ranks for every parallel dimension.

    World ranks are laid out ``[stage][zero-within-stage]`` with tensor-parallel
    partners adjacent (``tp_id = rank % tp_size``), as in the reference
    (``bmtrain/init.py:189-254``).
    """

    def __init__(self, rank: int, world_size: int, pipe_size: int, tp_size: int):
        if world_size % (pipe_size * tp_size) != 0:
            raise ValueError(
                "world size must be divisible by pipe_size * tp_size "
                f"(world {world_size}, pipe {pipe_size}, tp {tp_size})"
            )
        self.rank = rank
        self.world_size = world_size
        self.stages = pipe_size
        self.tp_size = tp_size
        self.stage_size = world_size // pipe_size
        self.dp_size = world_size // (pipe_size * tp_size)

        self.pipe_idx = rank % self.stage_size
        self.stage_id = rank // self.stage_size
        self.tp_id = rank % tp_size
        self.tp_idx = rank // tp_size
        self.pp_zero_idx = self.stage_id
        self.pp_zero_id = self.pipe_idx
        self.tp_zero_idx = self.tp_id
        self.tp_zero_id = self.tp_idx
        self.pp_tp_zero_idx = self.stage_id * tp_size + self.tp_id
        self.pp_tp_zero_id = self.pipe_idx // tp_size
        self.zero_idx = 0
        self.zero_id = rank

    # member lists (global ranks, group order) of the group this rank belongs to
    def pipe_ranks(self):
        return [s * self.stage_size + self.pipe_idx for s in range(self.stages)]

    def pp_zero_ranks(self):
        return [self.stage_id * self.stage_size + i for i in range(self.stage_size)]

    def tp_ranks(self):
        return [self.tp_idx * self.tp_size + i for i in range(self.tp_size)]

    def tp_zero_ranks(self):
        return [i * self.tp_size + self.tp_id for i in range(self.world_size // self.tp_size)]

    def pp_tp_zero_ranks(self):
        base = self.stage_id * self.stage_size
        return [base + i * self.tp_size + self.tp_id for i in range(self.stage_size // self.tp_size)]

    def get_group_id(self, group_name: str) -> int:
        return {"pipe": self.pipe_idx, "zero": self.zero_idx, "tp_zero": self.tp_zero_idx, "tp": self.tp_idx}[group_name]

    def get_group_rank(self, group_name: str) -> int:
        return {"pipe": self.stage_id, "zero": self.zero_id, "tp_zero": self.tp_zero_id, "tp": self.tp_id}[group_name]


topology = Topology  # reference spelling


def _all_groups(world_size: int, member_fn_name: str, pipe_size: int, tp_size: int):
    """Distinct member lists of one group kind over the whole world, in a fixed order."""
    seen, out = set(), []
    for r in range(world_size):
        members = tuple(getattr(Topology(r, world_size, pipe_size, tp_size), member_fn_name)())
        if members not in seen:
            seen.add(members)
            out.append(list(members))
    return out


def _make_comm(kind: str, fn: str, rank: int, world_size: int, pipe_size: int, tp_size: int) -> Communicator:
    """Create every group of one kind (collective call) and return the one this rank is in."""
    mine = None
    for members in _all_groups(world_size, fn, pipe_size, tp_size):
        group = dist.new_group(ranks=members) if len(members) > 1 else None
        if rank in members:
            mine = Communicator(group, members, rank, name=kind)
    assert mine is not None
    return mine


def _read_cpu_list(text: str):
    """``"0-3,8,10-11"`` -> [0, 1, 2, 3, 8, 10, 11] (format of the kernel's ``cpulist`` files)."""
    out = []
    for part in text.strip().split(","):
        if not part:
            continue
        lo, _, hi = part.partition("-")
        out.extend(range(int(lo), int(hi or lo) + 1))
    return out


def _numa_layout(local_size: int):
    """(cpus of every NUMA node, node of every local GPU) from sysfs, or None when that cannot be told (one node, no CUDA,
    no sysfs).  The offloading optimizer streams tens of bytes per parameter between host memory and the cores of its
    rank: on a host with several sockets those cores and that memory should be the ones the rank's GPU hangs on."""
    try:
        nodes = {}
        base = "/sys/devices/system/node"
        for entry in os.listdir(base):
            if entry.startswith("node") and entry[4:].isdigit():
                with open(os.path.join(base, entry, "cpulist")) as f:
                    nodes[int(entry[4:])] = _read_cpu_list(f.read())
        if len(nodes) < 2 or not torch.cuda.is_available():
            return None
        gpu_node = []
        for i in range(local_size):
            props = torch.cuda.get_device_properties(i)
            bus = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
            with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
                gpu_node.append(int(f.read().strip()))
        return nodes, gpu_node
    except (OSError, AttributeError, ValueError, RuntimeError, AssertionError):
        return None


def _split_cpus(cpus, local_rank: int, local_size: int, layout=None):
    """The cores of ``cpus`` that local rank ``local_rank`` gets.  Without a NUMA layout: equal consecutive parts.  With
    one: the cores of the node its GPU is attached to, shared out among the ranks whose GPUs sit on that node (a rank
    whose node is unknown or has no usable cores falls back to the equal split)."""
    if local_size <= 1 or len(cpus) < local_size:
        return list(cpus)
    per = len(cpus) // local_size
    equal = list(cpus[local_rank * per:(local_rank + 1) * per])
    if layout is None:
        return equal
    nodes, gpu_node = layout
    node = gpu_node[local_rank] if local_rank < len(gpu_node) else -1
    allowed = set(cpus)
    here = [c for c in nodes.get(node, []) if c in allowed]
    mates = [r for r in range(local_size) if r < len(gpu_node) and gpu_node[r] == node]
    if node < 0 or len(here) < len(mates) or local_rank not in mates:
        return equal
    share = len(here) // len(mates)
    k = mates.index(local_rank)
    return here[k * share:(k + 1) * share]


def _partition_cpus(local_rank: int, local_size: int):
    try:
        cpus = sorted(os.sched_getaffinity(0))
    except AttributeError:  # pragma: no cover - non linux
        return None
    if local_size <= 1 or len(cpus) < local_size:
        return cpus
    mine = _split_cpus(cpus, local_rank, local_size, _numa_layout(local_size))
    try:
        os.sched_setaffinity(0, mine)
    except OSError:  # pragma: no cover
        return cpus
    return mine


def init_distributed(
    init_method: str = "env://",
    seed: int = 0,
    pipe_size: int = -1,
    num_micro_batches: Optional[int] = None,
    tp_size: int = 1,
    *,
    device: Optional[str] = None,
    verbose: bool = True,
):
    """Initialise the runtime.  Launch one process per GPU with ``torchrun``.

    Args mirror ``bmtrain/init.py:14-20``.  ``device`` ("cuda"/"cpu", default:
    cuda when available, or the ``BMT_DEVICE`` environment variable) is an
    addition: on "cpu" the same engine runs over gloo.
    """
    from .utils import print_dict
    from .synchronize import synchronize

    torch.backends.cudnn.enabled = False

    rank = int(os.environ.get("RANK", "0"))
    world_size = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", str(rank)))
    local_size = int(os.environ.get("LOCAL_WORLD_SIZE", str(world_size)))
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "10010")
    os.environ.setdefault("RANK", str(rank))
    os.environ.setdefault("WORLD_SIZE", str(world_size))

    dev_kind = device or os.environ.get("BMT_DEVICE") or ("cuda" if torch.cuda.is_available() else "cpu")
    if dev_kind == "cuda":
        torch.cuda.set_device(local_rank % max(torch.cuda.device_count(), 1))
        dev = torch.device("cuda", torch.cuda.current_device())
        backend = "nccl"
    else:
        dev = torch.device("cpu")
        backend = "gloo"

    if not dist.is_initialized():
        kwargs = dict(backend=backend, init_method=init_method, rank=rank, world_size=world_size,
                      timeout=datetime.timedelta(seconds=int(os.environ.get("BMT_TIMEOUT", "1800"))))
        if backend == "nccl":
            kwargs["device_id"] = dev
        dist.init_process_group(**kwargs)

    pipe_enabled = pipe_size > 0
    pipe_size = pipe_size if pipe_size > 0 else 1
    config.update(
        initialized=True,
        rank=rank, world_size=world_size, local_rank=local_rank, local_size=local_size,
        pipe_size=pipe_size, pipe_enabled=pipe_enabled, tp_size=tp_size,
        device=dev, backend=backend, save_param_to_cpu=True,
        micros=(num_micro_batches if num_micro_batches else pipe_size) if pipe_enabled else 1,
    )

    if dev.type == "cuda":
        config["calc_stream"] = torch.cuda.current_stream()
        config["load_stream"] = torch.cuda.Stream(priority=-1)
        config["tp_comm_stream"] = torch.cuda.Stream(priority=-1)
        config["pp_comm_stream"] = torch.cuda.Stream(priority=-1)
        config["barrier_stream"] = torch.cuda.Stream()
        config["load_event"] = torch.cuda.Event()
    else:
        for k in ("calc_stream", "load_stream", "tp_comm_stream", "pp_comm_stream", "barrier_stream", "load_event"):
            config[k] = None

    topo = Topology(rank, world_size, pipe_size, tp_size)
    config["topology"] = topo
    config["zero_rank"] = topo.get_group_rank("zero") if pipe_size == 1 else topo.pp_zero_id
    config["tp_rank"] = topo.get_group_rank("tp")
    config["tp_zero_rank"] = topo.get_group_rank("tp_zero")
    config["tp_zero_size"] = topo.dp_size
    config["zero_size"] = world_size // pipe_size

    cpus = _partition_cpus(local_rank, local_size)
    if cpus:
        torch.set_num_threads(max(1, min(len(cpus), int(os.environ.get("BMT_MAX_THREADS", "64")))))
    config["cpus"] = cpus

    torch.manual_seed(seed)
    random.seed(seed)
    try:
        import numpy as np

        np.random.seed(seed)
    except ModuleNotFoundError:  # pragma: no cover
        pass

    world = list(range(world_size))
    config["comm"] = Communicator(dist.group.WORLD if world_size > 1 else None, world, rank, name="world")
    config["pipe_comm"] = config["pp_zero_comm"] = None
    config["tp_comm"] = config["tp_zero_comm"] = config["pp_tp_zero_comm"] = None
    if pipe_enabled:
        config["pipe_comm"] = _make_comm("pipe", "pipe_ranks", rank, world_size, pipe_size, tp_size)
        config["pp_zero_comm"] = _make_comm("pp_zero", "pp_zero_ranks", rank, world_size, pipe_size, tp_size)
    if tp_size > 1:
        config["tp_comm"] = _make_comm("tp", "tp_ranks", rank, world_size, pipe_size, tp_size)
        config["tp_zero_comm"] = _make_comm("tp_zero", "tp_zero_ranks", rank, world_size, pipe_size, tp_size)
    if pipe_size > 1 and tp_size > 1:
        config["pp_tp_zero_comm"] = _make_comm("pp_tp_zero", "pp_tp_zero_ranks", rank, world_size, pipe_size, tp_size)
    config["zero_comm"] = config["comm"]

    if verbose and os.environ.get("BMT_QUIET", "0") != "1":
        for i in range(world_size):
            if i == rank:
                print_dict("Initialization", {
                    "rank": rank, "local_rank": local_rank, "world_size": world_size, "local_size": local_size,
                    "master": f"{os.environ['MASTER_ADDR']}:{os.environ['MASTER_PORT']}",
                    "device": str(dev), "backend": backend, "cpus": cpus,
                })
            synchronize()
    else:
        synchronize()


def is_initialized() -> bool:
    return bool(config["initialized"])


def shutdown() -> None:
    """Tear the process groups down (tests call this between cases)."""
    from . import watchdog

    watchdog.stop()
    for value in list(config.values()) if hasattr(config, "values") else []:
        shm = getattr(value, "_shm", None)
        if shm is not None:
            shm.close()
            value._shm = None
    if config.get("device") is not None and config["device"].type == "cuda":
        from .parallel import symm

        torch.cuda.synchronize()
        symm.reset()
    if dist.is_initialized():
        dist.destroy_process_group()
    config["initialized"] = False
