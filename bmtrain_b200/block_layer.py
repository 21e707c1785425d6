"""ZeRO blocks and block lists.

A :class:`Block` wraps a module whose parameters are all
:class:`~bmtrain_b200.parameter.DistributedParameter` and makes it the unit of
parameter sharding (ZeRO-2/3), activation checkpointing and gradient
reduction.  Behavioural contract: reference ``bmtrain/block_layer.py:49-726``,
``bmtrain/zero_context.py`` and ``bmtrain/hook_func.py``.  The implementation
is organised differently:

* each block owns a few *flat buckets* (one per dtype / grad flag / optimizer
  group); a bucket is cut into equal partitions, one per rank of the ZeRO
  group, and the local partition is a single flat ``nn.Parameter``;
* the whole forward/backward of a block is ONE autograd node
  (:class:`_BlockFunction`) that gathers the buckets, runs (or re-runs) the
  inner module, and reduce-scatters the gradients;
* gathers and reduce-scatters are issued asynchronously and only awaited where
  their result is consumed: a block list prefetches the next block's
  parameters while the current one computes, and a gradient reduce-scatter runs
  under the backward pass of the following blocks.  Nothing in the steady state
  blocks the host.
"""
from __future__ import annotations

import inspect
import weakref
from collections import OrderedDict
from typing import Dict, Iterable, Iterator, List, Optional, Tuple, Union

import torch

from . import debug
from .comm import Communicator, DONE
from .global_var import config
from .parameter import DistributedParameter, gather_flat_shard
from .utils import round_up, tp_split_tensor

# element alignment of every parameter inside a bucket: 512 bytes, so that each
# tensor starts on a boundary TMA and 128-bit vector accesses can use
_ALIGN_BYTES = 512

# ---------------------------------------------------------------- pending work
_pending: List = []
_callback_queued = False
_extra_drains: List = []  # other subsystems (pipeline sends) register completion hooks here


# Bumped whenever parameter values change (optimizer step, checkpoint load): a gathered copy made before that -- e.g. a
# prefetch for a block that was then never run -- must not be used afterwards.
_param_epoch = [0]


def params_changed() -> None:
    _param_epoch[0] += 1


# Gradients of block-owned parameters that went through the fused reduce-scatter kernel have two companions per bucket:
# an fp32 copy of the partition gradient (created the first time a bucket accumulates over micro-steps; from then on the
# accumulation runs in fp32 and `.grad` is its rounding) and the sum of squares of the partition gradient (for the
# gradient norm).  Both describe `.grad` as the kernel left it: code that rewrites gradients in place (clipping) calls
# grads_modified(), after which the companions are rebuilt / ignored.
_grad_epoch = [0]
_fused_buckets = weakref.WeakSet()


def grads_modified() -> None:
    _grad_epoch[0] += 1


def _grad_companions() -> bool:
    """Off unless BMT_GRAD_FP32=1 (or ``config["grad_accum_fp32"]``): the extended kernel entry has been compiled and
    read, not yet run on a GPU."""
    import os

    return bool(config.get("grad_accum_fp32", False)) or os.environ.get("BMT_GRAD_FP32", "0") == "1"


def fused_sq_norms(parameters):
    """Sum of squares already known from the fused reduce-scatter: returns (ids of the parameters it covers, list of
    one-element fp32 device tensors to add up).  A bucket counts only if every one of its gradient holders is in
    ``parameters`` (its figure is for the whole partition) and nothing rewrote the gradients since."""
    wanted = {id(p) for p in parameters}
    covered, parts = set(), []
    for b in list(_fused_buckets):
        if getattr(b, "sq_tag", None) != _grad_epoch[0] or b.storage is None or b.storage.grad is None:
            continue
        if id(b.storage) in wanted:
            holders = [b.storage]
        else:
            holders = [s.param for s in b.slots if s.param.requires_grad]
            if not holders or any(id(h) not in wanted for h in holders):
                continue
        covered.update(id(h) for h in holders)
        parts.append(b.sqsum)
    return covered, parts


def update_ready(param, block: bool = True) -> bool:
    """An optimizer that applies its step asynchronously marks the parameters it is still rewriting
    (``_bmt_pending_update``).  ``block`` true: wait until the new values are in place (the current stream is made to wait
    for their upload); false: only tell whether they are."""
    hook = getattr(param, "_bmt_pending_update", None)
    return True if hook is None else hook(block)


def drain_pending() -> None:
    """Complete every outstanding gradient reduce-scatter (stream-level wait, no host block on NCCL)."""
    global _callback_queued
    _callback_queued = False
    while _pending:
        _pending.pop(0)()
    for hook in _extra_drains:
        hook()


def _queue_backward_callback() -> None:
    """Make sure pending reductions are completed when the running backward pass ends."""
    global _callback_queued
    if _callback_queued:
        return
    try:
        torch.autograd.Variable._execution_engine.queue_callback(drain_pending)
        _callback_queued = True
    except RuntimeError:
        # not inside a backward pass (e.g. torch.autograd.grad from a test): finish now
        drain_pending()


def _get_param_kw(param: DistributedParameter) -> str:
    """Bucket key of a parameter: dtype, grad flag and optimizer group."""
    kw = f"{str(param.dtype).split('.')[-1]}_{'grad' if param.requires_grad else 'nograd'}"
    if param.group is not None:
        kw += f"_g_{param.group}"
    return kw


class _Slot:
    """Where one inner parameter lives inside its bucket."""

    __slots__ = ("name", "param", "offset", "numel", "shape", "lo", "hi")

    def __init__(self, name, param, offset, numel, shape):
        self.name, self.param, self.offset, self.numel, self.shape = name, param, offset, numel, shape
        self.lo = self.hi = 0  # overlap with the local partition, in bucket coordinates


class _Bucket:
    """One flat, partitioned parameter buffer of a block."""

    def __init__(self, key: str, dtype: torch.dtype, group: Optional[str], comm: Communicator):
        self.key, self.dtype, self.group, self.comm = key, dtype, group, comm
        self.slots: List[_Slot] = []
        self.total = 0
        self.part = 0
        self.storage: Optional[torch.nn.Parameter] = None
        self.full: Optional[torch.Tensor] = None
        self.full_grad: Optional[torch.Tensor] = None
        self.work = None

    @property
    def begin(self) -> int:
        return self.comm.rank * self.part

    @property
    def end(self) -> int:
        return (self.comm.rank + 1) * self.part


def _rng_state():
    state = {"cpu": torch.get_rng_state()}
    if config["device"] is not None and config["device"].type == "cuda":
        state["cuda"] = torch.cuda.get_rng_state()
    return state


class _restore_rng:
    """Run a region under a saved RNG state and put the current one back afterwards."""

    def __init__(self, state):
        self.state = state

    def __enter__(self):
        self.outer = _rng_state()
        torch.set_rng_state(self.state["cpu"])
        if "cuda" in self.state:
            torch.cuda.set_rng_state(self.state["cuda"])

    def __exit__(self, *exc):
        torch.set_rng_state(self.outer["cpu"])
        if "cuda" in self.outer:
            torch.cuda.set_rng_state(self.outer["cuda"])


def _flatten_out(out):
    """Split a module output into (tensors, rebuild description)."""
    if isinstance(out, torch.Tensor):
        return [out], None
    if isinstance(out, (tuple, list)):
        tensors, spec = [], []
        for o in out:
            if isinstance(o, torch.Tensor):
                spec.append(len(tensors))
                tensors.append(o)
            else:
                spec.append(("const", o))
        return tensors, (type(out), spec)
    raise TypeError(f"a Block must return a tensor or a tuple/list of tensors, got {type(out)}")


def _rebuild_out(tensors, spec):
    if spec is None:
        return tensors[0]
    kind, items = spec
    vals = [tensors[i] if isinstance(i, int) else i[1] for i in items]
    return tuple(vals) if kind is tuple else vals


class _BlockFunction(torch.autograd.Function):
    """Forward/backward of one block as a single autograd node."""

    @staticmethod
    def forward(ctx, block: "Block", placeholder, arg_spec, *tensors):
        ctx.block = block
        ctx.arg_spec = arg_spec
        ctx.req = [t.requires_grad for t in tensors]
        ctx.checkpoint = block._use_checkpoint and not debug.get("_inspect_tensor", False)
        block._enter_forward(_fill(arg_spec, tensors))
        if ctx.checkpoint:
            ctx.rng = _rng_state()
            ctx.inputs = tensors
            with torch.no_grad():
                out = block._module(*_fill(arg_spec, tensors))
            flat, ctx.out_spec = _flatten_out(out)
        else:
            detached = [t.detach().requires_grad_(r) for t, r in zip(tensors, ctx.req)]
            with torch.enable_grad():
                out = block._module(*_fill(arg_spec, detached))
            graph_out, ctx.out_spec = _flatten_out(out)
            ctx.detached, ctx.graph_out = detached, graph_out
            flat = [o.detach() for o in graph_out]
        block._exit_forward()
        non_diff = [o for o in flat if not (o.is_floating_point() or o.is_complex())]
        if non_diff:
            ctx.mark_non_differentiable(*non_diff)
        block._last_out_spec = ctx.out_spec
        return tuple(flat)

    @staticmethod
    def backward(ctx, *grad_outs):
        block: Block = ctx.block
        block._enter_backward(_fill(ctx.arg_spec, ctx.inputs) if ctx.checkpoint else None)
        if ctx.checkpoint:
            detached = [t.detach().requires_grad_(r) for t, r in zip(ctx.inputs, ctx.req)]
            with _restore_rng(ctx.rng), torch.enable_grad():
                out = block._module(*_fill(ctx.arg_spec, detached))
            graph_out, _ = _flatten_out(out)
        else:
            detached, graph_out = ctx.detached, ctx.graph_out
        outs, grads = [], []
        for o, g in zip(graph_out, grad_outs):
            if g is not None and o.requires_grad:
                outs.append(o)
                grads.append(g)
        if outs:
            torch.autograd.backward(outs, grads)
        block._exit_backward()
        ctx.detached = ctx.graph_out = ctx.inputs = None
        return (None, None, None) + tuple(d.grad if r else None for d, r in zip(detached, ctx.req))


def _fill(arg_spec, tensors):
    return [tensors[a] if isinstance(a, int) else a[1] for a in arg_spec]


class Block(torch.nn.Module):
    """Unit of ZeRO sharding + activation checkpointing.

    Args:
        inner_module: module whose parameters are all ``DistributedParameter``.
        use_checkpoint: recompute the forward in backward instead of keeping activations.
        zero_level: 3 = gather parameters again in backward, 2 = keep the gathered copy from forward.
        initialized: parameters already carry values (skip :func:`init_parameters` for this block).
        mode: ``"BLOCK"`` / ``"ZERO"`` or ``"PIPE"`` (inside a pipeline list; uses the per-stage ZeRO group).
    """

    def __init__(self, inner_module: torch.nn.Module, use_checkpoint: bool = True, zero_level: int = 3,
                 initialized: bool = False, mode: str = "BLOCK", _share: Optional["Block"] = None):
        super().__init__()
        object.__setattr__(self, "_module", inner_module)
        self._inputs = None
        self._layer_dict = {}
        self._forward_block_ctx = None
        self._backward_block_ctx = None
        self._buckets: "OrderedDict[str, _Bucket]" = OrderedDict()
        self._slots: List[_Slot] = []
        self._initialized = initialized
        self._use_checkpoint = use_checkpoint
        self._is_first_layer = True
        self._is_last_layer = True
        self._pre_module = None
        self._next_module = None
        self._ref_block: Optional[Block] = None
        self._mode = mode
        self._micro_idx = 0
        self._resident = False
        self._need_release = True
        self.all_input_no_grad = False
        self.all_param_no_grad = False
        assert zero_level in (2, 3), "zero_level must be 2 or 3"
        self._zero_level = zero_level
        self._last_out_spec = None
        self._grad_mode = False
        self._slot_parity = 0
        if _share is not None:
            self.reference(_share)
        else:
            self.init_param_storage()

    # -------------------------------------------------------------- properties
    @property
    def _param_info(self):
        """List of per-parameter records (name, parameter, bucket key, offset, size, shape)."""
        return [
            {"parameter": s.param, "name": s.name, "offset": s.offset, "size": s.numel, "shape": s.shape,
             "kw_name": _get_param_kw(s.param)} for s in self._slots
        ]

    @property
    def _storage_params(self) -> Dict[str, torch.nn.Parameter]:
        return {k: b.storage for k, b in self._buckets.items()}

    @property
    def _storage_info(self):
        return {
            k: {"total": b.total, "partition_size": b.part, "begin": b.begin, "end": b.end,
                "group": b.group, "zero_comm": b.comm, "world_size": b.comm.size, "rank": b.comm.rank}
            for k, b in self._buckets.items()
        }

    def _zero_comm(self, param: DistributedParameter) -> Communicator:
        tp = bool(getattr(param, "_tp_mode", False)) and config["tp_size"] > 1
        if self._mode == "PIPE":
            comm = config["pp_tp_zero_comm"] if tp else config["pp_zero_comm"]
        else:
            comm = config["tp_zero_comm"] if tp else config["zero_comm"]
        return comm if comm is not None else config["zero_comm"]

    # ---------------------------------------------------------------- storage
    def init_param_storage(self) -> None:
        """Lay the inner parameters out in flat buckets and keep only the local partitions."""
        buckets: "OrderedDict[str, _Bucket]" = OrderedDict()
        for name, param in self._module.named_parameters():
            if not isinstance(param, DistributedParameter):
                raise ValueError(f"All parameters in a Block must be DistributedParameter: {name}")
            if param._in_block:
                raise ValueError(f"parameter {name} already belongs to another Block")
            comm = self._zero_comm(param)
            key = _get_param_kw(param)
            if getattr(param, "_tp_mode", False) and config["tp_size"] > 1 and "_g_" not in key:
                key += "_g_tp"
            if key not in buckets:
                buckets[key] = _Bucket(key, param.dtype, param.group, comm)
            b = buckets[key]
            align = max(1, _ALIGN_BYTES // param.element_size())
            offset = round_up(b.total, align)
            numel = param._original_shape.numel()
            slot = _Slot(name, param, offset, numel, param._original_shape)
            b.slots.append(slot)
            b.total = offset + numel
        dev = config["device"]
        for b in buckets.values():
            align = max(1, _ALIGN_BYTES // torch.empty((), dtype=b.dtype).element_size())
            b.part = round_up((b.total + b.comm.size - 1) // b.comm.size, align)
            b.total = b.part * b.comm.size
            requires_grad = any(s.param.requires_grad for s in b.slots)
            b.storage = torch.nn.Parameter(torch.zeros(b.part, dtype=b.dtype, device=dev), requires_grad=requires_grad)
            b.storage._bmt_bucket = b.key
            b.storage._bmt_bounds = (b.begin, b.end)
            b.storage._bmt_comm = b.comm
            for s in b.slots:
                p = s.param
                # current value (even split produced by DistributedParameter) -> overlap with our partition
                full = gather_flat_shard(p.data, s.numel, p._zero_comm)
                s.lo = max(s.offset, b.begin)
                s.hi = min(s.offset + s.numel, b.end)
                if s.hi > s.lo:
                    b.storage.data[s.lo - b.begin:s.hi - b.begin].copy_(full[s.lo - s.offset:s.hi - s.offset])
                else:
                    s.lo = s.hi = max(min(s.offset, b.end), b.begin)
                del full
                p._in_block = True
                p._zero_comm = b.comm
                p._start_partition = s.lo - s.offset
                p._end_partition = s.hi - s.offset
                p._block_owner = _WeakOwner(self)
                p.data = b.storage.data[s.lo - b.begin:s.hi - b.begin]
                self._slots.append(s)
        self._buckets = buckets
        self._slot_of = {id(s.param): (b, s) for b in buckets.values() for s in b.slots}

    def reference(self, block: "Block") -> None:
        """Share another block's parameter storage (weight-tied repetition of the same module)."""
        self._ref_block = block
        self._buckets = block._buckets
        self._slots = block._slots
        self._slot_of = block._slot_of
        self._initialized = True
        self._need_release = False

    def _load_param(self, param: DistributedParameter, value: torch.Tensor) -> None:
        """Write the local part of ``value`` (full tensor of one inner parameter) into the partition."""
        b, s = self._slot_of[id(param)]
        params_changed()
        if s.hi > s.lo:
            flat = value.reshape(-1)
            b.storage.data[s.lo - b.begin:s.hi - b.begin].copy_(flat[s.lo - s.offset:s.hi - s.offset])

    # ------------------------------------------------------ gather / release
    def _begin_gather(self, prefetch: bool = False) -> None:
        """Start the all-gather of every bucket (no-op when resident or already in flight).  ``prefetch``: called on behalf
        of a neighbouring block; a bucket whose optimizer update has not landed yet is then left for later instead of
        making the caller wait."""
        for b in self._buckets.values():
            if b.full is not None and getattr(b, "full_epoch", -1) == _param_epoch[0]:
                continue
            # the optimizer may hold the flat partition or the parameters that are views of it
            holders = [b.storage] + [s.param for s in b.slots]
            if not all([update_ready(h, block=not prefetch) for h in holders]):
                continue
            if b.full is not None and b.work is not None:
                b.work.wait()  # a stale prefetch: let it finish before its buffer is dropped
            b.full = torch.empty(b.total, dtype=b.dtype, device=b.storage.device)
            b.full_epoch = _param_epoch[0]
            b.work = b.comm.all_gather_into(b.full, b.storage.data, async_op=True)

    def _try_deferred_gather(self, args, backward: bool = False) -> bool:
        """ZeRO gather for a block nobody prefetched, when the inner module can pull its first GEMM's weight itself.

        The small parameters (norms, biases) and then the remaining big ones are pushed to all ranks by two kernels on the
        peer stream; the first GEMM's weight is left to the module, whose fused kernel gathers it while multiplying
        (``parallel/fused_ops.zero_gather_gemm``).  Returns False when the conditions are not met.
        """
        import os

        mod = self._module
        name = getattr(mod, "_bmt_first_gemm", None)
        # BMT_FUSED_GATHER: "0" never, "1" whenever possible, "auto" (default): for the recomputation in backward in ZeRO
        # groups of two.  Measured on B200s (benchmark/fused.py): with the device kept busy while the block is enqueued the
        # fused path takes 0.57 ms against 0.64 ms for all-gather + block on 2 GPUs, but 0.78 / 0.83 ms against 0.63 / 0.69 ms
        # on 4 / 8 GPUs (three cross-rank hand-shakes instead of one expose the skew between ranks), and at the cold start
        # of a forward pass its extra host work makes it slower everywhere.
        policy = os.environ.get("BMT_FUSED_GATHER", "auto")
        if name is None or policy == "0" or self._ref_block is not None:
            return False
        if policy == "auto" and not (backward and all(b.comm.size <= 2 for b in self._buckets.values())):
            return False
        if any(b.full is not None for b in self._buckets.values()) or not mod._bmt_can_fuse_first_gemm(*args):
            return False
        target = [(b, s) for b in self._buckets.values() for s in b.slots if s.name == name]
        if not target:
            return False
        b, slot = target[0]
        rt = self._peer_runtime(b)
        if rt is None or len(slot.shape) != 2 or slot.shape[1] % 8 or any(s.numel % 8 for s in b.slots):
            return False
        es = b.storage.element_size()
        key = ("zg", self._slot_parity, b.key, b.total, id(self) if self._mode == "PIPE" else 0)
        first_use = key not in rt.slots
        buf = rt.slot(key, b.total * es)
        free_row, done_a, done_b = rt.row(key + ("free",)), rt.row(key + ("doneA",)), rt.row(key + ("doneB",))
        if first_use:
            rt.signal_wait(free_row, 1, signal=True, wait=False)
        epoch = rt.next_epoch(free_row)
        small, big = [], []
        for s in b.slots:
            lo, hi = max(s.offset, b.begin), min(s.offset + s.numel, b.end)
            if hi <= lo or s is slot:
                continue
            rng = (b.storage.data_ptr() + (lo - b.begin) * es, lo * es, (hi - lo) * es)
            (small if s.numel <= 65536 else big).append(rng)
        if len(small) > 16 or len(big) > 16:
            return False
        cur = torch.cuda.current_stream()
        rt.stream.wait_stream(cur)
        with torch.cuda.stream(rt.stream):
            rt.push_ranges(buf, small, free_row, done_a, epoch, key + ("A",))
            rt.signal_wait(done_a, epoch, signal=False, wait=True)
            ev_small = torch.cuda.Event()
            ev_small.record(rt.stream)
        state = {"ev_rest": None}

        def push_rest(after: Optional[torch.cuda.Event] = None) -> torch.cuda.Event:
            """Start the push of the remaining big parameters on the peer stream (once); ``after``: an event of the
            compute stream the push waits for, so it does not compete for NVLink with the first GEMM's own gather."""
            if state["ev_rest"] is None:
                with torch.cuda.stream(rt.stream):
                    if after is not None:
                        rt.stream.wait_event(after)
                    rt.push_ranges(buf, big, free_row, done_b, epoch, key + ("B",))
                    rt.signal_wait(done_b, epoch, signal=False, wait=True)
                    ev = torch.cuda.Event()
                    ev.record(rt.stream)
                state["ev_rest"] = ev
            return state["ev_rest"]

        b.full = buf.tensor(b.dtype, b.total)
        b.full_epoch = _param_epoch[0]
        b.full_sym = (rt, free_row, epoch)
        mod._bmt_deferred_gather = dict(rt=rt, buf=buf, bucket=b, slot=slot, epoch=epoch, key=key, free_row=free_row,
                                        ev_small=ev_small, push_rest=push_rest)
        return True

    def _ensure_gathered(self, args=None, backward: bool = False) -> None:
        if args is not None:
            for b in self._buckets.values():
                if b.full is None:
                    for h in [b.storage] + [s.param for s in b.slots]:
                        update_ready(h)
            self._try_deferred_gather(args, backward)
        self._begin_gather()
        for b in self._buckets.values():
            if b.work is not None:
                b.work.wait()
                b.work = None
        for b in self._buckets.values():
            for s in b.slots:
                s.param.data = b.full[s.offset:s.offset + s.numel].view(s.shape)
        self._resident = True

    def _point_to_local(self) -> None:
        for b in self._buckets.values():
            for s in b.slots:
                s.param.data = b.storage.data[s.lo - b.begin:s.hi - b.begin]

    def _release_params(self) -> None:
        self._point_to_local()
        for b in self._buckets.values():
            sym = getattr(b, "full_sym", None)
            if sym is not None and b.full is not None:
                # the gathered copy lives in a peer-visible ring slot: tell the peers it may be overwritten by the next gather
                rt, free_row, epoch = sym
                rt.signal_wait(free_row, epoch + 1, signal=True, wait=False)
                b.full_sym = None
            b.full = None
            b.work = None
        if getattr(self._module, "_bmt_deferred_gather", None) is not None:
            self._module._bmt_deferred_gather = None
        self._resident = False

    def _peer_runtime(self, b: _Bucket):
        """NVLink peer-memory runtime for this bucket's ZeRO group, or None (CPU ranks, one rank, fp32, disabled)."""
        if not b.storage.is_cuda or b.comm.size == 1 or b.dtype not in (torch.float16, torch.bfloat16):
            return None
        from .parallel import symm

        return symm.peer_runtime(b.comm)

    def _grad_slot_key(self, b: _Bucket):
        # Blocks of a plain list alternate between two staging slots (a slot is free again once the reduce-scatter of the
        # block after next has been waited for).  Inside a pipeline stage every block keeps its full gradients alive
        # across all micro-batches, so each block needs a slot of its own.
        return ("grad", self._slot_parity, b.key, b.total, id(self) if self._mode == "PIPE" else 0)

    def _prepare_grads(self) -> None:
        """Full-size zeroed gradient buffers; inner ``.grad`` fields become views into them."""
        for b in self._buckets.values():
            needs = [s for s in b.slots if s.param.requires_grad]
            for s in b.slots:
                s.param.grad = None
            if not needs:
                continue
            if b.full_grad is None:
                rt = self._peer_runtime(b)
                if rt is not None:
                    # staging buffer in peer-visible memory; peers must have finished reading its previous contents
                    key = self._grad_slot_key(b)
                    buf = rt.slot(key, b.total * b.storage.element_size(), multicast=True)
                    done_row = rt.row(key + ("done",))
                    if rt.epochs.get(done_row, 0) > 0:
                        rt.signal_wait(done_row, rt.epochs[done_row], signal=False, wait=True)
                    b.full_grad = buf.tensor(b.dtype, b.total).zero_()
                    b.full_grad_buf = buf
                else:
                    b.full_grad = torch.zeros(b.total, dtype=b.dtype, device=b.storage.device)
                    b.full_grad_buf = None
            for s in needs:
                s.param.grad = b.full_grad[s.offset:s.offset + s.numel].view(s.shape)

    def _scatter_grads(self) -> None:
        """Reduce-scatter the full gradient buffers onto the partitions (asynchronously)."""
        for b in self._buckets.values():
            for s in b.slots:
                s.param.grad = None
        self._point_to_local()
        for b in self._buckets.values():
            if b.full_grad is None:
                continue
            full_grad, b.full_grad = b.full_grad, None
            accumulate = b.storage.grad is not None
            rt = self._peer_runtime(b) if getattr(b, "full_grad_buf", None) is not None else None
            if rt is not None:
                # fused path: one kernel on the peer stream reads every rank's staging buffer over NVLink, sums in
                # fp32, adds the gradient accumulated so far, checks inf/nan and writes the partition
                from .parallel.symm import StreamWork

                key = self._grad_slot_key(b)
                piece = b.storage.grad if accumulate else torch.empty(b.part, dtype=b.dtype, device=full_grad.device)
                grad32 = sqsum = None
                if _grad_companions():
                    grad32 = getattr(b, "grad32", None)
                    if accumulate and (grad32 is None or b.grad32_tag != _grad_epoch[0]):
                        # first accumulation of this bucket (or the gradient was rewritten in place since the kernel last
                        # wrote the fp32 copy): start the fp32 copy from what `.grad` holds
                        if grad32 is None:
                            grad32 = b.grad32 = torch.empty(b.part, dtype=torch.float32, device=full_grad.device)
                        grad32.copy_(piece)
                    if getattr(b, "sqsum", None) is None:
                        b.sqsum = torch.zeros(1, dtype=torch.float32, device=full_grad.device)
                        _fused_buckets.add(b)
                    sqsum = b.sqsum
                rt.stream.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(rt.stream):
                    if sqsum is not None:
                        sqsum.zero_()
                    rt.reduce_scatter(b.full_grad_buf, rt.row(key + ("ready",)), b.part, piece, accumulate, acc32=grad32, sqsum=sqsum)
                    if sqsum is not None:
                        b.grad32_tag = b.sq_tag = _grad_epoch[0]
                    done_row = rt.row(key + ("done",))
                    rt.signal_wait(done_row, rt.next_epoch(done_row), signal=True, wait=False)
                    ev = torch.cuda.Event()
                    ev.record(rt.stream)
                work = StreamWork(ev)
                fused = True
            else:
                piece = torch.empty(b.part, dtype=b.dtype, device=full_grad.device)
                work = b.comm.reduce_scatter_into(piece, full_grad, "sum", async_op=True)
                fused = False
            if not accumulate:
                b.storage.grad = piece
            for s in b.slots:
                if s.param.requires_grad:
                    s.param.grad = b.storage.grad[s.lo - b.begin:s.hi - b.begin]

            def finish(work=work, b=b, piece=piece, full_grad=full_grad, accumulate=accumulate, fused=fused):
                work.wait()
                if accumulate and not fused:
                    b.storage.grad.add_(piece)

            if work is DONE:
                finish()
            else:
                _pending.append(finish)
                _queue_backward_callback()
            # let an offloading optimizer start moving this partition's gradient to the host right away
            for holder in [b.storage] + [s.param for s in b.slots]:
                hook = getattr(holder, "_bmt_grad_hook", None)
                if hook is not None and holder.grad is not None and holder.numel() > 0:
                    hook(holder, None if accumulate else work)

    # ------------------------------------------------------------- scheduling
    def _enter_forward(self, args=None) -> None:
        self._ensure_gathered(args)
        nxt = self.next_module()
        if nxt is not None and nxt._mode != "PIPE":
            nxt._begin_gather(prefetch=True)

    def _exit_forward(self) -> None:
        if self._mode == "PIPE" and self._micro_idx != config["micros"] - 1:
            return  # later micro-batches reuse the gathered parameters
        if self._zero_level == 2 and self._grad_mode:
            # ZeRO-2: keep the gathered buffers for backward, show the shards meanwhile
            self._point_to_local()
            self._resident = False
        else:
            self._release_params()

    def _enter_backward(self, args=None) -> None:
        self._ensure_gathered(args, backward=True)
        self._prepare_grads()
        pre = self.pre_module()
        if pre is not None and pre._mode != "PIPE" and pre._zero_level == 3:
            pre._begin_gather(prefetch=True)

    def _exit_backward(self) -> None:
        if self._mode == "PIPE":
            last = self._micro_idx == 0
            self._micro_idx -= 1
            if not last:
                return  # gradients keep accumulating in the full buffers until micro-batch 0
        self._scatter_grads()
        self._release_params()

    # ------------------------------------------------------------------ links
    def set_pre_module(self, pre_module) -> None:
        if pre_module is not None:
            self._pre_module = pre_module
            pre_module._next_module = self

    def pre_module(self):
        return self._pre_module if not self._is_first_layer else None

    def next_module(self):
        return self._next_module if not self._is_last_layer else None

    # ---------------------------------------------------------------- forward
    def forward(self, *args, **kwargs):
        if kwargs:
            bound = inspect.signature(self._module.forward).bind(*args, **kwargs)
            bound.apply_defaults()
            args = bound.args
        grad_on = torch.is_grad_enabled()
        tensors, arg_spec = [], []
        for a in args:
            if isinstance(a, torch.Tensor):
                arg_spec.append(len(tensors))
                tensors.append(a)
            else:
                arg_spec.append(("const", a))
        self.all_input_no_grad = not any(t.requires_grad for t in tensors)
        self.all_param_no_grad = not any(s.param.requires_grad for s in self._slots)
        self._grad_mode = grad_on and not (self.all_input_no_grad and self.all_param_no_grad)

        if not self._grad_mode:
            # nothing to differentiate: gather, run once, release
            self._enter_forward()
            try:
                out = self._module(*args)
            finally:
                self._exit_forward()
            return out

        placeholder = torch.empty(0, requires_grad=True) if self.all_input_no_grad else None
        flat = _BlockFunction.apply(self, placeholder, arg_spec, *tensors)
        return _rebuild_out(list(flat), self._last_out_spec)

    # ------------------------------------------------ transparency of the wrapper
    def __getattr__(self, name: str):
        if name == "_module":
            return object.__getattribute__(self, "_module")
        return getattr(object.__getattribute__(self, "_module"), name)

    def __setattr__(self, name, value):
        object.__setattr__(self, name, value)

    def __getattribute__(self, name: str):
        if name == "_parameters":
            return object.__getattribute__(self, "_module")._parameters
        return super().__getattribute__(name)

    def __delattr__(self, name):
        object.__delattr__(self, name)

    def _named_members(self, get_members_fn, prefix="", recurse=True, **kwargs):
        kwargs.setdefault("remove_duplicate", True)
        return self._module._named_members(get_members_fn, prefix, recurse, **kwargs)

    def named_modules(self, memo=None, prefix: str = "", remove_duplicate: bool = True):
        if memo is None:
            memo = set()
        if self not in memo:
            if remove_duplicate:
                memo.add(self)
            yield prefix, self
            for name, module in self._module._modules.items():
                if module is None:
                    continue
                sub_prefix = prefix + ("." if prefix else "") + name
                yield from module.named_modules(memo, sub_prefix, remove_duplicate)

    def named_children(self):
        return self._module.named_children()

    def train(self, mode: bool = True):
        self._module.train(mode)
        return self

    def eval(self):
        self._module.eval()
        return self

    def __repr__(self):
        return self._module.__repr__()

    # -------------------------------------------------------------- state dict
    def state_dict(self, *args, destination=None, prefix="", keep_vars=False):
        """Full (gathered, tensor-parallel shards joined) values keyed like the inner module's state dict."""
        if args:  # positional legacy form: (destination, prefix, keep_vars)
            destination = args[0] if len(args) > 0 else destination
            prefix = args[1] if len(args) > 1 else prefix
            keep_vars = args[2] if len(args) > 2 else keep_vars
        if destination is None:
            destination = OrderedDict()
            destination._metadata = OrderedDict()
        self._save_to_state_dict(destination, prefix, keep_vars)
        return destination

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        was_resident = self._resident
        with torch.no_grad():
            self._ensure_gathered()
            try:
                for mod_prefix, mod in self._module.named_modules(prefix=prefix[:-1] if prefix.endswith(".") else prefix):
                    p = (mod_prefix + ".") if mod_prefix else ""
                    for name, param in mod._parameters.items():
                        if param is None:
                            continue
                        if isinstance(param, DistributedParameter):
                            full = param.tp_gather(param.data).detach()
                            destination[p + name] = full.cpu() if config["save_param_to_cpu"] else full.clone()
                        else:  # pragma: no cover - blocks only hold distributed parameters
                            destination[p + name] = param.detach()
                    for name, buf in mod._buffers.items():
                        if buf is not None and name not in mod._non_persistent_buffers_set:
                            destination[p + name] = buf if keep_vars else buf.detach()
            finally:
                if not was_resident:
                    self._release_params()

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict,
                              missing_keys, unexpected_keys, error_msgs):
        from .store import DistributedTensorWrapper

        known = set()
        for mod_prefix, mod in self._module.named_modules(prefix=prefix[:-1] if prefix.endswith(".") else prefix):
            p = (mod_prefix + ".") if mod_prefix else ""
            items = [(n, v, True) for n, v in mod._parameters.items() if v is not None]
            items += [(n, v, False) for n, v in mod._buffers.items()
                      if v is not None and n not in mod._non_persistent_buffers_set]
            for name, target, is_param in items:
                key = p + name
                known.add(key)
                if key not in state_dict:
                    if strict:
                        missing_keys.append(key)
                    continue
                value = state_dict[key]
                expect = target._tp_original_shape if isinstance(target, DistributedParameter) else target.shape
                if tuple(value.shape) != tuple(expect):
                    error_msgs.append(
                        f"size mismatch for {key}: copying a param with shape {tuple(value.shape)} from checkpoint, "
                        f"the shape in current model is {tuple(expect)}."
                    )
                    continue
                if isinstance(value, DistributedTensorWrapper):
                    value = value.broadcast()
                with torch.no_grad():
                    if isinstance(target, DistributedParameter):
                        if target._tp_mode and target._tp_split_dim >= 0:
                            value = tp_split_tensor(value, target._tp_split_dim)
                        self._load_param(target, value.to(target.dtype))
                    else:
                        target.copy_(value)
        if strict:
            for key in state_dict.keys():
                if key.startswith(prefix) and key not in known:
                    unexpected_keys.append(key)

    # ------------------------------------------------------------------- init
    def grouped_parameters(self):
        """``(group, [flat partition parameters])`` pairs of this block."""
        ret: Dict[Optional[str], List[torch.nn.Parameter]] = {}
        if self._ref_block is not None:
            return
        for b in self._buckets.values():
            ret.setdefault(b.group, []).append(b.storage)
        yield from ret.items()

    def init_parameters(self) -> None:
        """Run every parameter's ``init_method`` on a full-size temporary and keep the local part.

        Every rank draws the same full tensor (same seed), so the values match a
        single-process initialisation exactly (reference ``bmtrain/block_layer.py:515-558``).
        """
        if self._ref_block is not None:
            return
        dev = config["device"]
        for b in self._buckets.values():
            for s in b.slots:
                p = s.param
                if p._init_method is None:
                    continue
                tmp = torch.empty(p._tp_original_shape, dtype=p.dtype, device=dev)
                p._init_method(tmp)
                if p._tp_mode and p._tp_split_dim >= 0:
                    tmp = tp_split_tensor(tmp, p._tp_split_dim)
                self._load_param(p, tmp)
                del tmp


class _WeakOwner:
    """Callable back-reference parameter -> owning block that does not register as a submodule."""

    def __init__(self, block: Block):
        import weakref

        self._ref = weakref.ref(block)

    def __call__(self) -> Block:
        return self._ref()


def _block_wrapper(module, module_dict: dict, mode: str = "BLOCK") -> Block:
    """Entry of a block list as a :class:`Block`.  ``module_dict`` maps ``id(inner module)`` to the block that already
    owns it: a raw module listed twice becomes a weight-tied block sharing the first one's storage, while the same
    ``Block`` object (or two blocks around one module) in a list is an error."""
    if isinstance(module, Block):
        inner = module._module
        if mode == "PIPE" and module._mode != "PIPE":
            raise AssertionError('a Block inside a PipelineTransformerBlockList must be created with mode="PIPE"')
        if id(inner) in module_dict:
            raise AssertionError("the same bmt.Block appears twice in one block list")
        module_dict[id(inner)] = module
        return module
    owner = module_dict.get(id(module))
    if owner is not None:
        return Block(module, initialized=True, mode=mode, _share=owner)
    module_dict[id(module)] = block = Block(module, mode=mode)
    return block


class TransformerBlockList(torch.nn.Module):
    """A list of blocks that is called as a whole: ``out = blocks(hidden, *other_args)``.

    The first ``num_hidden`` outputs of each block replace the first
    ``num_hidden`` inputs of the next one; the remaining arguments are passed
    to every block unchanged.  Neighbouring blocks are linked, so each block
    starts the gather of the block that runs after it (the next one in
    forward, the previous one in backward) before it computes, and a block's
    gradient reduction runs under the backward pass of the blocks before it.
    Contract: reference ``bmtrain/block_layer.py:651-726``.
    """

    _modules: Dict[str, Block]

    def __init__(self, modules: Iterable[Block], num_hidden: int = 1) -> None:
        super().__init__()
        owners: dict = {}
        chain: List[Block] = [_block_wrapper(m, owners) for m in modules]
        for i, block in enumerate(chain):
            block.set_pre_module(chain[i - 1] if i else None)
            block._is_first_layer = i == 0
            block._is_last_layer = i == len(chain) - 1
            block._slot_parity = i % 2  # neighbouring blocks alternate between two peer-visible gradient staging slots
            self.add_module(str(i), block)
        self.num_hidden = num_hidden

    def __len__(self) -> int:
        return len(self._modules)

    def __iter__(self) -> Iterator[Block]:
        return iter(self._modules.values())

    def __getitem__(self, index: Union[int, str]) -> Block:
        if isinstance(index, int) and index < 0:
            index += len(self)
        return self._modules[str(index)]

    def forward(self, *args, return_hidden_states: bool = False):
        self.return_hidden_states = return_hidden_states
        k = self.num_hidden
        carried, shared = tuple(args[:k]), tuple(args[k:])
        seen: List[List[torch.Tensor]] = [[] for _ in range(k)]  # inputs of every block, per carried position
        produced: Tuple = ()
        for block in self._modules.values():
            if return_hidden_states:
                for trail, value in zip(seen, carried):
                    trail.append(value)
            produced = block(*carried, *shared)
            if not isinstance(produced, tuple):
                produced = (produced,)
            carried = produced[:k]
        if return_hidden_states:
            return produced + tuple(torch.stack(trail, dim=0) for trail in seen)
        return produced[0] if k == 1 else tuple(produced[:k])
