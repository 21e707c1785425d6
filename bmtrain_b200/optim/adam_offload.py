"""Adam with the optimizer state in host memory (reference: ``bmtrain/optim/adam_offload.py:13-386``).

fp32 master weights and both moments live in pinned host DRAM.  A step is a
three-stage software pipeline over fixed-size chunks of every shard:

    D2H copy of the half gradient (copy stream 1)
      -> AVX-512 Adam on a persistent host thread pool
        -> H2D copy of the updated half parameter (copy stream 2)

so PCIe traffic in both directions overlaps the host math.  The pipeline runs on
a worker thread of the native library (``csrc/runtime.cu``): ``step`` queues the
work in the order in which the next forward pass needs the parameters and
returns; whoever gathers a parameter first waits for the batch that updates it
(``_bmt_pending_update``), so the next step's forward pass runs under the tail of
this step's optimizer.  When the loss scale of the coming step is known
(``OptimManager.backward`` announces it), parameters whose gradients are
complete are already stepped *during backward* into a second set of state
arrays; ``step`` adopts those results if no overflow was found and nothing else
changed, and drops them otherwise, so a skipped step leaves the state bit for
bit as it was.  State-dict layout (``state``/``param_groups``/``is_whole``) and
the ``gather`` option follow the reference, so checkpoints resume
bit-identically.
"""
from __future__ import annotations

import ctypes
import math
import weakref
from collections import defaultdict
from copy import deepcopy
from itertools import chain

import torch

from ..ops import adam as _adam
from ._distributed import state_dict_gather
from .adam import _partition_bounds, _zero_grad

_CHUNK = 1 << 23  # elements per pipeline stage (16 MiB of half data)
_live = weakref.WeakSet()  # optimizers that may have asynchronous batches queued


def finish_all_updates() -> None:
    """Wait for every offloading optimizer's queued batches (``bmt.synchronize`` calls this)."""
    for opt in list(_live):
        opt.synchronize()


class _OffloadJob(ctypes.Structure):
    """Mirror of ``BmtOffloadJob`` (``csrc/api.h``)."""

    _fields_ = [("grad_ready", ctypes.c_void_p), ("p32", ctypes.c_void_p), ("m", ctypes.c_void_p), ("v", ctypes.c_void_p),
                ("p32_out", ctypes.c_void_p), ("m_out", ctypes.c_void_p), ("v_out", ctypes.c_void_p),
                ("p16_host", ctypes.c_void_p), ("g16_host", ctypes.c_void_p), ("p_dev", ctypes.c_void_p),
                ("n", ctypes.c_int64), ("beta1", ctypes.c_float), ("beta2", ctypes.c_float), ("eps", ctypes.c_float),
                ("lr", ctypes.c_float), ("scale", ctypes.c_float), ("wd", ctypes.c_float), ("bc1", ctypes.c_float),
                ("bc2", ctypes.c_float), ("bf16", ctypes.c_int), ("upload", ctypes.c_int)]


_STATE_KEYS = ("_param_fp32", "exp_avg", "exp_avg_sq")


def _pinned(shape, dtype, pin):
    t = torch.empty(shape, dtype=dtype, device="cpu")
    if pin:
        try:
            t = t.pin_memory()
        except RuntimeError:  # pragma: no cover - no CUDA runtime
            pass
    return t


class AdamOffloadOptimizer(torch.optim.Optimizer):
    """Adam whose fp32 state and math live on the host; the device only holds half parameters and gradients."""

    _bmtrain_optimizer = True

    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0, hold_steps=0, record_delta=False,
                 math: str = "cpu"):
        if not 0.0 <= lr:
            raise ValueError(f"Invalid learning rate: {lr}")
        if not 0.0 <= eps:
            raise ValueError(f"Invalid epsilon value: {eps}")
        if not 0.0 <= betas[0] < 1.0:
            raise ValueError(f"Invalid beta parameter at index 0: {betas[0]}")
        if not 0.0 <= betas[1] < 1.0:
            raise ValueError(f"Invalid beta parameter at index 1: {betas[1]}")
        if not 0.0 <= weight_decay:
            raise ValueError(f"Invalid weight_decay value: {weight_decay}")
        self.avg_delta = 0
        self.var_delta = 0
        super().__init__(params, dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self._hold_steps = hold_steps
        self.record_delta = record_delta
        # where the arithmetic runs: "cpu" (AVX-512 thread pool; default), "gpu" (state chunks streamed host -> HBM -> host
        # with cudaMemcpyAsync on side streams, Adam kernel on the device) or "auto" (both engines at once, split by their
        # measured rates).  All three keep the fp32 state in host memory and are bound by how fast that memory can be
        # streamed: on the 16-vCPU single-GPU host the device path is PCIe-bound and slower than the host path, on the
        # 8-GPU host the three are within 5 % of each other.
        import os as _os

        self._math = _os.environ.get("BMT_OFFLOAD_MATH", math)
        self._gpu_pipe = None
        # "auto" splits every step between the two engines: the first `_gpu_fraction` of the elements take the streamed
        # device path (PCIe-bound), the rest the host path (host-memory-bound), both at the same time; the split follows
        # the measured rates for the first steps and is then frozen
        self._gpu_fraction = float(_os.environ.get("BMT_OFFLOAD_GPU_FRACTION", "0.4"))
        self._tune_steps = 0
        self._last_timing = None
        self._d2h = self._h2d = None
        self._ahead_owners = []  # parameters that own a second set of state arrays
        self._staged = {}  # param -> event of a gradient copy that was started during backward
        # asynchronous pipeline: tickets of queued batches per parameter, results computed ahead of `step`, and what the
        # coming step will be called with (announced by OptimManager.backward; None = unknown, nothing is computed ahead)
        self._async = _os.environ.get("BMT_OFFLOAD_ASYNC", "1") != "0"
        self._ahead_budget = int(float(_os.environ.get("BMT_OFFLOAD_AHEAD_GB", "4")) * (1 << 30))
        self._tickets = {}   # param -> [ticket, ...]
        self._keep = {}      # ticket -> objects whose raw handles the queued batch uses
        self._ahead = {}     # param -> dict(ticket=, key=hyper-parameters the result was computed with)
        self._announced_scale = None
        self.stats = {"ahead_queued": 0, "ahead_adopted": 0, "ahead_requeued": 0, "ahead_dropped": 0}
        _live.add(self)
        for group in self.param_groups:
            for p in group["params"]:
                if (p.is_cuda and not self._use_gpu_math(p)   # chunks that may switch engines are staged at step time
                        and (getattr(p, "_bmt_bucket", None) is not None or getattr(p, "_in_block", False))):
                    p._bmt_grad_hook = self._on_grad_ready
        if record_delta:
            for group in self.param_groups:
                for p in group["params"]:
                    p._delta_info = torch.zeros(4, dtype=torch.float32)

    def _use_gpu_math(self, p) -> bool:
        """Whether the parameter may take the device path at all (the per-step split decides how much of it does)."""
        if not p.is_cuda or p.dtype == torch.float32 or self.record_delta:
            return False
        return self._math in ("gpu", "auto")

    def _retune(self) -> None:
        """Move the split towards equal finishing times of the two engines (first 16 steps only)."""
        if self._math != "auto" or self._last_timing is None or self._tune_steps >= 16:
            return
        ev0, ev1, n_gpu, t_cpu, n_cpu = self._last_timing
        self._last_timing = None
        if n_gpu == 0 or n_cpu == 0:
            return
        ev1.synchronize()
        t_gpu = ev0.elapsed_time(ev1) / 1e3
        if t_gpu <= 0 or t_cpu <= 0:
            return
        r_gpu, r_cpu = n_gpu / t_gpu, n_cpu / t_cpu
        self._gpu_fraction = min(0.95, max(0.05, 0.5 * self._gpu_fraction + 0.5 * r_gpu / (r_gpu + r_cpu)))
        self._tune_steps += 1

    # ------------------------------------------------------- GPU-streamed step
    def _gpu_streamed_step(self, items, scale, ev_begin=None, ev_end=None) -> None:
        """Adam on the device with the state streamed through: for every chunk, (master, m, v) travel host -> HBM on the
        upload stream, the multi-tensor Adam kernel updates them together with the half parameter in place (the gradient
        never leaves the device), and the three arrays travel back on the download stream.  Three staging slots keep the
        two copy engines and the kernel busy at the same time; nothing here blocks the host."""
        if self._gpu_pipe is None:
            dev = items[0][0].device
            n = _CHUNK
            self._gpu_pipe = {
                "up": torch.cuda.Stream(), "down": torch.cuda.Stream(), "math": torch.cuda.Stream(),
                "slots": [tuple(torch.empty(n, dtype=torch.float32, device=dev) for _ in range(3)) for _ in range(3)],
                "free": [None, None, None], "turn": 0, "host_done": {},
            }
        pipe = self._gpu_pipe
        up, down, math_s = pipe["up"], pipe["down"], pipe["math"]
        cur = torch.cuda.current_stream()
        math_s.wait_stream(cur)   # gradients are final, the previous step's parameter readers are done
        up.wait_stream(cur)
        if ev_begin is not None:
            ev_begin.record(up)
        for p, state, group, lo, hi in items:
            n = hi - lo
            if n == 0:
                continue
            k = pipe["turn"] % 3
            pipe["turn"] += 1
            slot = pipe["slots"][k]
            host = [state["_param_fp32"].view(-1)[lo:hi], state["exp_avg"].view(-1)[lo:hi], state["exp_avg_sq"].view(-1)[lo:hi]]
            key = (id(p), lo)
            with torch.cuda.stream(up):
                if pipe["free"][k] is not None:
                    up.wait_event(pipe["free"][k])          # the slot's previous contents have been written back
                if key in pipe["host_done"]:
                    up.wait_event(pipe["host_done"][key])   # last step's write-back of this chunk has landed in host memory
                for d, h in zip(slot, host):
                    d[:n].copy_(h, non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(up)
            beta1, beta2 = group["betas"]
            lr = 0.0 if state["step"] < self._hold_steps else group["lr"]
            with torch.cuda.stream(math_s):
                math_s.wait_event(ev_in)
                grad = p.grad.reshape(-1)[lo:hi]
                if group.get("maximize", False):
                    grad = -grad
                _adam.adam_half_multi([(slot[0][:n], p.data.view(-1)[lo:hi], grad.contiguous(), slot[1][:n], slot[2][:n])],
                                      beta1, beta2, group["eps"], lr, scale, group["weight_decay"], state["step"])
                ev_math = torch.cuda.Event()
                ev_math.record(math_s)
            with torch.cuda.stream(down):
                down.wait_event(ev_math)
                for d, h in zip(slot, host):
                    h.copy_(d[:n], non_blocking=True)
                ev_out = torch.cuda.Event()
                ev_out.record(down)
            pipe["free"][k] = ev_out
            pipe["host_done"][key] = ev_out
        if ev_end is not None:
            ev_end.record(down)
        cur.wait_stream(math_s)   # later kernels see the updated parameters

    def _host_state_ready(self) -> None:
        """Block until queued updates and every write-back of the streamed step have reached host memory (before the
        host reads the state)."""
        self._drop_ahead()
        self.synchronize()
        if self._gpu_pipe is not None:
            self._gpu_pipe["down"].synchronize()

    # ------------------------------------------------------------ host memory
    def host_bytes(self) -> int:
        """Host memory this rank's optimizer needs: fp32 master, two moments, and the half-precision staging copies of
        gradient and parameter (16 bytes per half-precision parameter element, 16 per fp32 one)."""
        total = 0
        for group in self.param_groups:
            for p in group["params"]:
                if p.requires_grad:
                    total += p.numel() * (12 + (4 if p.dtype == torch.float32 else 4))
        return total

    def _check_host_memory(self) -> None:
        """Before the first allocation: refuse with a clear message when the host cannot hold the state of all ranks of
        this machine (page-locking more memory than there is takes the machine down long before an allocation fails)."""
        from ..global_var import config

        if getattr(self, "_host_checked", False):
            return
        self._host_checked = True
        try:
            with open("/proc/meminfo") as f:
                info = dict(line.split(":", 1) for line in f)
            avail = int(info["MemAvailable"].split()[0]) * 1024
        except (OSError, KeyError, ValueError):
            return
        need = self.host_bytes() * max(1, int(config.get("local_size", 1) or 1))
        if need > 0.9 * avail:
            raise MemoryError(
                f"AdamOffloadOptimizer needs about {need / 2 ** 30:.0f} GiB of host memory on this machine "
                f"({self.host_bytes() / 2 ** 30:.1f} GiB per rank x {config.get('local_size', 1)} ranks) but only "
                f"{avail / 2 ** 30:.0f} GiB are available; use more machines, a smaller model, or AdamOptimizer")

    # ------------------------------------------------------------------ state
    def _init_state(self, p):
        self._check_host_memory()
        state = self.state[p]
        pin = p.is_cuda
        state["step"] = 0
        state["exp_avg"] = _pinned(p.size(), torch.float32, pin).zero_()
        state["exp_avg_sq"] = _pinned(p.size(), torch.float32, pin).zero_()
        state["_param_fp32"] = _pinned(p.size(), torch.float32, pin)
        state["_param_fp32"].copy_(p.detach())
        self._make_staging(p, state)
        return state

    @staticmethod
    def _make_staging(p, state):
        pin = p.is_cuda
        if p.dtype == torch.float32:
            state["_grad_fp32"] = _pinned(p.size(), torch.float32, pin)
        else:
            state["_param_fp16"] = _pinned(p.size(), p.dtype, pin)
            state["_grad_fp16"] = _pinned(p.size(), p.dtype, pin)

    def _streams(self):
        if self._d2h is None:
            self._d2h = torch.cuda.Stream()
            self._h2d = torch.cuda.Stream()
        return self._d2h, self._h2d

    # -------------------------------------------------- early gradient staging
    def _on_grad_ready(self, p, work) -> None:
        """Called by the owning block when the reduce-scatter of ``p.grad`` has been issued (``work``), or with
        ``None`` when an earlier staged copy became stale (gradient accumulation)."""
        if work is None:
            self._staged.pop(p, None)
            self._drop_ahead(p)
            return
        state = self.state.get(p)
        if not state or p.dtype == torch.float32 or p.grad is None:
            return  # first step: host buffers do not exist yet
        d2h, _ = self._streams()
        from ..comm import DONE

        if work is DONE:
            d2h.wait_stream(torch.cuda.current_stream())
        else:
            with torch.cuda.stream(d2h):
                work.wait()
        with torch.cuda.stream(d2h):
            state["_grad_fp16"].view(-1).copy_(p.grad.reshape(-1), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(d2h)
        p.grad.record_stream(d2h)   # the copy may outlive this call: the gradient's memory must not be reused before it ran
        self._staged[p] = ev
        self._step_ahead(p, state, ev)

    def _invalidate_staged(self) -> None:
        """Gradients were modified after backward (clipping): copies made during backward, and anything computed from
        them, are stale."""
        self._drop_ahead()
        self._staged.clear()

    # ------------------------------------------------------ asynchronous plumbing
    def _lib(self):
        from ..ops import _native

        lib = _native.cuda_lib()
        if not getattr(lib, "_bmt_offload_typed", False):
            lib.bmt_offload_submit.restype = ctypes.c_int64
            lib.bmt_offload_submit_uploads.restype = ctypes.c_int64
            lib.bmt_offload_wait.argtypes = [ctypes.c_int64, ctypes.c_void_p]
            lib.bmt_offload_poll.argtypes = [ctypes.c_int64]
            lib.bmt_offload_cancel.argtypes = [ctypes.c_int64]
            lib._bmt_offload_typed = True
        return lib

    def _pending_update(self, p, block: bool) -> bool:
        """Hook installed on a parameter while batches that rewrite it are queued.  ``block`` false: only report whether
        they are done.  Otherwise wait for them and make the current stream wait for their uploads; returns True."""
        tickets = self._tickets.get(p)
        if tickets:
            lib = self._lib()
            if not block and not all(lib.bmt_offload_poll(t) for t in tickets):
                return False
            stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
            for t in tickets:
                rc = lib.bmt_offload_wait(t, stream)
                self._keep.pop(t, None)
                if rc != 0:
                    raise RuntimeError(f"offloaded Adam batch failed (stage {rc >> 16}, CUDA error {rc & 0xffff})")
            del self._tickets[p]
        if getattr(p, "_bmt_pending_update", None) is not None:
            p._bmt_pending_update = None
        return True

    def _track(self, p, ticket: int, keep=None) -> None:
        """Remember a queued batch of ``p``.  ``keep``: objects the worker uses by raw handle (the events guarding the
        gradient copies); they must outlive the batch, so they are held until it has been waited for."""
        if ticket <= 0:
            raise RuntimeError(f"could not queue an offloaded Adam batch (code {ticket})")
        self._tickets.setdefault(p, []).append(ticket)
        if keep:
            self._keep[ticket] = keep
        p._bmt_pending_update = lambda block=True, p=p: self._pending_update(p, block)

    def synchronize(self) -> None:
        """Block until every queued update has been applied and uploaded (host state and device parameters final)."""
        for p in list(self._tickets):
            self._pending_update(p, True)
        if self._h2d is not None:
            self._h2d.synchronize()

    def _hyper(self, p, state, group, scale):
        """Everything a result computed ahead of ``step`` depends on besides the gradient and the old state."""
        step = state["step"] + 1
        lr = 0.0 if step < self._hold_steps else group["lr"]
        return (float(scale), step, float(lr), tuple(group["betas"]), float(group["eps"]), float(group["weight_decay"]),
                bool(group.get("maximize", False)))

    def _jobs_for(self, p, state, group, scale, step, pieces, out_state=None, upload=True):
        """ctypes job array for the ranges ``pieces`` = [(lo, hi, event)] of one half-precision device parameter."""
        arr = (_OffloadJob * len(pieces))()
        beta1, beta2 = group["betas"]
        out_state = out_state if out_state is not None else state
        for c, (lo, hi, ev) in zip(arr, pieces):
            c.grad_ready = ev.cuda_event if ev is not None else None
            for dst, key in (("p32", "_param_fp32"), ("m", "exp_avg"), ("v", "exp_avg_sq")):
                setattr(c, dst, state[key].data_ptr() + lo * 4)
                setattr(c, dst + "_out", out_state[key].data_ptr() + lo * 4)
            c.p16_host = state["_param_fp16"].data_ptr() + lo * 2
            c.g16_host = state["_grad_fp16"].data_ptr() + lo * 2
            c.p_dev = p.data.data_ptr() + lo * 2
            c.n = hi - lo
            c.beta1, c.beta2, c.eps = beta1, beta2, group["eps"]
            c.lr = 0.0 if step < self._hold_steps else group["lr"]
            c.scale, c.wd = scale, group["weight_decay"]
            c.bc1, c.bc2 = 1.0 - math.pow(beta1, step), 1.0 - math.pow(beta2, step)
            c.bf16 = 1 if p.dtype == torch.bfloat16 else 0
            c.upload = 1 if upload else 0
        return arr

    def _cpu_fn(self):
        from ..ops import _native

        cpu_lib = _native.cpu_lib()
        return None if cpu_lib is None else ctypes.cast(cpu_lib.bmt_adam_cpu_ex, ctypes.c_void_p)

    # ------------------------------------------------ stepping ahead, during backward
    def _expect_step(self, scale) -> None:
        """The coming ``step`` will be called with this loss scale (``OptimManager.backward``)."""
        self._announced_scale = scale

    def _step_ahead(self, p, state, event) -> None:
        """Queue the update of ``p`` now, into a second set of state arrays, from the gradient copy ``event`` guards."""
        if (not self._async or self._announced_scale is None or self._math != "cpu" or self.record_delta
                or p in self._ahead or p.dtype == torch.float32):
            return
        fn = self._cpu_fn()
        if fn is None:
            return
        group = next(g for g in self.param_groups if any(q is p for q in g["params"]))
        if group.get("maximize", False):
            return
        need = 3 * 4 * p.numel()
        if "_ahead_state" not in state:
            used = sum(3 * 4 * q.numel() for q in self._ahead_owners)
            if used + need > self._ahead_budget:
                return
            # touched here, once: the first write to fresh pages would otherwise cost page faults inside a later step
            state["_ahead_state"] = {k: torch.empty_like(state[k], pin_memory=False).fill_(0.0) for k in _STATE_KEYS}
            self._ahead_owners.append(p)
        key = self._hyper(p, state, group, self._announced_scale)
        n = p.numel()
        pieces = [(lo, min(n, lo + _CHUNK), event if lo == 0 else None) for lo in range(0, n, _CHUNK)]
        jobs = self._jobs_for(p, state, group, key[0], key[1], pieces, out_state=state["_ahead_state"], upload=False)
        _, h2d = self._streams()
        ticket = self._lib().bmt_offload_submit(jobs, ctypes.c_int(len(pieces)), fn, ctypes.c_void_p(h2d.cuda_stream))
        if ticket > 0:
            self._ahead[p] = dict(ticket=ticket, key=key, event=event)
            self.stats["ahead_queued"] += 1

    def _drop_ahead(self, p=None) -> None:
        """Forget results computed ahead (all, or those of ``p``); a batch that is running is waited for first."""
        lib = None
        for q in ([p] if p is not None else list(self._ahead)):
            rec = self._ahead.pop(q, None)
            if rec is None:
                continue
            lib = lib or self._lib()
            self.stats["ahead_dropped"] += 1
            if not lib.bmt_offload_cancel(rec["ticket"]):
                lib.bmt_offload_wait(rec["ticket"], None)

    def _adopt_ahead(self, p, state, group, scale) -> bool:
        """Make the result computed ahead for ``p`` the current state if it was computed with exactly the arguments this
        step has, and queue its upload.  False: there is none (or it was dropped) and ``p`` has to be stepped now."""
        rec = self._ahead.pop(p, None)
        if rec is None:
            return False
        lib = self._lib()
        if lib.bmt_offload_cancel(rec["ticket"]):
            self.stats["ahead_requeued"] += 1
            return False          # it had not been started: it takes its turn in forward order instead
        if rec["key"] != self._hyper(p, state, group, scale):
            self.stats["ahead_dropped"] += 1
            lib.bmt_offload_wait(rec["ticket"], None)
            return False
        rc = lib.bmt_offload_wait(rec["ticket"], None)
        if rc != 0:
            raise RuntimeError(f"offloaded Adam batch failed (stage {rc >> 16}, CUDA error {rc & 0xffff})")
        other = state["_ahead_state"]
        for k in _STATE_KEYS:
            state[k], other[k] = other[k], state[k]
        state["step"] += 1
        self.stats["ahead_adopted"] += 1
        n = p.numel()
        jobs = self._jobs_for(p, state, group, scale, state["step"], [(0, n, None)])
        _, h2d = self._streams()
        self._track(p, lib.bmt_offload_submit_uploads(jobs, ctypes.c_int(1), ctypes.c_void_p(h2d.cuda_stream)))
        return True

    # ------------------------------------------------------------------- step
    @torch.no_grad()
    def step(self, closure=None, scale=1):
        from ..block_layer import params_changed

        params_changed()
        self.synchronize()   # batches of the previous step (long finished in a training loop)
        self._announced_scale = None
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()

        work = []  # (param, state, group, lo, hi, event)
        stepped = set()  # parameters whose step counter was already advanced
        gpu_items = []  # (param, state, group, lo, hi) for the device-side streamed path
        on_gpu = False
        for group in self.param_groups:
            for p in group["params"]:
                if p.grad is None or not p.requires_grad:
                    continue
                if p.grad.is_sparse:
                    raise RuntimeError("Adam does not support sparse gradients, please consider SparseAdam instead")
                if p.dtype not in (torch.float32, torch.float16, torch.bfloat16):
                    raise RuntimeError("Adam only supports fp32, fp16 and bf16 gradients")
                state = self.state[p]
                if len(state) == 0:
                    state = self._init_state(p)
                n = p.numel()
                if p in self._ahead and self._adopt_ahead(p, state, group, scale):
                    continue
                if self._use_gpu_math(p) and n > 0:
                    for lo in range(0, n, _CHUNK):
                        gpu_items.append((p, state, group, lo, min(n, lo + _CHUNK)))
                    continue
                on_gpu = on_gpu or p.is_cuda
                if p.dtype == torch.float32 or n == 0:
                    work.append((p, state, group, 0, n, None))
                else:
                    for lo in range(0, n, _CHUNK):
                        work.append((p, state, group, lo, min(n, lo + _CHUNK), None))

        n_gpu = n_cpu_moved = 0
        if gpu_items:
            self._retune()
            total = sum(hi - lo for _, _, _, lo, hi in gpu_items)
            budget = total if self._math == "gpu" else int(total * self._gpu_fraction)
            stepped_gpu = set()
            keep = []
            for it in gpu_items:
                p, state, group, lo, hi = it
                if id(p) not in stepped_gpu:
                    stepped_gpu.add(id(p))
                    state["step"] += 1
                if n_gpu + (hi - lo) <= budget or self._math == "gpu":
                    keep.append(it)
                    n_gpu += hi - lo
                else:
                    # host engine takes this chunk; its last device-side write-back must have landed first
                    pipe = self._gpu_pipe
                    if pipe is not None and (id(p), lo) in pipe["host_done"]:
                        pipe["host_done"].pop((id(p), lo)).synchronize()
                    work.append((p, state, group, lo, hi, "stepped"))
                    n_cpu_moved += hi - lo
                    on_gpu = True
            ev0 = ev1 = None
            if keep:
                ev0 = torch.cuda.Event(enable_timing=True)
                ev1 = torch.cuda.Event(enable_timing=True)
                self._gpu_streamed_step(keep, scale, ev0, ev1)
            self._pending_timing = (ev0, ev1, n_gpu, n_cpu_moved)
        import time as _time

        t_cpu0 = _time.perf_counter()
        if on_gpu:
            d2h, h2d = self._streams()
            d2h.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(d2h):
                for i, (p, state, group, lo, hi, tag) in enumerate(work):
                    if tag == "stepped":
                        stepped.add(id(p))
                    if p in self._staged:
                        work[i] = (p, state, group, lo, hi, self._staged[p])
                        continue
                    key = "_grad_fp32" if p.dtype == torch.float32 else "_grad_fp16"
                    g = p.grad.reshape(-1)
                    g.record_stream(d2h)   # step() returns before the copy has run
                    state[key].view(-1)[lo:hi].copy_(g[lo:hi], non_blocking=True)
                    ev = torch.cuda.Event()
                    ev.record(d2h)
                    work[i] = (p, state, group, lo, hi, ev)

        if on_gpu and not self.record_delta:
            work = self._run_native(work, stepped, scale, h2d)
        rest_uploads = any(p.is_cuda for p, *_ in work)

        sum_delta = sum_sq_delta = 0.0
        total_numel = 0
        for p, state, group, lo, hi, ev in work:
            if ev is not None:
                ev.synchronize()
            beta1, beta2 = group["betas"]
            sign = -1.0 if group.get("maximize", False) else 1.0
            if id(p) not in stepped:
                stepped.add(id(p))
                first = True
            else:
                first = False
            if p.dtype == torch.float32:
                grad = state["_grad_fp32"] if p.is_cuda else p.grad
                grad = grad * (sign / scale)
                lr = 0.0 if state["step"] < self._hold_steps else group["lr"]
                torch.optim._functional.adam(
                    [state["_param_fp32"]], [grad], [state["exp_avg"]], [state["exp_avg_sq"]], [],
                    [torch.tensor(float(state["step"]))],
                    amsgrad=False, beta1=beta1, beta2=beta2, lr=lr, weight_decay=group["weight_decay"],
                    eps=group["eps"], maximize=False,
                )
                state["step"] += 1
                if p.is_cuda:
                    with torch.cuda.stream(h2d):
                        p.data.copy_(state["_param_fp32"], non_blocking=True)
                else:
                    p.data.copy_(state["_param_fp32"])
                continue
            if first:
                state["step"] += 1
            if hi == lo:
                continue
            lr = 0.0 if state["step"] < self._hold_steps else group["lr"]
            if p.is_cuda:
                grad = state["_grad_fp16"].view(-1)[lo:hi]
            else:
                grad = p.grad.reshape(-1)[lo:hi].contiguous()
            if sign < 0:
                grad = -grad
            out_half = state["_param_fp16"].view(-1)[lo:hi]
            delta = p._delta_info if self.record_delta else None
            _adam.adam_cpu(
                state["_param_fp32"].view(-1)[lo:hi], out_half, delta, grad,
                state["exp_avg"].view(-1)[lo:hi], state["exp_avg_sq"].view(-1)[lo:hi],
                beta1, beta2, group["eps"], lr, scale, group["weight_decay"], state["step"],
            )
            total_numel += hi - lo
            if self.record_delta:
                sum_delta += float(delta[2])
                sum_sq_delta += float(delta[3])
            if p.is_cuda:
                with torch.cuda.stream(h2d):
                    p.data.view(-1)[lo:hi].copy_(out_half, non_blocking=True)
            else:
                p.data.view(-1)[lo:hi].copy_(out_half)
        self._drop_ahead()   # leftovers (parameters that had no gradient this time)
        if on_gpu and not self._async:
            self.synchronize()
            torch.cuda.current_stream().wait_stream(h2d)
        elif on_gpu and rest_uploads:
            torch.cuda.current_stream().wait_stream(h2d)
        pend = getattr(self, "_pending_timing", None)
        if pend is not None and pend[0] is not None:
            self._last_timing = (pend[0], pend[1], pend[2], _time.perf_counter() - t_cpu0, pend[3])
        self._pending_timing = None
        self._staged.clear()
        if self.record_delta and total_numel:
            self.avg_delta = sum_delta / total_numel
            self.var_delta = sum_sq_delta / total_numel - self.avg_delta ** 2
        return loss

    def _run_native(self, work, stepped, scale, h2d):
        """Queue the half-precision device parameters' chunks on the native worker (event wait -> host Adam -> upload,
        ``csrc/runtime.cu``), one batch per parameter in the order given (= the order in which a forward pass uses
        them); returns the work items it does not cover (fp32 parameters, host tensors)."""
        fn = self._cpu_fn()
        if fn is None:
            return work
        rest, per_param = [], {}
        for item in work:
            p, state, group, lo, hi, ev = item
            if p.is_cuda and p.dtype in (torch.float16, torch.bfloat16) and not group.get("maximize", False) and hi > lo:
                per_param.setdefault(p, (state, group, []))[2].append((lo, hi, ev))
            else:
                rest.append(item)
        lib = self._lib()
        for p, (state, group, pieces) in per_param.items():
            if id(p) not in stepped:
                stepped.add(id(p))
                state["step"] += 1
            jobs = self._jobs_for(p, state, group, scale, state["step"], pieces)
            self._track(p, lib.bmt_offload_submit(jobs, ctypes.c_int(len(pieces)), fn, ctypes.c_void_p(h2d.cuda_stream)),
                        keep=[ev for _, _, ev in pieces if ev is not None])
        return rest

    def get_avg_delta(self):
        return self.avg_delta if self.record_delta else 0

    def get_var_delta(self):
        return self.var_delta if self.record_delta else 0

    # ------------------------------------------------------------- state dict
    def state_dict(self, gather: bool = False) -> dict:
        self._host_state_ready()
        param_mappings = {}
        start_index = 0

        def pack_group(group):
            nonlocal start_index
            packed = {k: v for k, v in group.items() if k != "params"}
            param_mappings.update({id(p): i for i, p in enumerate(group["params"], start_index) if id(p) not in param_mappings})
            packed["params"] = [param_mappings[id(p)] for p in group["params"]]
            start_index += len(packed["params"])
            return packed

        def cut_states(state):
            return {k: state[k] for k in ("step", "exp_avg", "exp_avg_sq", "_param_fp32")}

        param_groups = [pack_group(g) for g in self.param_groups]
        packed_state = {(param_mappings[id(k)] if isinstance(k, torch.Tensor) else k): cut_states(v)
                        for k, v in self.state.items() if len(v) > 0}
        states = {"state": packed_state, "param_groups": param_groups}
        if gather:
            states = deepcopy(states)
            params = list(chain.from_iterable(g["params"] for g in self.param_groups))
            comms = {}
            for i, p in enumerate(params):
                c = getattr(p, "_bmt_comm", None) or getattr(p, "_zero_comm", None)
                if c is not None:
                    comms[i] = c
            states = state_dict_gather(states, comms)
            states["is_whole"] = True
        else:
            states["is_whole"] = False
        return states

    def load_state_dict(self, state_dict: dict) -> None:
        self._host_state_ready()
        # the state objects are replaced below: results computed ahead and the second sets of arrays go with the old ones
        self._drop_ahead()
        self._ahead_owners = []
        if self._gpu_pipe is not None:
            self._gpu_pipe["host_done"].clear()
        state_dict = deepcopy(state_dict)
        groups = self.param_groups
        saved_groups = state_dict["param_groups"]
        if len(groups) != len(saved_groups):
            raise ValueError("loaded state dict has a different number of parameter groups")
        if any(len(g["params"]) != len(s["params"]) for g, s in zip(groups, saved_groups)):
            raise ValueError("loaded state dict contains a parameter group that doesn't match the size of optimizer's group")
        id_map = dict(zip(chain.from_iterable(g["params"] for g in saved_groups),
                          chain.from_iterable(g["params"] for g in groups)))
        is_whole = state_dict.get("is_whole", False)
        state = defaultdict(dict)
        for k, v in state_dict["state"].items():
            if k not in id_map:
                state[k] = v
                continue
            param = id_map[k]
            if is_whole:
                bounds = _partition_bounds(param)
                if bounds is not None:
                    for key in ("_param_fp32", "exp_avg_sq", "exp_avg"):
                        if key in v:
                            v[key] = v[key][bounds[0]:bounds[1]]
            if "_param_fp32" not in v:
                v["_param_fp32"] = param.detach().to("cpu", torch.float32)
            for name in ("exp_avg", "exp_avg_sq", "_param_fp32"):
                if name in v:
                    src = v[name].to("cpu", torch.float32).reshape(param.shape)
                    dst = _pinned(param.size(), torch.float32, param.is_cuda)
                    dst.copy_(src)
                    v[name] = dst
            self._make_staging(param, v)
            state[param] = v
        param_groups = []
        for g, ng in zip(groups, saved_groups):
            ng["params"] = g["params"]
            param_groups.append(ng)
        self.__setstate__({"state": state, "param_groups": param_groups})

    def zero_grad(self, set_to_none: bool = False):
        self._drop_ahead()   # a skipped step: what was computed from these gradients is not wanted
        if self._staged:
            # a skipped step may leave copies in flight: let them finish before the gradients are overwritten
            for ev in self._staged.values():
                ev.synchronize()
            self._staged.clear()
        _zero_grad(self, set_to_none)
