"""Headline benchmark: tokens/s of ZeRO-3 training on the reference's example GPT (and, with ``--config llama13b``, of
the Llama-13B-shaped ZeRO-3 x tensor-parallel-2 configuration).

Config (the reference's example/train.py model): 8 pre-LN blocks, d_model 2560, 32 heads x 80, FFN 8192, vocab 10240,
bias, learned positions (512), fp16 with OptimManager dynamic loss scaling (2**20), ZeRO-3 TransformerBlockList,
AdamOffloadOptimizer (fp32 state in host memory, weight decay 1e-2), per-GPU batch 2 x 512 uniform random tokens,
random-init weights.  Weak scaling: per-GPU work is fixed as N grows.

    python bench.py --gpus 1 --steps 10 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 10 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref, same loop

    torchrun ... bench.py --gpus 8 --config llama13b [--layers 40] [--micro-batch 2]   # second named configuration:
        40 layers, d 5120, 40 heads x 128, SwiGLU 13824, RMSNorm, RoPE, vocab 32000, bf16, seq 4096, global batch 64
        sequences per step (gradient accumulation over micro-batches), ZeRO-3 x tp 2, AdamOptimizer, vocabulary-parallel
        fused cross-entropy; the reference arm builds the same decoder from the reference's own layers
        (baseline/llama_reference.py)

Rank 0 prints ONE JSON line.  `value` is device-timed (CUDA events around exactly K steps, inputs already on the
device, max over ranks); `e2e` repeats the measurement with every step's inputs copied from pinned host memory and
the loss read back to the host.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
MODEL = dict(num_layers=8, vocab_size=10240, dim_model=2560, dim_head=80, num_heads=32, dim_ff=8192, max_distance=512)
BATCH, SEQ = 2, 512
PUBLISHED_TOKENS_PER_GPU_S = 29.42 * 512  # reference README: GPT-2 13B on 4x8 V100, best batch size


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--config", default="gpt-example", choices=["gpt-example", "llama13b"])
    ap.add_argument("--layers", type=int, default=0, help="llama13b: number of layers (default 40; fewer = a reduced run, said so in the output)")
    ap.add_argument("--micro-batch", type=int, default=2, help="llama13b: sequences per micro-batch and data-parallel rank")
    ap.add_argument("--global-batch", type=int, default=64, help="llama13b: sequences per optimizer step over the whole job")
    ap.add_argument("--optimizer", default="offload", choices=["offload", "adam"],
                    help="offload = AdamOffloadOptimizer (the headline config); adam = AdamOptimizer with the state in HBM "
                         "(a secondary measurement: the step is then bound by the GPU, not by host memory)")
    return ap.parse_args()


class ClockSampler:
    """Samples SM clocks, power and throttle reasons of this rank's GPU while the timed region runs.

    The figures are the ones `nvidia-smi --query-gpu=clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.*` prints,
    read through NVML from a thread of this process every 100 ms: a looping nvidia-smi process needs a CPU core of its own
    (more than 100 ms per sample here), which slows the host-side optimizer of the rank it shares cores with and, through
    the max over ranks, the whole job.  Without the NVML binding the nvidia-smi loop is used at a slower rate.
    """

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    BITS = (("hw_slowdown", 0x8), ("hw_thermal_slowdown", 0x40), ("sw_thermal_slowdown", 0x20), ("sw_power_cap", 0x4))

    def __init__(self, index: int):
        self.proc = self.thread = None
        self.sm, self.mx, self.power, self.reasons = [], [], [], set()
        try:
            import threading

            import pynvml
            import torch

            pynvml.nvmlInit()
            try:
                uuid = str(torch.cuda.get_device_properties(index).uuid)
                handle = pynvml.nvmlDeviceGetHandleByUUID(("GPU-" + uuid) if not uuid.startswith("GPU-") else uuid)
            except Exception:
                handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self._nvml, self._handle = pynvml, handle
            self._sample()  # fails here, not in the thread, when a query is unsupported
            self._stop = threading.Event()
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
            self.sm, self.mx, self.power, self.reasons = [], [], [], set()
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "500"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            pass

    def _sample(self):
        n, h = self._nvml, self._handle
        self.sm.append(float(n.nvmlDeviceGetClockInfo(h, n.NVML_CLOCK_SM)))
        self.mx.append(float(n.nvmlDeviceGetMaxClockInfo(h, n.NVML_CLOCK_SM)))
        self.power.append(n.nvmlDeviceGetPowerUsage(h) / 1000.0)
        get = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        mask = int(get(h))
        for name, bit in self.BITS:
            if mask & bit:
                self.reasons.add(name)

    def _loop(self):
        while not self._stop.wait(0.1):
            try:
                self._sample()
            except Exception:
                return

    def _summary(self, source):
        sm = self.sm
        busy = sorted(sm)[len(sm) // 2:] if sm else []  # the top half of the samples are the ones taken under load
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(self.mx) if self.mx else None,
                "power_w_max": max(self.power) if self.power else None, "samples": len(sm), "reasons": sorted(self.reasons),
                "source": source}

    def stop(self):
        if self.thread is not None:
            self._stop.set()
            self.thread.join(timeout=2)
            return self._summary("NVML, 100 ms")
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        for line in out.strip().splitlines():
            f = [x.strip() for x in line.split(",")]
            if len(f) < 8:
                continue
            try:
                self.sm.append(float(f[0])); self.mx.append(float(f[1])); self.power.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[4:8]):
                if val.lower().startswith("active"):
                    self.reasons.add(name)
        return self._summary("nvidia-smi -lms 500")


def setup_env(args):
    os.environ.setdefault("RANK", "0")
    os.environ.setdefault("WORLD_SIZE", "1")
    os.environ.setdefault("LOCAL_RANK", os.environ["RANK"])
    os.environ.setdefault("LOCAL_WORLD_SIZE", os.environ["WORLD_SIZE"])
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29517")
    os.environ.setdefault("BMT_QUIET", "1")
    world = int(os.environ["WORLD_SIZE"])
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")


def build_ours(opt_kind="offload"):
    import torch
    import bmtrain_b200 as bmt

    bmt.init_distributed(seed=0)
    model = bmt.models.GPT(**MODEL, bias=True, dtype=torch.half)
    bmt.init_parameters(model)
    loss_func = bmt.loss.FusedCrossEntropy(ignore_index=-100)
    opt_cls = bmt.optim.AdamOffloadOptimizer if opt_kind == "offload" else bmt.optim.AdamOptimizer
    optimizer = opt_cls(model.parameters(), weight_decay=1e-2)
    lr_scheduler = bmt.lr_scheduler.Noam(optimizer, start_lr=1e-3, warmup_iter=40, end_iter=1000, num_iter=0)
    om = bmt.optim.OptimManager(loss_scale=2 ** 20)
    om.add_optimizer(optimizer, lr_scheduler)

    def loss_of(logits, targets):
        return loss_func(logits.view(-1, logits.size(-1)), targets.view(-1))

    from bmtrain_b200.ops import _native
    import ctypes

    lib = _native.cuda_lib()
    lib.bmt_launch_count.restype = ctypes.c_int64
    return bmt, model, om, loss_of, lib.bmt_launch_count


def build_reference(opt_kind="offload"):
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
    sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref", "example"))
    import torch
    import bmtrain as bmt
    from models import GPT  # the reference's own example model

    bmt.init_distributed(seed=0)
    model = GPT(num_layers=MODEL["num_layers"], vocab_size=MODEL["vocab_size"], dim_model=MODEL["dim_model"],
                dim_head=MODEL["dim_head"], num_heads=MODEL["num_heads"], dim_ff=MODEL["dim_ff"],
                max_distance=MODEL["max_distance"], bias=True, dtype=torch.half)
    bmt.init_parameters(model)
    loss_func = torch.nn.CrossEntropyLoss(ignore_index=-100)
    opt_cls = bmt.optim.AdamOffloadOptimizer if opt_kind == "offload" else bmt.optim.AdamOptimizer
    optimizer = opt_cls(model.parameters(), weight_decay=1e-2)
    lr_scheduler = bmt.lr_scheduler.Noam(optimizer, start_lr=1e-3, warmup_iter=40, end_iter=1000, num_iter=0)
    om = bmt.optim.OptimManager(loss_scale=2 ** 20)
    om.add_optimizer(optimizer, lr_scheduler)

    def loss_of(logits, targets):
        return loss_func(logits.view(-1, logits.size(-1)).float(), targets.view(-1))

    return bmt, model, om, loss_of, (lambda: 0)


LLAMA = dict(vocab_size=32000, dim_model=5120, num_heads=40, dim_ff=13824)
LLAMA_SEQ = 4096


def run_llama(args, emit):
    """``--config llama13b``: one optimizer step = global batch of sequences, accumulated over micro-batches."""
    import torch

    layers = args.layers or 40
    tp = 2
    if args.impl == "reference":
        sys.path.insert(0, os.path.join(ROOT, "baseline", "_ref"))
        sys.path.insert(0, os.path.join(ROOT, "baseline"))
        import bmtrain as bmt
        from llama_reference import RefLlama

        bmt.init_distributed(seed=0, tp_size=tp)
        model = RefLlama(layers, dtype=torch.bfloat16, **LLAMA)
        launch_count = lambda: 0
        finish_updates = lambda: None
    else:
        import bmtrain_b200 as bmt

        bmt.init_distributed(seed=0, tp_size=tp)
        model = bmt.models.Llama(layers, dtype=torch.bfloat16, **LLAMA)
        from bmtrain_b200.ops import _native
        import ctypes

        lib = _native.cuda_lib()
        lib.bmt_launch_count.restype = ctypes.c_int64
        launch_count = lib.bmt_launch_count
        finish_updates = bmt.optim.adam_offload.finish_all_updates
    bmt.init_parameters(model)
    loss_func = bmt.loss.FusedCrossEntropy(ignore_index=-100, parallel=True)
    optimizer = bmt.optim.AdamOptimizer(model.parameters(), lr=1e-4, weight_decay=1e-2)
    om = bmt.optim.OptimManager(loss_scale=None)
    om.add_optimizer(optimizer)
    rank, world = bmt.rank(), bmt.world_size()
    if world % tp:
        raise SystemExit("llama13b needs an even number of GPUs (tp = 2)")
    dp = world // tp
    dp_rank = rank // tp
    per_rank = args.global_batch // dp
    mb = args.micro_batch
    micro_steps = per_rank // mb
    if micro_steps * mb * dp != args.global_batch:
        raise SystemExit("global batch must be a multiple of dp x micro-batch")
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator().manual_seed(2000 + dp_rank)   # the two ranks of a tensor-parallel pair see the same sequences
    host = [torch.randint(0, LLAMA["vocab_size"], (mb, LLAMA_SEQ + 1), generator=gen).pin_memory() for _ in range(4)]
    on_dev = [h.to(dev) for h in host]

    def step(batches, e2e):
        om.zero_grad()
        total = None
        for i in range(micro_steps):
            ids = batches[i % len(batches)]
            if e2e:
                ids = ids.to(dev, non_blocking=True)
            logits = model(ids[:, :-1].contiguous())                      # (s, b, vocab / tp)
            target = ids[:, 1:].t().contiguous().view(-1)
            loss = loss_func(logits.reshape(-1, logits.shape[-1]), target) / micro_steps
            om.backward(loss)
            total = loss.detach() if total is None else total + loss.detach()
        om.step()
        return float(total) if e2e else total

    for _ in range(max(args.warmup, 1)):
        step(on_dev, False)

    # One timed pass (a step takes seconds): every micro-batch comes from pinned host memory and the loss is read back, so
    # the pass is the end-to-end measurement; `value` is its CUDA-event time, `e2e` the larger of that and the wall clock.
    finish_updates()
    bmt.synchronize()
    torch.cuda.synchronize()
    sampler = ClockSampler(torch.cuda.current_device()) if rank == 0 else None
    l0 = launch_count()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    last = None
    for _ in range(args.steps):
        last = step(host, True)
    finish_updates()
    end.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) * 1e3
    bmt.synchronize()
    t = torch.tensor([start.elapsed_time(end), max(start.elapsed_time(end), wall), float(last)], device=dev)
    t = bmt.distributed.all_reduce(t, "max")
    ms, ms_e2e, final_loss = float(t[0]), float(t[1]), float(t[2])
    launches = launch_count() - l0
    clocks = sampler.stop() if sampler else None
    tokens = args.global_batch * LLAMA_SEQ * args.steps
    value = tokens / (ms / 1e3)
    n_params = layers * (4 * 5120 * 5120 + 3 * 5120 * 13824) + 2 * 32000 * 5120
    if rank == 0:
        emit({
            "metric": "tokens/sec/box (device-timed, max over ranks)", "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic uniform token ids, random-init weights", "impl": args.impl,
            "config": {"model": f"Llama-13B-shaped decoder, {layers} layers" + ("" if layers == 40 else " (REDUCED from 40)")
                                + ", d 5120, 40 heads x 128, SwiGLU 13824, RMSNorm, RoPE, vocab 32000",
                       "global_batch": args.global_batch, "seq_len": LLAMA_SEQ, "micro_batch": mb, "micro_steps": micro_steps,
                       "parallelism": f"zero3 x tp{tp} (dp {dp})", "optimizer": "AdamOptimizer (state in HBM), no loss scaling",
                       "loss": "FusedCrossEntropy(parallel=True)", "activation_checkpointing": True,
                       "l2": "inputs larger than L2: every step streams tens of GB of weights and activations"},
            "clocks": clocks,
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s", "h2d_bytes_per_step": micro_steps * mb * (LLAMA_SEQ + 1) * 8,
                    "d2h_bytes_per_step": 4, "timing": "max(CUDA events, wall clock), inputs from pinned host memory, loss read back"},
            "gpu_launches": launches, "final_loss": round(final_loss, 4),
            "model_tflops_per_gpu": 6.0 * n_params * tokens / (ms / 1e3) / world / 1e12,
        })
    try:
        if torch.distributed.is_initialized():
            torch.distributed.destroy_process_group()
    except Exception:
        pass


def main():
    args = parse()
    setup_env(args)
    # stdout carries exactly one line, the JSON result: everything libraries print (NCCL banner, loss-scale notices of
    # either arm) goes to stderr instead
    sys.stdout.flush()
    result_fd = os.dup(1)
    os.dup2(2, 1)

    def emit(obj):
        sys.stdout.flush()
        os.write(result_fd, (json.dumps(obj) + "\n").encode())

    if args.impl == "reference" and not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "bmtrain")):
        emit({"impl": "reference", "unavailable": "baseline/_ref is not installed on this machine"})
        return
    import torch

    if not torch.cuda.is_available():
        emit({"impl": args.impl, "unavailable": "no CUDA device"})
        return
    if args.config == "llama13b":
        try:
            run_llama(args, emit)
        except Exception as exc:
            if args.impl != "reference":
                raise
            import traceback

            traceback.print_exc()
            emit({"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"})
        return
    try:
        bmt, model, om, loss_of, launch_count = (build_reference if args.impl == "reference" else build_ours)(args.optimizer)
    except Exception as exc:  # the reference may fail to import/run on this image
        if args.impl == "reference":
            emit({"impl": "reference", "unavailable": f"{type(exc).__name__}: {str(exc)[:200]}"})
            return
        raise
    rank, world = bmt.rank(), bmt.world_size()
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator().manual_seed(1000 + rank)
    n_batches = 4
    host = [torch.randint(0, MODEL["vocab_size"], (BATCH, SEQ + 1), generator=gen).pin_memory() for _ in range(n_batches)]
    pos = torch.arange(SEQ, device=dev)[None].expand(BATCH, -1).contiguous()
    mask = torch.ones(BATCH, SEQ, dtype=torch.bool, device=dev)
    on_dev = [h.to(dev) for h in host]
    skipped = 0
    # our optimizer applies its step on a worker thread while the next forward pass runs; a timed region ends only when
    # that worker is idle, so K timed steps always contain K complete optimizer steps
    finish_updates = getattr(getattr(bmt.optim, "adam_offload", None), "finish_all_updates", None) or (lambda: None)

    def step(ids, read_loss, marks=None):
        nonlocal skipped
        inp, tgt = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
        if marks is not None:
            marks["f0"].record()
        logits = model(inp, pos, mask)
        loss = loss_of(logits, tgt)
        om.zero_grad()
        if marks is not None:
            marks["f1"].record()
        before = om.loss_scale
        om.backward(loss)
        if marks is not None:
            marks["b1"].record()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
        om.step()
        if marks is not None:
            finish_updates()
            torch.cuda.synchronize()
            marks["opt_ms"] = (time.perf_counter() - t0) * 1e3
        if om.loss_scale < before:
            skipped += 1
        return loss.item() if read_loss else loss

    # loss-scale settling (not timed, not counted as warm-up): run until a step is not skipped for overflow
    for i in range(24):
        s0 = skipped
        step(on_dev[i % n_batches], False)
        if skipped == s0:
            break
    for i in range(args.warmup):
        step(on_dev[i % n_batches], False)

    def timed(e2e: bool):
        nonlocal skipped
        skipped = 0
        finish_updates()
        bmt.synchronize()
        torch.cuda.synchronize()
        sampler = ClockSampler(torch.cuda.current_device()) if rank == 0 and os.environ.get("BMT_BENCH_NO_CLOCKS") != "1" else None
        l0 = launch_count()
        stats0 = dict(getattr(om.optimizers[0], "stats", {}))
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record()
        last = None
        for i in range(args.steps):
            if e2e:
                ids = host[i % n_batches].to(dev, non_blocking=True)
                last = step(ids, True)
            else:
                last = step(on_dev[i % n_batches], False)
        finish_updates()
        end.record()
        torch.cuda.synchronize()
        wall_ms = (time.perf_counter() - t0) * 1e3
        bmt.synchronize()
        ms = max(start.elapsed_time(end), wall_ms)   # the optimizer's host part runs outside any stream: wall clock bounds it
        t = torch.tensor([ms, float(skipped), float(last)], device=dev, dtype=torch.float32)
        if world > 1:
            t = bmt.distributed.all_reduce(t, "max")  # same call in both arms (each arm's own collective layer)
        clocks = sampler.stop() if sampler else None
        now = dict(getattr(om.optimizers[0], "stats", {}))
        offload_stats.append({k: now[k] - stats0.get(k, 0) for k in now})
        return float(t[0]), int(t[1]), launch_count() - l0, clocks, float(t[2])

    offload_stats = []   # per timed pass: parameter updates computed during backward (queued / adopted / re-queued / dropped)
    ms, skip_dev, launches, clocks, _ = timed(False)
    ms_e2e, skip_e2e, _, _, final_loss = timed(True)

    # where the time goes (not part of the timed regions): device time of forward and backward, wall time of a complete,
    # un-overlapped optimizer step, and the communication that computation does not hide (= forward + backward with
    # real collectives minus the same with rank-local stand-ins; 0 on one GPU)
    def phase_probe(n):
        acc = {"forward": 0.0, "backward": 0.0, "optimizer": 0.0}
        for i in range(n):
            marks = {k: torch.cuda.Event(enable_timing=True) for k in ("f0", "f1", "b1")}
            finish_updates()
            torch.cuda.synchronize()
            step(on_dev[i % n_batches], False, marks)
            acc["forward"] += marks["f0"].elapsed_time(marks["f1"]) / n
            acc["backward"] += marks["f1"].elapsed_time(marks["b1"]) / n
            acc["optimizer"] += marks["opt_ms"] / n
        return acc

    phases = phase_probe(3)
    exposed = 0.0
    if world > 1 and args.impl == "ours":
        from bmtrain_b200.comm import local_collectives

        with local_collectives():
            phase_probe(1)
            quiet = phase_probe(3)
        exposed = max(0.0, phases["forward"] + phases["backward"] - quiet["forward"] - quiet["backward"])
        phase_probe(1)   # back on real collectives
    pt = torch.tensor([phases["forward"], phases["backward"], phases["optimizer"], exposed], device=dev)
    if world > 1:
        pt = bmt.distributed.all_reduce(pt, "max")
    phase_ms = {"forward": round(float(pt[0]), 2), "backward": round(float(pt[1]), 2),
                "optimizer_unoverlapped": round(float(pt[2]), 2),
                "exposed_comm": round(float(pt[3]), 2) if args.impl == "ours" else None}

    tokens = world * BATCH * SEQ * args.steps
    value = tokens / (ms / 1e3)
    if rank == 0:
        out = {
            "metric": "tokens/sec/box (device-timed, max over ranks); exposed comm/step in phase_ms", "value": value,
            "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms / args.steps,
            "higher_is_better": True, "scaling": "weak",
            "vs_baseline": value / (PUBLISHED_TOKENS_PER_GPU_S * world),
            "dtype": "fp16", "data": "synthetic uniform token ids, random-init weights",
            "impl": args.impl,
            "config": {"model": "GPT 8x d2560 (32 heads x 80, FFN 8192, vocab 10240, bias, max_distance 512)",
                       "global_batch": BATCH * world, "seq_len": SEQ, "parallelism": f"zero3-dp{world}",
                       "optimizer": ("AdamOffloadOptimizer" if args.optimizer == "offload" else "AdamOptimizer")
                                    + " + OptimManager(loss_scale=2**20)",
                       "loss": "fused cross-entropy kernel on fp16 logits" if args.impl == "ours"
                               else "nn.CrossEntropyLoss on logits.float() (as in the reference's example/train.py)",
                       "l2": "inputs larger than L2: each step streams 1.1 GB of fp16 weights plus activations (L2 is 126 MB)",
                       "baseline_note": "vs_baseline divides by the reference README's best published figure "
                                        "(29.42 samples/GPU/s x 512 tokens, GPT-2 13B on 32 V100) x n_gpus"},
            "clocks": clocks,
            "e2e": {"value": tokens / (ms_e2e / 1e3), "unit": "tokens/s",
                    "h2d_bytes_per_step": BATCH * (SEQ + 1) * 8, "d2h_bytes_per_step": 4,
                    "timing": "max(CUDA events, wall clock) around K steps incl. pinned-host input copy and loss read-back"},
            "gpu_launches": launches,
            "overflow_skipped_steps": {"device_timed": skip_dev, "e2e": skip_e2e},
            "final_loss": round(final_loss, 4),
            "offload_stats": {"device_timed": offload_stats[0], "e2e": offload_stats[1]},
            "phase_ms": phase_ms,
            "exposed_comm_fraction": round(float(pt[3]) / (ms / args.steps), 4) if args.impl == "ours" else None,
            "timing_note": "value: max(CUDA events, wall clock) over K steps, each region starts and ends with the "
                           "optimizer's worker thread idle",
        }
        emit(out)
    try:
        if torch.distributed.is_initialized():
            torch.distributed.destroy_process_group()
    except Exception:
        pass


if __name__ == "__main__":
    main()
