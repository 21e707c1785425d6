"""Training-step benchmark for any model shape and parallel layout of this package.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 -m bmtrain_b200.benchmark.model_step \\
        --model llama --layers 8 --dim 5120 --heads 40 --ffn 13824 --seq 4096 --batch 1 --tp 2 --dtype bf16

Every rank runs ``--steps`` steps of forward, loss, backward and optimizer step on synthetic tokens (``--warmup`` untimed
ones first); the step time is device-timed with CUDA events and reported as the maximum over ranks together with
tokens per second of the whole job, per-phase times (forward / backward / optimizer, each the maximum over ranks) and the
peak device memory.  Parallelism: ``--tp`` tensor parallel (sequence sharded between the linears), ``--pp`` pipeline
stages with ``--micros`` micro-batches, the remaining ranks are ZeRO data parallel (``--zero 2|3``).

(The reference ships one hard-wired example loop, ``example/train.py``; shapes and layouts are edited in the source.)
"""
from __future__ import annotations

import argparse
import json
import os
import time

import torch

import bmtrain_b200 as bmt
from bmtrain_b200.global_var import config


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gpt", choices=["gpt", "llama"])
    ap.add_argument("--layers", type=int, default=8)
    ap.add_argument("--dim", type=int, default=2560)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--kv-heads", type=int, default=0, help="llama: number of key/value heads (0 = same as --heads)")
    ap.add_argument("--ffn", type=int, default=8192)
    ap.add_argument("--vocab", type=int, default=10240)
    ap.add_argument("--activation", default="relu", choices=["relu", "gelu"], help="gpt: feed-forward activation")
    ap.add_argument("--seq", type=int, default=512)
    ap.add_argument("--batch", type=int, default=2, help="sequences per data-parallel rank and step")
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--pp", type=int, default=1)
    ap.add_argument("--micros", type=int, default=0, help="pipeline micro-batches (default: number of stages)")
    ap.add_argument("--zero", type=int, default=3, choices=[2, 3])
    ap.add_argument("--optimizer", default="adam", choices=["adam", "offload"])
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args()
    os.environ.setdefault("BMT_QUIET", "1")
    kw = {}
    if args.pp > 1:
        kw.update(pipe_size=args.pp, num_micro_batches=args.micros or args.pp)
    bmt.init_distributed(seed=0, tp_size=args.tp, **kw)
    dev = config["device"]
    cuda = dev.type == "cuda"
    dt = (torch.bfloat16 if args.dtype == "bf16" else torch.float16) if cuda else torch.float32
    rank, world = bmt.rank(), bmt.world_size()
    if args.model == "gpt":
        model = bmt.models.GPT(args.layers, args.vocab, args.dim, args.dim // args.heads, args.heads, args.ffn, args.seq,
                               bias=True, dtype=dt, zero_level=args.zero, activation=args.activation)
    else:
        model = bmt.models.Llama(args.layers, args.vocab, args.dim, args.heads, args.ffn, num_kv_heads=args.kv_heads or None,
                                 dtype=dt, zero_level=args.zero)
    bmt.init_parameters(model)
    n_params = sum(p._original_shape.numel() if hasattr(p, "_original_shape") else p.numel() for p in model.parameters())
    loss_fn = bmt.loss.FusedCrossEntropy(ignore_index=-100, parallel=args.tp > 1)
    opt_cls = bmt.optim.AdamOffloadOptimizer if args.optimizer == "offload" else bmt.optim.AdamOptimizer
    optimizer = opt_cls(model.parameters(), lr=1e-4, weight_decay=1e-2)
    om = bmt.optim.OptimManager(loss_scale=2 ** 16 if dt == torch.float16 else None)
    om.add_optimizer(optimizer)
    dp_rank = rank // args.tp  # ranks of one tensor-parallel group see the same samples
    gen = torch.Generator().manual_seed(1234 + dp_rank)
    batches = [torch.randint(0, args.vocab, (args.batch, args.seq + 1), generator=gen).to(dev) for _ in range(4)]
    pos = torch.arange(args.seq, device=dev)[None].expand(args.batch, -1).contiguous()
    mask = torch.ones(args.batch, args.seq, dtype=torch.bool, device=dev)
    timer = bmt.utils.StepTimer()

    def step(ids):
        inp, tgt = ids[:, :-1].contiguous(), ids[:, 1:].contiguous()
        with timer.phase("forward"):
            logits = model(inp, pos, mask) if args.model == "gpt" else model(inp)
            if args.tp > 1:
                tgt = tgt.t().contiguous()  # tensor-parallel models return (seq, batch, vocab / tp)
            loss = loss_fn(logits.reshape(-1, logits.shape[-1]), tgt.reshape(-1))
        with timer.phase("backward"):
            om.zero_grad()
            om.backward(loss)
        with timer.phase("optimizer"):
            om.step()
        return loss

    for i in range(args.warmup):
        step(batches[i % 4])
        timer.finish_step(reduce=False)
    timer = bmt.utils.StepTimer()
    bmt.synchronize()
    if cuda:
        torch.cuda.synchronize()
        torch.cuda.reset_peak_memory_stats()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
    t0 = time.perf_counter()
    phases = []
    for i in range(args.steps):
        loss = step(batches[i % 4])
        phases.append(timer.finish_step())
    if cuda:
        end.record()
        torch.cuda.synchronize()
        ms = start.elapsed_time(end)
    else:
        ms = (time.perf_counter() - t0) * 1e3
    t = torch.tensor([ms], dtype=torch.float32, device=dev)
    t = bmt.distributed.all_reduce(t, "max") if world > 1 else t
    ms = float(t[0]) / args.steps
    dp = world // (args.tp * args.pp) * (args.pp if args.pp > 1 else 1)  # pipeline ranks each feed their own samples
    tokens = dp * args.batch * args.seq
    mean = {k: sum(p[k] for p in phases) / len(phases) for k in phases[0]}
    out = {
        "model": args.model, "layers": args.layers, "dim": args.dim, "heads": args.heads, "ffn": args.ffn, "vocab": args.vocab,
        "seq": args.seq, "batch_per_dp_rank": args.batch, "params": int(n_params), "dtype": str(dt).replace("torch.", ""),
        "world": world, "tp": args.tp, "pp": args.pp, "zero": args.zero, "optimizer": args.optimizer,
        "ms_per_step": round(ms, 3), "tokens_per_s": round(tokens / ms * 1e3, 1),
        "phase_ms_max_over_ranks": {k: round(v, 3) for k, v in mean.items()},
        "model_tflops_per_gpu": round(6.0 * n_params * tokens / ms / 1e9 / world * (4.0 / 3.0), 1),
        "peak_mem_gb": round(torch.cuda.max_memory_allocated() / 2 ** 30, 2) if cuda else None,
        "final_loss": float(loss.detach().float().cpu()),
        "note": "model_tflops counts 6 * params * tokens plus the recomputed forward (x 4/3), attention scores excluded",
    }
    if rank == 0:
        print(json.dumps(out), flush=True)
    bmt.synchronize()
    bmt.shutdown()


if __name__ == "__main__":
    main()
