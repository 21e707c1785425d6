"""Timings of the four fused compute+collective paths against the same work done as NCCL collective + separate kernels.

Run on W GPUs of one NVLink domain::

    python -m torch.distributed.run --nproc-per-node W --master-addr 127.0.0.1 -m bmtrain_b200.benchmark.fused

Every number is device-timed with CUDA events after warm-up, the maximum over ranks, with a large scratch write between
iterations so the operands do not sit in L2.  For each path the report gives

* ``fused``: the single kernel working on peer memory,
* ``split``: NCCL collective followed by (or following) this package's plain kernels,
* ``roofline``: the slower of the arithmetic at the measured sustained GEMM rate and the bytes that have to cross
  NVLink at the measured peer-copy bandwidth (both overridable on the command line),
* ``fraction`` = roofline / fused.

(The reference has no counterpart: its collectives and GEMMs are separate NCCL / cuBLAS calls.)
"""
from __future__ import annotations

import argparse
import json
import os

import torch

import bmtrain_b200 as bmt
from bmtrain_b200.global_var import config


_busy = {}


def _timer(fn, iters: int, warmup: int, flush, host_ahead: bool = False, after_warmup=None) -> float:
    """Device time of ``fn`` (CUDA events, mean over ``iters``, maximum over ranks).  ``host_ahead``: a long matrix product
    is queued in front of the start event, so ``fn`` is enqueued while the device is still busy and its host-side cost
    does not show (the situation of a training step once the host runs ahead of the device)."""
    comm = config["comm"]
    if host_ahead and not _busy:
        _busy["a"] = torch.randn(8192, 8192, device=config["device"], dtype=torch.bfloat16)
        _busy["b"] = torch.randn(8192, 8192, device=config["device"], dtype=torch.bfloat16)
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if after_warmup is not None:
        after_warmup()   # e.g. clear the in-kernel timing counters so they cover the timed iterations only
    comm.barrier()
    total = 0.0
    for _ in range(iters):
        flush.add_(1.0)
        comm.barrier()  # ranks enter together: a fused kernel's waits then measure transfer, not skew
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if host_ahead:
            for _ in range(3):
                torch.mm(_busy["a"], _busy["b"])   # about 2.5 ms of device work
        start.record()
        fn()
        end.record()
        torch.cuda.synchronize()
        total += start.elapsed_time(end)
    t = torch.tensor([total / iters], dtype=torch.float32, device=config["device"])
    comm.all_reduce(t, "max")
    return float(t.item())


def _host_ms(fn, iters: int) -> float:
    """Host time to enqueue ``fn`` (no device sync inside the timed part), maximum over ranks."""
    import time

    total = 0.0
    for _ in range(iters):
        torch.cuda.synchronize()
        config["comm"].barrier()
        t0 = time.perf_counter()
        fn()
        total += time.perf_counter() - t0
        torch.cuda.synchronize()
    t = torch.tensor([total / iters * 1e3], dtype=torch.float32, device=config["device"])
    config["comm"].all_reduce(t, "max")
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=8192, help="tokens of the whole tensor-parallel group")
    ap.add_argument("--hidden", type=int, default=5120)
    ap.add_argument("--ffn", type=int, default=13824)
    ap.add_argument("--block-dim", type=int, default=2560, help="hidden size of the ZeRO block (paths 1 and 2)")
    ap.add_argument("--block-ffn", type=int, default=8192)
    ap.add_argument("--block-tokens", type=int, default=1024)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--gemm-tflops", type=float, default=1355.4, help="sustained dense bf16 rate used for the roofline")
    ap.add_argument("--link-gbs", type=float, default=770.0, help="peer-copy bandwidth per direction per GPU")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    args = ap.parse_args()
    os.environ.setdefault("BMT_QUIET", "1")
    bmt.init_distributed(seed=0)
    comm, dev = config["comm"], config["device"]
    W, rank = comm.size, comm.rank
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    from bmtrain_b200.ops import gemm as G
    from bmtrain_b200.ops import infnan
    from bmtrain_b200.parallel import fused_ops, symm, tp_fused

    rt = symm.peer_runtime(comm)
    if rt is None:
        raise SystemExit("peer memory is not available between these ranks")
    flush = torch.zeros(96 * 1024 * 1024, dtype=torch.float32, device=dev)  # 384 MiB > L2
    rows = []
    gen = torch.Generator(device=dev).manual_seed(7 + rank)

    def rnd(*shape):
        return (torch.randn(*shape, generator=gen, device=dev, dtype=torch.float32) * 0.05).to(dt)

    def report(name, shape, fused_ms, split_ms, flops, link_bytes, extra=None):
        roof_ms = max(flops / (args.gemm_tflops * 1e9), link_bytes / (args.link_gbs * 1e6))
        row = {"path": name, "ranks": W, "shape": shape, "fused_ms": round(fused_ms, 4), "split_ms": round(split_ms, 4),
               "roofline_ms": round(roof_ms, 4), "fraction_of_roofline": round(roof_ms / fused_ms, 3),
               "speedup_vs_split": round(split_ms / fused_ms, 3)}
        if extra:
            row.update(extra)
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)

    # ---------------------------------------------------------- (3) all-gather -> GEMM (column-parallel input gather)
    M, K, N = args.tokens, args.hidden, 3 * args.hidden // W
    x_loc, w = rnd(M // W, K), rnd(N, K)
    x_all = torch.empty(M, K, dtype=dt, device=dev)

    def split_ag():
        comm.all_gather_into(x_all, x_loc)
        return G.gemm_nt(x_all, w)

    def lib_ag():
        comm.all_gather_into(x_all, x_loc)
        return x_all @ w.t()

    before = fused_ops.calls["ag_gemm"]
    fused_ops.kernel_stats()
    t_f = _timer(lambda: tp_fused.all_gather_gemm(x_loc, w, None, comm), args.iters, args.warmup, flush,
                 after_warmup=fused_ops.kernel_stats)
    stats3 = fused_ops.kernel_stats()
    assert fused_ops.calls["ag_gemm"] > before, "fused all-gather -> GEMM did not run"
    t_s = _timer(split_ag, args.iters, args.warmup, flush)
    t_l = _timer(lib_ag, args.iters, args.warmup, flush)
    report("(3) all-gather -> GEMM", [M, N, K], t_f, t_s, 2.0 * M * N * K, (W - 1) * (M // W) * K * 2,
           {"nccl_plus_library_gemm_ms": round(t_l, 4), "kernel_stats": stats3})

    # ------------------------------------------------------- (4) GEMM -> reduce-scatter (row-parallel output scatter)
    M, K, N = args.tokens, args.ffn // W // 8 * 8, args.hidden
    x, w = rnd(M, K), rnd(N, K)
    out = torch.empty(M // W, N, dtype=dt, device=dev)

    def split_rs():
        full = G.gemm_nt(x, w)
        comm.reduce_scatter_into(out, full, "sum")

    def lib_rs():
        full = x @ w.t()
        comm.reduce_scatter_into(out, full, "sum")

    before = fused_ops.calls["gemm_rs"]
    fused_ops.kernel_stats()
    t_f = _timer(lambda: tp_fused.gemm_reduce_scatter(x, w, None, comm), args.iters, args.warmup, flush,
                 after_warmup=fused_ops.kernel_stats)
    stats4 = fused_ops.kernel_stats()
    assert fused_ops.calls["gemm_rs"] > before, "fused GEMM -> reduce-scatter did not run"
    t_s = _timer(split_rs, args.iters, args.warmup, flush)
    t_l = _timer(lib_rs, args.iters, args.warmup, flush)
    report("(4) GEMM -> reduce-scatter", [M, N, K], t_f, t_s, 2.0 * M * N * K, (W - 1) * (M // W) * N * 2,
           {"nccl_plus_library_gemm_ms": round(t_l, 4), "kernel_stats": stats4})

    # --------------------------- (2) gradient reduce-scatter + fp32 accumulate + scale + inf/nan (one block's gradients)
    d, f = args.block_dim, args.block_ffn
    block_params = 4 * d * d + 2 * d * f + 9 * d + f
    part = (block_params + W - 1) // W // 256 * 256
    full = rt.slot(("bench_rs",), W * part * 2)
    full.tensor(dt, W * part).copy_(rnd(W * part))
    acc = rnd(part)
    row = rt.row(("bench_rs", "row"))
    plain_full = full.tensor(dt, W * part).clone()
    tmp = torch.empty(part, dtype=dt, device=dev)
    flag = torch.zeros(1, dtype=torch.uint8, device=dev)

    def fused_rs():
        rt.reduce_scatter(full, row, part, acc, accumulate=True, scale=1.0)

    def split_grad_rs():
        comm.reduce_scatter_into(tmp, plain_full, "sum")
        acc.add_(tmp)
        infnan.has_inf_nan(acc, flag)

    t_f = _timer(fused_rs, args.iters, args.warmup, flush)
    t_s = _timer(split_grad_rs, args.iters, args.warmup, flush)
    report("(2) grad reduce-scatter + accumulate + inf/nan", [W, part], t_f, t_s, 0.0, (W - 1) * part * 2)
    rt.check()
    if symm.nvls_wanted():
        # the same reduction summed inside the switch: every rank receives `part` elements instead of (W - 1) * part
        mc = rt.slot(("bench_rs_mc",), W * part * 2, multicast=True)
        if getattr(mc, "mc_ptr", 0):
            mc.tensor(dt, W * part).copy_(plain_full)
            acc2, row2 = acc.clone(), rt.row(("bench_rs_mc", "row"))
            t_m = _timer(lambda: rt.reduce_scatter(mc, row2, part, acc2, accumulate=True, scale=1.0), args.iters, args.warmup, flush)
            report("(2) the same through multimem.ld_reduce (NVLS)", [W, part], t_m, t_s, 0.0, part * 2,
                   {"roofline_note": "link bytes = one partition: the switch sums, a rank receives the result only"})
            ref = torch.empty(part, dtype=dt, device=dev)
            comm.reduce_scatter_into(ref, plain_full, "sum")
            chk = torch.zeros(part, dtype=dt, device=dev)
            rt.reduce_scatter(mc, row2, part, chk, accumulate=False, scale=1.0)
            torch.cuda.synchronize()
            err = ((chk.float() - ref.float()).abs().max() / ref.float().abs().max().clamp_min(1e-6)).item()
            if rank == 0:
                print(json.dumps({"check": "multimem reduce-scatter vs NCCL", "max_rel_err": err}), flush=True)
            rt.check()

    # ------------------------------- push all-gather kernel alone (moves the block's other parameters in path 1) vs NCCL
    gbuf = rt.slot(("bench_push",), W * part * 2)
    p_free, p_done = rt.row(("bench_push", "free")), rt.row(("bench_push", "done"))
    rt.signal_wait(p_free, 1, signal=True, wait=False)
    shard = rnd(part)
    gathered = torch.empty(W * part, dtype=dt, device=dev)

    def push_gather():
        epoch = rt.next_epoch(p_free)
        rt.push_ranges(gbuf, [(shard.data_ptr(), rank * part * 2, part * 2)], p_free, p_done, epoch, ("bench_push",))
        rt.signal_wait(p_done, epoch, signal=False, wait=True)
        rt.signal_wait(p_free, epoch + 1, signal=True, wait=False)

    t_f = _timer(push_gather, args.iters, args.warmup, flush)
    t_s = _timer(lambda: comm.all_gather_into(gathered, shard), args.iters, args.warmup, flush)
    report("(0) push all-gather kernel vs NCCL all-gather", [W, part], t_f, t_s, 0.0, (W - 1) * part * 2)
    rt.check()

    # ------------------------------------------------- (1) ZeRO-3 gather fused with the block's first GEMM (forward)
    from bmtrain_b200.block_layer import Block, TransformerBlockList
    from bmtrain_b200.models.gpt import TransformerEncoder

    def make(zero_level):
        torch.manual_seed(0)
        blk = Block(TransformerEncoder(d, d // 32, 32, f, bias=True, dtype=dt), use_checkpoint=True, zero_level=zero_level)
        lst = TransformerBlockList([blk])
        bmt.init_parameters(lst)
        return lst

    hidden = rnd(2, args.block_tokens // 2, d)
    mask = torch.ones(2, args.block_tokens // 2, dtype=torch.bool, device=dev)

    def fwd(lst):
        return lst(hidden, mask)  # grad mode on: a ZeRO-2 block then keeps its gathered parameters between calls

    z3 = make(3)
    before = fused_ops.calls["zero_gather_gemm"]
    os.environ["BMT_FUSED_GATHER"] = "1"
    fused_ops.kernel_stats()
    t_f = _timer(lambda: fwd(z3), args.iters, args.warmup, flush, after_warmup=fused_ops.kernel_stats)
    stats1 = fused_ops.kernel_stats()
    host_f = _host_ms(lambda: fwd(z3), args.iters)
    t_f_ahead = _timer(lambda: fwd(z3), args.iters, 1, flush, host_ahead=True)
    ran_fused = fused_ops.calls["zero_gather_gemm"] > before
    os.environ["BMT_FUSED_GATHER"] = "0"
    t_s = _timer(lambda: fwd(z3), args.iters, args.warmup, flush)
    host_s = _host_ms(lambda: fwd(z3), args.iters)
    t_s_ahead = _timer(lambda: fwd(z3), args.iters, 1, flush, host_ahead=True)
    os.environ["BMT_FUSED_GATHER"] = "1"
    z2 = make(2)
    t_res = _timer(lambda: fwd(z2), args.iters, args.warmup, flush)  # parameters stay gathered: compute only
    t_res_ahead = _timer(lambda: fwd(z2), args.iters, 1, flush, host_ahead=True)
    tok = args.block_tokens
    flops = 2.0 * tok * (4 * d * d + 2 * d * f) + 4.0 * tok * (tok // 2) * d
    report("(1) ZeRO-3 gather + block forward (first GEMM fused with the gather)", [tok, d, f], t_f, t_s, flops,
           (W - 1) * part * 2, {"fused_kernel_ran": ran_fused,
                                "host_ahead_ms": {"fused": round(t_f_ahead, 4), "split": round(t_s_ahead, 4),
                                                  "compute_only": round(t_res_ahead, 4),
                                                  "note": "same measurement with the device kept busy while the block is "
                                                          "enqueued (backward of a training step); fused_ms / split_ms are "
                                                          "cold starts where the host-side cost of enqueueing shows"},
                                "host_enqueue_ms": {"fused": round(host_f, 4), "split": round(host_s, 4)},
                                "kernel_stats": stats1, "compute_only_ms": round(t_res, 4),
                                "roofline_note": "roofline uses max(link time, arithmetic); compute_only_ms is the same "
                                                 "block with resident parameters"})
    rt.check()
    bmt.synchronize()
    if rank == 0:
        print(json.dumps({"summary": rows}))
    bmt.shutdown()


if __name__ == "__main__":
    main()
