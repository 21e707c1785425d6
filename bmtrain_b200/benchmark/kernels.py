"""Single-GPU kernel micro-benchmarks against the measured roofline.

    python -m bmtrain_b200.benchmark.kernels --op gemm --m 8192 --n 8192 --k 8192 --dtype bf16 --layout nt
    python -m bmtrain_b200.benchmark.kernels --op gemm_block_shapes      # the 15 GEMMs of the benchmark block vs the library
    python -m bmtrain_b200.benchmark.kernels --op adam --n 268435456
    python -m bmtrain_b200.benchmark.kernels --op norm|ce|softmax ...
    python -m bmtrain_b200.benchmark.kernels --op attention --batch 2 --seq 4096 --heads 20 --kv-heads 20 --head-dim 128

Timing: CUDA events on the launching stream, 3 warm-up launches, a >L2 buffer is rewritten between timed launches
(``--flush``, default on) so every launch starts with a cold L2.  Peaks come from ``MEASURED_PEAKS.json`` at the
repository root when present (fallback: 6.65 TB/s, 1.59 PFLOP/s).
"""
from __future__ import annotations

import argparse
import json
import os

import torch

_ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks():
    try:
        with open(os.path.join(_ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return p["hbm_gbs"], p["bf16_tflops"], "measured"
    except (OSError, KeyError, ValueError):
        return 6650.0, 1590.0, "fallback"


def time_it(fn, iters: int, flush: bool) -> float:
    scratch = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    total = 0.0
    for _ in range(iters):
        if scratch is not None:
            scratch.fill_(1)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        total += s.elapsed_time(e)
    return total / iters


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--op", default="gemm", choices=["gemm", "gemm_block_shapes", "adam", "norm", "norm_bwd", "rmsnorm", "ce", "ce_bwd", "softmax", "softmax_bwd", "embedding",
                                                  "embedding_bwd", "infnan", "sqnorm", "colsum", "rope", "swiglu", "attention"])
    ap.add_argument("--batch", type=int, default=2)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=20)
    ap.add_argument("--kv-heads", type=int, default=0)
    ap.add_argument("--head-dim", type=int, default=128)
    ap.add_argument("--no-causal", action="store_true")
    ap.add_argument("--fwd-only", action="store_true", help="attention: time the fused forward kernel alone (for ncu captures)")
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16"])
    ap.add_argument("--layout", default="nt", choices=["nt", "nn", "tn"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--no-flush", action="store_true")
    ap.add_argument("--compare-library", action="store_true", help="gemm: also time torch.matmul (cuBLAS) on the same operands")
    args = ap.parse_args()
    dt = torch.bfloat16 if args.dtype == "bf16" else torch.float16
    hbm, tflops, src = peaks()
    from bmtrain_b200.ops import adam as A, cross_entropy as CE, gemm as G, norm as N

    flush = not args.no_flush
    dev = "cuda"
    if args.op == "gemm":
        m, n, k = args.m, args.n, args.k
        if args.layout == "nt":
            a, b = torch.randn(m, k, device=dev, dtype=dt), torch.randn(n, k, device=dev, dtype=dt)
            fn = lambda: G.gemm_nt(a, b)
        elif args.layout == "nn":
            a, b = torch.randn(m, k, device=dev, dtype=dt), torch.randn(k, n, device=dev, dtype=dt)
            fn = lambda: G.gemm_nn(a, b)
        else:
            a, b = torch.randn(k, m, device=dev, dtype=dt), torch.randn(k, n, device=dev, dtype=dt)
            fn = lambda: G.gemm_tn(a, b)
        ms = time_it(fn, args.iters, flush)
        ach = 2.0 * m * n * k / ms / 1e9
        out = {"op": f"gemm_{args.layout}", "m": m, "n": n, "k": k, "dtype": args.dtype, "ms": ms,
               "tflops": ach, "frac_of_peak": ach / tflops, "peak_source": src}
        if args.compare_library:
            # the library GEMM (cuBLAS through torch.matmul) on the same operands: a yardstick, never on a product path
            lib_fn = {"nt": lambda: torch.matmul(a, b.t()), "nn": lambda: torch.matmul(a, b), "tn": lambda: torch.matmul(a.t(), b)}[args.layout]
            lib_ms = time_it(lib_fn, args.iters, flush)
            out.update({"library_ms": lib_ms, "vs_library": lib_ms / ms})
        print(json.dumps(out))
    elif args.op == "gemm_block_shapes":
        # forward / dgrad / wgrad GEMMs of one block of the headline model (GPT d2560, FFN 8192, vocab 10240) at --m tokens
        # (default here: 1024 = batch 2 x 512), each as 20 back-to-back launches in a CUDA graph (launch gaps excluded, L2
        # warm: weights of one GEMM fit), against torch.matmul (cuBLAS) the same way
        t = args.m if args.m != 8192 else 1024
        d_, dff, voc = 2560, 8192, 10240
        shapes = [("nt", t, 3 * d_, d_), ("nt", t, d_, d_), ("nt", t, dff, d_), ("nt", t, d_, dff), ("nt", t, voc, d_),
                  ("nn", t, dff, d_), ("nn", t, d_, dff), ("nn", t, d_, d_), ("nn", t, d_, 3 * d_), ("nn", t, d_, voc),
                  ("tn", d_, dff, t), ("tn", dff, d_, t), ("tn", d_, d_, t), ("tn", 3 * d_, d_, t), ("tn", voc, d_, t)]
        side = torch.cuda.Stream()

        def graph_time(fn):
            with torch.cuda.stream(side):
                for _ in range(5):
                    fn()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(g, stream=side):
                    for _ in range(20):
                        fn()
            torch.cuda.synchronize()
            g.replay()
            torch.cuda.synchronize()
            s0, e0 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s0.record()
            g.replay()
            g.replay()
            e0.record()
            torch.cuda.synchronize()
            return s0.elapsed_time(e0) / 40

        rows, tot_ours, tot_lib = [], 0.0, 0.0
        for lay, m, n, k in shapes:
            if lay == "nt":
                a, b = torch.randn(m, k, device=dev, dtype=dt), torch.randn(n, k, device=dev, dtype=dt)
                o = torch.empty(m, n, device=dev, dtype=dt)
                f1, f2 = (lambda: G.gemm_nt(a, b, out=o)), (lambda: torch.matmul(a, b.t(), out=o))
            elif lay == "nn":
                a, b = torch.randn(m, k, device=dev, dtype=dt), torch.randn(k, n, device=dev, dtype=dt)
                o = torch.empty(m, n, device=dev, dtype=dt)
                f1, f2 = (lambda: G.gemm_nn(a, b, out=o)), (lambda: torch.matmul(a, b, out=o))
            else:
                a, b = torch.randn(k, m, device=dev, dtype=dt), torch.randn(k, n, device=dev, dtype=dt)
                o = torch.empty(m, n, device=dev, dtype=dt)
                f1, f2 = (lambda: G.gemm_tn(a, b, out=o)), (lambda: torch.matmul(a.t(), b, out=o))
            ours, libt = graph_time(f1), graph_time(f2)
            tot_ours += ours
            tot_lib += libt
            rows.append({"layout": lay, "m": m, "n": n, "k": k, "ours_us": round(ours * 1e3, 1), "library_us": round(libt * 1e3, 1),
                         "ours_tflops": round(2.0 * m * n * k / ours / 1e9), "vs_library": round(libt / ours, 3)})
        print(json.dumps({"op": "gemm_block_shapes", "tokens": t, "dtype": args.dtype, "shapes": rows,
                          "sum_ours_us": round(tot_ours * 1e3, 1), "sum_library_us": round(tot_lib * 1e3, 1),
                          "vs_library": round(tot_lib / tot_ours, 3)}))
    elif args.op == "adam":
        n = args.n
        p32 = torch.randn(n, device=dev)
        p16, g = p32.to(dt), torch.randn(n, device=dev).to(dt)
        m_ = torch.zeros(n, device=dev, dtype=torch.float16 if dt == torch.float16 else torch.float32)
        v = torch.zeros(n, device=dev)
        fn = lambda: A.adam_half_multi([(p32, p16, g, m_, v)], 0.9, 0.999, 1e-8, 1e-3, 1.0, 0.01, 3)
        ms = time_it(fn, args.iters, flush)
        nbytes = n * (2 * (4 + 2 + m_.element_size() + 4) + 2)
        print(json.dumps({"op": "adam", "n": n, "dtype": args.dtype, "ms": ms, "gbs": nbytes / ms / 1e6,
                          "frac_of_peak": nbytes / ms / 1e6 / hbm, "peak_source": src}))
    elif args.op == "norm":
        x = torch.randn(args.m, args.n, device=dev, dtype=dt)
        w, b = torch.ones(args.n, device=dev, dtype=dt), torch.zeros(args.n, device=dev, dtype=dt)
        fn = lambda: N.layer_norm(x, w, b)
        ms = time_it(fn, args.iters, flush)
        nbytes = 2 * x.numel() * 2
        print(json.dumps({"op": "layernorm_fwd", "rows": args.m, "d": args.n, "ms": ms, "gbs": nbytes / ms / 1e6,
                          "frac_of_peak": nbytes / ms / 1e6 / hbm, "peak_source": src}))
    elif args.op == "attention":
        # fused tcgen05 attention against the two-GEMM + softmax form on the same strided (packed projection) operands;
        # FLOPs: 4 s^2 d per head forward (halved under a causal mask), 2.5 x that backward
        from bmtrain_b200.ops import attention as AT

        b, s_, h, d = args.batch, args.seq, args.heads, args.head_dim
        hk = args.kv_heads or h
        g = h // hk
        causal = not args.no_causal
        packed = torch.randn(b, s_, hk, g + 2, d, device=dev, dtype=dt) * 0.5
        q = packed[:, :, :, :g].reshape(b, s_, h, d).requires_grad_()
        k = packed[:, :, :, g].clone().requires_grad_()
        v = packed[:, :, :, g + 1].clone().requires_grad_()
        flops_f = 4.0 * b * h * s_ * s_ * d * (0.5 if causal else 1.0)
        go = torch.randn(b, s_, h, d, device=dev, dtype=dt)
        res = {"op": "attention", "batch": b, "seq": s_, "heads": h, "kv_heads": hk, "head_dim": d, "causal": causal,
               "dtype": args.dtype, "peak_source": src}
        modes = (("fused", "1"),) if args.fwd_only else (("fused", "1"), ("two_gemm", "0"))
        for name, flag in modes:
            os.environ["BMT_FLASH_ATTN"] = flag
            fwd = lambda: AT.attention(q, k, v, causal=causal)
            with torch.no_grad():
                ms_f = time_it(fwd, args.iters, flush)
            res[name + "_fwd_ms"] = ms_f
            res[name + "_fwd_tflops"] = flops_f / ms_f / 1e9
            if args.fwd_only:
                continue

            def both():
                q.grad = k.grad = v.grad = None
                AT.attention(q, k, v, causal=causal).backward(go)

            ms_fb = time_it(both, args.iters, flush)
            res[name + "_fwd_bwd_ms"] = ms_fb
            res[name + "_fwd_bwd_tflops"] = 3.5 * flops_f / ms_fb / 1e9
        res["fused_fwd_frac_of_peak"] = res["fused_fwd_tflops"] / tflops
        print(json.dumps(res))
    elif args.op in ("norm_bwd", "rmsnorm", "ce_bwd", "softmax", "softmax_bwd", "embedding", "embedding_bwd", "infnan", "sqnorm",
                     "colsum", "rope", "swiglu"):
        # memory-bound kernels: achieved = algorithmic bytes / time, against the measured copy bandwidth
        import ctypes

        from bmtrain_b200.ops import _native, elementwise as EW, embedding as EMB, infnan as IN

        lib = _native.cuda_lib()
        m, n = args.m, args.n
        code = 0 if dt == torch.float16 else 1
        if args.op == "rmsnorm":
            x, w = torch.randn(m, n, device=dev, dtype=dt), torch.ones(n, device=dev, dtype=dt)
            fn, nbytes = (lambda: N.rms_norm(x, w)), 2 * x.numel() * 2
        elif args.op == "norm_bwd":
            x = torch.randn(m, n, device=dev, dtype=dt, requires_grad=True)
            w, b = torch.ones(n, device=dev, dtype=dt, requires_grad=True), torch.zeros(n, device=dev, dtype=dt, requires_grad=True)
            y = N.layer_norm(x, w, b)
            g = torch.randn_like(y)
            fn, nbytes = (lambda: torch.autograd.grad(y, (x, w, b), g, retain_graph=True)), 3 * x.numel() * 2
        elif args.op == "ce_bwd":
            x = torch.randn(m, n, device=dev, dtype=dt)
            t = torch.randint(0, n, (m,), device=dev)
            mx, se, _ = CE.row_stats(x, t)
            lse, gl = mx + se.log(), torch.ones(m, device=dev)
            out = torch.empty_like(x)
            fn, nbytes = (lambda: CE.ce_backward(x, t, lse, gl)), 2 * x.numel() * 2
        elif args.op in ("softmax", "softmax_bwd"):
            # (batch, heads, seq, seq) scores of the two-GEMM attention form
            b_, h_, s_ = args.batch, args.heads, args.seq
            p_ = torch.randn(b_, h_, s_, s_, device=dev, dtype=dt)
            dp = torch.randn_like(p_)
            if args.op == "softmax":
                fn = lambda: lib.bmt_masked_softmax(ctypes.c_int64(b_), ctypes.c_int64(h_), ctypes.c_int64(s_), ctypes.c_int64(s_),
                                                    ctypes.c_int64(s_), _native.ptr(p_), ctypes.c_int(code), ctypes.c_int(1), None, None,
                                                    _native.stream_handle())
                nbytes = 2 * p_.numel() * 2 * 0.5   # causal: about half of every row is read and written
            else:
                fn = lambda: lib.bmt_softmax_bwd(ctypes.c_int64(b_ * h_ * s_), ctypes.c_int64(s_), ctypes.c_int64(s_), _native.ptr(p_),
                                                 _native.ptr(dp), ctypes.c_float(0.1), ctypes.c_int(code), _native.stream_handle())
                nbytes = 3 * p_.numel() * 2
        elif args.op in ("embedding", "embedding_bwd"):
            w = torch.randn(n, args.k, device=dev, dtype=dt)          # (vocab, d)
            ids = torch.randint(0, n, (m,), device=dev)
            g = torch.randn(m, args.k, device=dev, dtype=dt)
            if args.op == "embedding":
                fn, nbytes = (lambda: EMB.embedding_forward(ids, w)), 2 * m * args.k * 2
            else:
                fn, nbytes = (lambda: EMB.embedding_backward(ids, g, n)), (m * args.k + n * args.k) * 2
        elif args.op in ("infnan", "sqnorm"):
            x = torch.randn(args.n, device=dev, dtype=dt)
            flag, tot = torch.zeros(1, dtype=torch.uint8, device=dev), torch.zeros(1, device=dev)
            fn = (lambda: IN.multi_has_inf_nan([x], flag)) if args.op == "infnan" else (lambda: IN.multi_sq_norm([x], tot))
            nbytes = x.numel() * 2
        elif args.op == "colsum":
            from ..ops import gemm as G
            x = torch.randn(m, n, device=dev, dtype=dt)
            fn = lambda: G.bias_grad(x)
            nbytes = x.numel() * 2
        elif args.op == "rope":
            hk = args.kv_heads or args.heads
            g_ = args.heads // hk
            packed = torch.randn(args.batch, args.seq, hk, g_ + 2, args.head_dim, device=dev, dtype=dt)
            fn, nbytes = (lambda: EW.rope_qkv(packed, g_)), 2 * packed.numel() * 2
        else:  # swiglu
            x = torch.randn(m, 2 * n, device=dev, dtype=dt)
            fn, nbytes = (lambda: EW.swiglu(x)), 3 * m * n * 2
        with torch.no_grad() if args.op != "norm_bwd" else torch.enable_grad():
            ms = time_it(fn, args.iters, flush)
        print(json.dumps({"op": args.op, "m": m, "n": n, "dtype": args.dtype, "ms": ms, "gbs": nbytes / ms / 1e6,
                          "frac_of_peak": nbytes / ms / 1e6 / hbm, "peak_source": src}))
    elif args.op == "ce":
        x = torch.randn(args.m, args.n, device=dev, dtype=dt)
        t = torch.randint(0, args.n, (args.m,), device=dev)
        fn = lambda: CE.row_stats(x, t)
        ms = time_it(fn, args.iters, flush)
        nbytes = x.numel() * 2
        print(json.dumps({"op": "ce_row_stats", "rows": args.m, "classes": args.n, "ms": ms, "gbs": nbytes / ms / 1e6,
                          "frac_of_peak": nbytes / ms / 1e6 / hbm, "peak_source": src}))


if __name__ == "__main__":
    main()
