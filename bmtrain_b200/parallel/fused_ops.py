"""Python side of the fused tensor-parallel kernels (``csrc/gemm_sm100.cu``, FusedComm modes 1 and 2).

Buffers that peers write into (the reduce-scatter inbox, the gathered activation matrix and its arrival counters) are
symmetric buffers of the communicator's :class:`~bmtrain_b200.parallel.symm.PeerRuntime`, keyed by problem shape and
used as a ring of two, so that a call may start while the previous result is still being consumed.  Each call takes
one epoch on its flag rows; "free" (this rank's buffer may be overwritten) is published by the kernel when it starts,
i.e. after everything queued earlier on the stream has finished.

A gathered matrix returned by :func:`ag_gemm` aliases ring memory: it is valid until the second following call with
the same shape.
"""
from __future__ import annotations

import ctypes
import os
from typing import Dict, Optional, Tuple

import torch

from ..comm import Communicator
from ..ops import _native
from ..ops.gpt_block import _i64, _int, _f32, _c_void_p
from . import symm

_COMM_CTAS = int(os.environ.get("BMT_COMM_CTAS", "0"))  # 0: balance math and transfer per call (bmt_fused_comm_ctas)


def _comm_ctas(flops: float, push_bytes: float, remote_bytes: float) -> int:
    if _COMM_CTAS > 0:
        return _COMM_CTAS
    lib = _native.cuda_lib()
    return int(lib.bmt_fused_comm_ctas(ctypes.c_double(flops), ctypes.c_double(push_bytes), ctypes.c_double(remote_bytes)))
calls = {"gemm_rs": 0, "ag_gemm": 0, "zero_gather_gemm": 0}  # how often each fused kernel ran (tests and benchmarks read this)


class _GemmDesc(ctypes.Structure):
    _fields_ = [
        ("m", _i64), ("n", _i64), ("k", _i64),
        ("a", _c_void_p), ("lda", _i64), ("a_major", _int), ("a_bs0", _i64), ("a_bs1", _i64),
        ("b", _c_void_p), ("ldb", _i64), ("b_major", _int), ("b_bs0", _i64), ("b_bs1", _i64),
        ("c", _c_void_p), ("ldc", _i64), ("c_dtype", _int), ("c_bs0", _i64), ("c_bs1", _i64),
        ("batch_inner", _i64), ("batch_outer", _i64), ("b_inner_div", _i64),
        ("bias", _c_void_p), ("act", _int), ("accumulate", _int), ("alpha", _f32), ("ab_dtype", _int),
        ("residual", _c_void_p), ("ldr", _i64), ("aux", _c_void_p), ("ld_aux", _i64), ("aux_mode", _int),
    ]


_DT = {torch.float16: 0, torch.bfloat16: 1}


def kernel_stats() -> dict:
    """Device-side timing of the fused GEMM kernels launched since the last call (cleared by reading; host sync)."""
    out = (ctypes.c_ulonglong * 8)()
    _native.check(_native.cuda_lib().bmt_fused_stats(out), "fused kernel statistics")
    n = max(int(out[4]), 1)
    return {"kernels": int(out[4]), "producer_wait_us_sum": out[0] / 1e3, "producer_wait_us_max": out[3] / 1e3,
            "pusher_us_max": out[1] / 1e3, "cta_us_max": out[2] / 1e3, "producer_wait_us_per_kernel": out[0] / 1e3 / n,
            "rs_wait_us_max": out[5] / 1e3, "rs_total_us_max": out[6] / 1e3, "rs_wait_us_sum": out[7] / 1e3}


_reserved = [None]


def _reserve_sms() -> None:
    """When kernels of another parallel dimension run next to the fused ones (``symm.no_spin``), the fused grids leave
    ``BMT_RESERVED_SMS`` SMs (default 16) free: their CTAs hold an SM while they wait for rows of another rank, and an NCCL
    gather of the ZeRO group that cannot start on this rank keeps a rank of another pair waiting -- a cycle over pairs
    and groups that only the bounded waits would break.  (NCCL's own grid can be capped to fit with ``NCCL_MAX_CTAS``.)"""
    want = int(os.environ.get("BMT_RESERVED_SMS", "16")) if symm.no_spin() else 0
    if _reserved[0] != want:
        _native.cuda_lib().bmt_gemm_reserve_sms(ctypes.c_int(want))
        _reserved[0] = want


def _next_parity(rt, key: Tuple) -> int:
    # ring positions and grid counters belong to the runtime: they start over together with its epochs when the
    # process group is torn down and set up again, and two communicators never share them
    ring = rt.cache.setdefault(("ring",), {})
    ring[key] = (ring.get(key, -1) + 1) % 2
    return ring[key]


def _grid_counter(rt, key: Tuple, device) -> torch.Tensor:
    table = rt.cache.setdefault(("grid_counters",), {})
    if key not in table:
        table[key] = torch.zeros(2, dtype=torch.int32, device=device)
    return table[key]


def _tma_ready(t: torch.Tensor) -> torch.Tensor:
    """``t`` in a layout the TMA descriptors accept (row-major, 16-byte aligned rows).  Whether the fused kernel is
    used must not depend on a rank-local property such as a pointer or a stride -- a rank that fell back alone would
    leave its peers waiting -- so a non-conforming operand is copied instead of being a reason to fall back."""
    if t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0:
        return t
    return t.contiguous().clone() if t.is_contiguous() else t.contiguous()


def gemm_rs(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], comm: Communicator, b_is_kn: bool) -> Optional[torch.Tensor]:
    """``reduce_scatter_rows(x @ W^T)`` (+ bias) in one kernel; None when the shapes do not fit the fused kernel."""
    rt = symm.peer_runtime(comm)
    M, K = x.shape
    N = weight.shape[1] if b_is_kn else weight.shape[0]
    W = comm.size
    if rt is None or x.dtype not in _DT or M % W or N % 8 or K % 8:
        return None
    x, weight = _tma_ready(x), _tma_ready(weight)
    lib = _native.cuda_lib()
    _reserve_sms()
    rows = M // W
    es = x.element_size()
    base = ("rs", M, N, K, x.dtype, b_is_kn)
    key = base + (_next_parity(rt, base),)
    inbox = rt.slot(key, W * rows * N * es)
    free_row, done_row = rt.row(key + ("free",)), rt.row(key + ("done",))
    epoch = rt.next_epoch(free_row)
    rt.epochs[done_row] = epoch
    grid_counter = _grid_counter(rt, key, x.device)
    out = torch.empty(rows, N, dtype=x.dtype, device=x.device)
    d = _GemmDesc()
    d.m, d.n, d.k = M, N, K
    d.a, d.lda, d.a_major = x.data_ptr(), x.stride(0), 0
    d.b, d.ldb, d.b_major = weight.data_ptr(), weight.stride(0), 1 if b_is_kn else 0
    d.ab_dtype, d.alpha = _DT[x.dtype], 1.0
    slots = (ctypes.c_void_p * W)(*[p + comm.rank * rows * N * es for p in inbox.ptrs])
    if symm.no_spin():
        # deliver / wait / sum as three launches (see symm.no_spin)
        if epoch == 1:
            rt.signal_wait(free_row, 1, signal=True, wait=False)
        _native.check(lib.bmt_gemm_reduce_scatter_main(
            ctypes.byref(d), ctypes.c_int(W), ctypes.c_int(comm.rank), rt.flag_ptrs, ctypes.c_int(free_row), ctypes.c_int(done_row),
            ctypes.c_uint(epoch), slots, ctypes.c_void_p(inbox.local_ptr), ctypes.c_int64(rows), _native.ptr(grid_counter),
            _native.ptr(rt.status), ctypes.c_double(rt.timeout_s), _native.stream_handle()), "GEMM -> reduce-scatter, deliver kernel")
        rt.signal_wait(done_row, epoch, signal=False, wait=True)
        _native.check(lib.bmt_gemm_rs_reduce(
            ctypes.c_void_p(inbox.local_ptr), ctypes.c_int64(rows), ctypes.c_int64(N), ctypes.c_int(W), ctypes.c_int(comm.rank),
            rt.flag_ptrs, ctypes.c_int(free_row), ctypes.c_uint(epoch), _native.ptr(grid_counter), _native.ptr(out), _native.ptr(bias),
            ctypes.c_int(_DT[x.dtype]), _native.stream_handle()), "GEMM -> reduce-scatter, sum kernel")
        calls["gemm_rs"] += 1
        return out
    _native.check(lib.bmt_gemm_reduce_scatter(
        ctypes.byref(d), ctypes.c_int(W), ctypes.c_int(comm.rank), rt.flag_ptrs, ctypes.c_int(free_row), ctypes.c_int(done_row),
        ctypes.c_uint(epoch), slots, ctypes.c_void_p(inbox.local_ptr), ctypes.c_int64(rows), _native.ptr(grid_counter),
        _native.ptr(out), _native.ptr(bias), _native.ptr(rt.status), ctypes.c_double(rt.timeout_s), _native.stream_handle()),
        "fused GEMM -> reduce-scatter kernel")
    calls["gemm_rs"] += 1
    return out


def ag_gemm(x_local: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], comm: Communicator, b_is_kn: bool,
            return_gathered: bool):
    """``all_gather_rows(x_local) @ W^T`` in one kernel; None when the shapes do not fit the fused kernel."""
    rt = symm.peer_runtime(comm)
    m, K = x_local.shape
    N = weight.shape[1] if b_is_kn else weight.shape[0]
    W = comm.size
    if rt is None or x_local.dtype not in _DT or m % 128 or K % 8 or N % 8:
        return None
    weight = _tma_ready(weight)
    if not x_local.is_contiguous() or x_local.data_ptr() % 16:
        x_local = x_local.contiguous()  # the pushers copy flat 32 KiB pieces
    lib = _native.cuda_lib()
    _reserve_sms()
    es = x_local.element_size()
    # everything that decides how the pushers cut the rows (pusher count, runs per block) has to be constant per key: the
    # per-block counters on the peers grow by the same amount every time the key's buffers are used
    base = ("ag", m, K, N, x_local.dtype, b_is_kn)
    key = base + (_next_parity(rt, base),)
    gathered = rt.slot(key, W * m * K * es)
    counters = rt.slot(key + ("cnt",), max(256, W * (m // 128) * 4))
    free_row = rt.row(key + ("free",))
    epoch = rt.next_epoch(free_row)
    out = torch.empty(W * m, N, dtype=x_local.dtype, device=x_local.device)
    d = _GemmDesc()
    d.m, d.n, d.k = W * m, N, K
    d.a, d.lda, d.a_major = gathered.local_ptr, K, 0
    d.b, d.ldb, d.b_major = weight.data_ptr(), weight.stride(0), 1 if b_is_kn else 0
    d.c, d.ldc, d.c_dtype = out.data_ptr(), N, _DT[x_local.dtype]
    d.bias = None if bias is None else bias.data_ptr()
    d.ab_dtype, d.alpha = _DT[x_local.dtype], 1.0
    # this rank's own rows go into place with a device-to-device copy (far faster than the pusher CTAs, which then only
    # serve the peers); the kernel does not wait for them
    mine = gathered.tensor(x_local.dtype, m * K, comm.rank * m * K * es).view(m, K)
    mine.copy_(x_local)
    ctas = _comm_ctas(2.0 * W * m * N * K, float((W - 1) * m * K * es), float((W - 1) * m * K * es))
    _native.check(lib.bmt_all_gather_gemm(
        ctypes.byref(d), ctypes.c_int(W), ctypes.c_int(comm.rank), rt.flag_ptrs, ctypes.c_int(free_row), ctypes.c_uint(epoch),
        _native.ptr(x_local), ctypes.c_int64(x_local.stride(0)), ctypes.c_int64(m), gathered.ptr_table(), counters.ptr_table(),
        ctypes.c_int(ctas), ctypes.c_int(1), _native.ptr(rt.status), ctypes.c_double(rt.timeout_s), _native.stream_handle()),
        "fused all-gather -> GEMM kernel")
    calls["ag_gemm"] += 1
    if return_gathered:
        return out, gathered.tensor(x_local.dtype, W * m * K).view(W * m, K)
    return out


def zero_gather_gemm(x: torch.Tensor, out: torch.Tensor, bias: Optional[torch.Tensor], ctx: dict) -> None:
    """``out = x @ W^T + bias`` where ``W`` is a ZeRO-sharded weight that nobody has gathered yet: the kernel's pusher
    CTAs deliver every rank's part of ``W`` to all ranks while the tiles whose rows have arrived are already being
    multiplied (``ctx`` comes from ``Block._try_deferred_gather``)."""
    lib = _native.cuda_lib()
    rt, buf, b, slot, epoch, key = ctx["rt"], ctx["buf"], ctx["bucket"], ctx["slot"], ctx["epoch"], ctx["key"]
    N, K = slot.shape
    W = b.comm.size
    es = x.element_size()
    w0, w1 = slot.offset, slot.offset + slot.numel
    geo = rt.cache.get(key + ("geo",))
    if geo is None:
        first = (ctypes.c_int64 * W)()
        count = (ctypes.c_int64 * W)()
        for j in range(W):
            lo, hi = max(w0, j * b.part), min(w1, (j + 1) * b.part)
            first[j], count[j] = max(lo - w0, 0), max(hi - lo, 0)
        chunks = (N + 127) // 128
        # the number of pusher CTAs decides how the pushes are cut, so every rank has to pick the same one: agree on the
        # largest token count (first use only; host sync)
        rows = torch.tensor([x.shape[0]], dtype=torch.int64, device=x.device)
        b.comm.all_reduce(rows, "max")
        ctas = _comm_ctas(2.0 * int(rows.item()) * N * K, float((W - 1) * max(count) * es), float((W - 1) * max(count) * es))
        exp_host = (ctypes.c_uint * chunks)()
        others = (ctypes.c_int64 * W)(*[0 if j == b.comm.rank else count[j] for j in range(W)])  # the own part is copied, not pushed
        lib.bmt_zero_gather_expected(ctypes.c_int64(N), ctypes.c_int64(K), ctypes.c_int(W), first, others, ctypes.c_int(ctas), exp_host)
        expected = torch.tensor(list(exp_host), dtype=torch.int32, device=x.device)
        counters = rt.slot(key + ("cnt",), max(256, chunks * 4))
        geo = dict(first=list(first), count=list(count), expected=expected, ctas=ctas, counters=counters.ptr_table(),
                   weight_on_rank=(ctypes.c_void_p * W)(*[p + w0 * es for p in buf.ptrs]), buf=buf)
        rt.cache[key + ("geo",)] = geo
    if geo["buf"] is not buf:   # the ring slot was reallocated
        geo["weight_on_rank"] = (ctypes.c_void_p * W)(*[p + w0 * es for p in buf.ptrs])
        geo["buf"] = buf
    first, count = geo["first"], geo["count"]
    d = _GemmDesc()
    d.m, d.n, d.k = x.shape[0], N, K
    d.a, d.lda, d.a_major = x.data_ptr(), x.stride(0), 0
    d.b, d.ldb, d.b_major = buf.local_ptr + w0 * es, K, 0
    d.c, d.ldc, d.c_dtype = out.data_ptr(), out.stride(0), _DT[x.dtype]
    d.bias = None if bias is None else bias.data_ptr()
    d.ab_dtype, d.alpha = _DT[x.dtype], 1.0
    me = b.comm.rank
    src = b.storage.data_ptr() + (w0 + first[me] - b.begin) * es if count[me] > 0 else b.storage.data_ptr()
    if count[me] > 0:
        # own part: plain device-to-device copy into this rank's gathered buffer; the pusher CTAs only serve the peers
        lo = w0 + first[me]
        buf.tensor(x.dtype, count[me], lo * es).copy_(b.storage.data[lo - b.begin:lo - b.begin + count[me]])
    _native.check(lib.bmt_zero_gather_gemm(
        ctypes.byref(d), ctypes.c_int(W), ctypes.c_int(me), rt.flag_ptrs, ctypes.c_int(ctx["free_row"]), ctypes.c_uint(epoch),
        ctypes.c_void_p(src), ctypes.c_int64(first[me]), ctypes.c_int64(count[me]), geo["weight_on_rank"], geo["counters"],
        _native.ptr(geo["expected"]), ctypes.c_int(geo["ctas"]), ctypes.c_int(1), _native.ptr(rt.status), ctypes.c_double(rt.timeout_s),
        _native.stream_handle()), "fused ZeRO gather -> GEMM kernel")
    calls["zero_gather_gemm"] += 1
