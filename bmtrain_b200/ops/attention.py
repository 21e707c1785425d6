"""Multi-head attention core: ``softmax(scale * Q K^T + mask) V``.

The reference example materialises the scores with two ``bmm`` calls and a
``(b, S, S)`` boolean mask (``example/layers/attention.py:78-104``).  Here the
two contractions run as batched tcgen05 GEMMs straight on the strided
``(b, s, heads, dim)`` views (no permute/contiguous copies) and the masked
softmax -- causal flag, per-sample key lengths and/or a dense boolean mask --
is one fused in-place kernel; backward uses the same GEMM kernel in its NT /
NN / TN forms plus one fused ``dS = P * (dP - rowsum(dP * P))`` kernel.
Grouped-query attention is supported (``kv heads`` divides ``heads``).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

from . import _native

_DT = {torch.float16: 0, torch.bfloat16: 1}


def _reference_attention(q, k, v, scale, causal, mask, kv_lens):
    b, sq, h, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    if hk != h:
        k = k.repeat_interleave(h // hk, dim=2)
        v = v.repeat_interleave(h // hk, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), k.float()) * scale
    keep = torch.ones(b, 1, sq, sk, dtype=torch.bool, device=q.device)
    if causal:
        keep = keep & torch.ones(sq, sk, dtype=torch.bool, device=q.device).tril(sk - sq)
    if mask is not None:
        keep = keep & mask.view(b, 1, sq, sk)
    if kv_lens is not None:
        keep = keep & (torch.arange(sk, device=q.device)[None, None, None, :] < kv_lens.view(b, 1, 1, 1))
    s = s.masked_fill(~keep, float("-inf"))
    p = torch.softmax(s, dim=-1)
    p = torch.where(keep, p, torch.zeros_like(p))
    p = torch.nan_to_num(p, nan=0.0)
    return torch.einsum("bhqk,bkhd->bqhd", p, v.float()).to(q.dtype)


def _softmax_args(mask, kv_lens):
    m = None if mask is None else mask.to(torch.uint8).contiguous()
    l = None if kv_lens is None else kv_lens.to(torch.int32).contiguous()
    return m, l


class AttentionFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, causal, mask, kv_lens):
        lib = _native.cuda_lib()
        b, sq, h, d = q.shape
        sk, hk = k.shape[1], k.shape[2]
        assert h % hk == 0 and q.stride(3) == 1 and k.stride(3) == 1 and v.stride(3) == 1
        group = h // hk
        # scores (b, h, sq, sk): batch inner = head (kv head = head // group), outer = sample
        assert d % 8 == 0, "head dimension must be a multiple of 8"
        skp = (sk + 7) // 8 * 8  # row pitch keeps every row 16-byte aligned for TMA
        p = torch.empty(b, h, sq, skp, dtype=q.dtype, device=q.device)[..., :sk]
        _bgemm_heads(lib, "nt", sq, sk, d, q, k, p, b, h, group, scale)
        m8, l32 = _softmax_args(mask, kv_lens)
        _native.check(lib.bmt_masked_softmax(
            ctypes.c_int64(b), ctypes.c_int64(h), ctypes.c_int64(sq), ctypes.c_int64(sk), ctypes.c_int64(p.stride(2)), _native.ptr(p),
            ctypes.c_int(_DT[q.dtype]), ctypes.c_int(1 if causal else 0), _native.ptr(m8), _native.ptr(l32),
            _native.stream_handle()), "masked softmax kernel")
        o = torch.empty(b, sq, h, d, dtype=q.dtype, device=q.device)
        _bgemm_heads(lib, "pv", sq, d, sk, p, v, o, b, h, group, 1.0)
        ctx.save_for_backward(q, k, v, p)
        ctx.scale, ctx.group = scale, group
        return o

    @staticmethod
    def backward(ctx, do):
        lib = _native.cuda_lib()
        q, k, v, p = ctx.saved_tensors
        b, sq, h, d = q.shape
        sk, hk = k.shape[1], k.shape[2]
        group = ctx.group
        do = do.contiguous()
        # dP = dO V^T
        dp = torch.empty(b, h, sq, p.stride(2), dtype=p.dtype, device=p.device)[..., :sk]
        _bgemm_heads(lib, "nt", sq, sk, d, do, v, dp, b, h, group, 1.0)
        # dS = P * (dP - rowsum(dP * P)) * scale   (in place into dp)
        _native.check(lib.bmt_softmax_bwd(
            ctypes.c_int64(b * h * sq), ctypes.c_int64(sk), ctypes.c_int64(p.stride(2)), _native.ptr(p), _native.ptr(dp), ctypes.c_float(ctx.scale),
            ctypes.c_int(_DT[q.dtype]), _native.stream_handle()), "softmax backward kernel")
        dq = torch.empty(b, sq, h, d, dtype=q.dtype, device=q.device)
        _bgemm_heads(lib, "pv", sq, d, sk, dp, k, dq, b, h, group, 1.0)          # dQ = dS K
        if group == 1:
            dk = torch.empty(b, sk, h, d, dtype=q.dtype, device=q.device)
            dv = torch.empty(b, sk, h, d, dtype=q.dtype, device=q.device)
            _bgemm_heads(lib, "tn", sk, d, sq, dp, q, dk, b, h, 1, 1.0)          # dK = dS^T Q
            _bgemm_heads(lib, "tn", sk, d, sq, p, do, dv, b, h, 1, 1.0)          # dV = P^T dO
        else:
            dk_full = torch.empty(b, sk, h, d, dtype=q.dtype, device=q.device)
            dv_full = torch.empty(b, sk, h, d, dtype=q.dtype, device=q.device)
            _bgemm_heads(lib, "tn", sk, d, sq, dp, q, dk_full, b, h, 1, 1.0)
            _bgemm_heads(lib, "tn", sk, d, sq, p, do, dv_full, b, h, 1, 1.0)
            dk = dk_full.view(b, sk, hk, group, d).float().sum(3).to(q.dtype)
            dv = dv_full.view(b, sk, hk, group, d).float().sum(3).to(q.dtype)
        return dq, dk, dv, None, None, None, None


def _bgemm_heads(lib, kind, m, n, kdim, a, b_, c, batch, heads, group, alpha):
    """The three batched forms used by attention.

    kind "nt": a (b, m, h, kdim) strided, b (b, n, hk, kdim) strided  -> c (b, h, m, n)
    kind "pv": a (b, h, m, kdim) dense,   b (b, kdim, hk, n) strided  -> c (b, m, h, n)
    kind "tn": a (b, h, kdim, m) dense,   b (b, kdim, h, n) strided   -> c (b, m, h, n)
    """
    if kind == "nt":
        a_ld, a_bs = a.stride(1), (a.stride(2), a.stride(0))
        b_ld, b_bs = b_.stride(1), (b_.stride(2), b_.stride(0))
        c_ld, c_bs = c.stride(2), (c.stride(1), c.stride(0))
        a_major, b_major = 0, 0
    elif kind == "pv":
        a_ld, a_bs = a.stride(2), (a.stride(1), a.stride(0))
        b_ld, b_bs = b_.stride(1), (b_.stride(2), b_.stride(0))
        c_ld, c_bs = c.stride(1), (c.stride(2), c.stride(0))
        a_major, b_major = 0, 1
    else:
        a_ld, a_bs = a.stride(2), (a.stride(1), a.stride(0))
        b_ld, b_bs = b_.stride(1), (b_.stride(2), b_.stride(0))
        c_ld, c_bs = c.stride(1), (c.stride(2), c.stride(0))
        a_major, b_major = 1, 1
    od = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[c.dtype]
    _native.check(lib.bmt_gemm_batched(
        ctypes.c_int64(m), ctypes.c_int64(n), ctypes.c_int64(kdim),
        _native.ptr(a), ctypes.c_int64(a_ld), ctypes.c_int(a_major), ctypes.c_int64(a_bs[0]), ctypes.c_int64(a_bs[1]),
        _native.ptr(b_), ctypes.c_int64(b_ld), ctypes.c_int(b_major), ctypes.c_int64(b_bs[0]), ctypes.c_int64(b_bs[1]),
        _native.ptr(c), ctypes.c_int64(c_ld), ctypes.c_int(od), ctypes.c_int64(c_bs[0]), ctypes.c_int64(c_bs[1]),
        ctypes.c_int64(heads), ctypes.c_int64(batch), ctypes.c_int64(group if kind != "tn" else 1),
        ctypes.c_float(alpha), ctypes.c_int(_DT[a.dtype]), _native.stream_handle()), "batched tcgen05 GEMM")


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: Optional[float] = None, causal: bool = False,
              mask: Optional[torch.Tensor] = None, kv_lens: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``q`` (b, sq, h, d), ``k``/``v`` (b, sk, hk, d) with ``hk | h``; returns (b, sq, h, d).

    ``mask``: optional boolean (b, sq, sk), True = attend.  ``kv_lens``: optional (b,) valid key counts.
    Fully masked rows give zeros.
    """
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    if not q.is_cuda:
        return _reference_attention(q, k, v, scale, causal, mask, kv_lens)
    return AttentionFunction.apply(q, k, v, scale, causal, mask, kv_lens)
