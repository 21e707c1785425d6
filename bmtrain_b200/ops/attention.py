"""Multi-head attention core: ``softmax(scale * Q K^T + mask) V``.

The reference example materialises the scores with two ``bmm`` calls and a
``(b, S, S)`` boolean mask (``example/layers/attention.py:78-104``).  Here the
forward pass is one fused tcgen05 kernel (``csrc/attn_sm100.cu``): scores and
probabilities stay in tensor memory / shared memory, only the output and one
log-sum-exp per row reach HBM.  Causal flag, per-sample key lengths and a
dense boolean mask are applied inside the kernel; grouped-query attention is
supported (``kv heads`` divides ``heads``).  Head dims that the fused kernel
does not take (not a multiple of 16, or above 128) use the two-GEMM form:
batched tcgen05 GEMMs on the strided ``(b, s, heads, dim)`` views plus a fused
masked-softmax kernel, with a backward built from the same pieces (NT / NN / TN
GEMMs and one fused ``dS = P * (dP - rowsum(dP * P))`` kernel).  The fused
backward recomputes the probabilities per 128 x 128 tile from q, k and the
saved log-sum-exp and accumulates dK / dV in tensor memory.
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


def _strides3(t):
    """{token, head, batch} element strides of a (b, s, h, d) tensor as a ctypes array."""
    return (ctypes.c_int64 * 3)(t.stride(1), t.stride(2), t.stride(0))


def flash_usable(q, k, v) -> bool:
    """Whether the fused kernel takes these operands (shape/stride rules of ``bmt_flash_attn_fwd``)."""
    import os

    d = q.shape[-1]
    if os.environ.get("BMT_FLASH_ATTN", "1") == "0" or d % 16 or d > 128 or q.dtype not in _DT:
        return False
    for t in (q, k, v):
        if t.stride(3) != 1 or t.data_ptr() % 16 or any(t.stride(i) % 8 for i in range(3)):
            return False
    return True


def flash_forward(q, k, v, scale, causal, mask8, lens32):
    """Fused forward: returns ``(o (b, sq, h, d), lse (b, h, sq) fp32)``."""
    lib = _native.cuda_lib()
    b, sq, h, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    o = torch.empty(b, sq, h, d, dtype=q.dtype, device=q.device)
    lse = torch.empty(b, h, sq, dtype=torch.float32, device=q.device)
    _native.check(lib.bmt_flash_attn_fwd(
        ctypes.c_int64(b), ctypes.c_int64(sq), ctypes.c_int64(sk), ctypes.c_int(h), ctypes.c_int(hk), ctypes.c_int(d),
        _native.ptr(q), _strides3(q), _native.ptr(k), _strides3(k), _native.ptr(v), _strides3(v), _native.ptr(o), _strides3(o),
        _native.ptr(lse), ctypes.c_float(scale), ctypes.c_int(1 if causal else 0), _native.ptr(mask8), _native.ptr(lens32),
        ctypes.c_int(_DT[q.dtype]), _native.stream_handle()), "fused attention forward")
    return o, lse


def flash_backward(q, k, v, o, lse, do, scale, causal, mask8, lens32):
    """Fused backward: returns ``(dq, dk, dv)`` shaped like ``q, k, v`` (contiguous)."""
    lib = _native.cuda_lib()
    b, sq, h, d = q.shape
    sk, hk = k.shape[1], k.shape[2]
    dq = torch.empty(b, sq, h, d, dtype=q.dtype, device=q.device)
    dk = torch.empty(b, sk, hk, d, dtype=q.dtype, device=q.device)
    dv = torch.empty(b, sk, hk, d, dtype=q.dtype, device=q.device)
    dq_acc = torch.empty(b * sq * h * d, dtype=torch.float32, device=q.device)
    delta = torch.empty(b * h * sq, dtype=torch.float32, device=q.device)
    _native.check(lib.bmt_flash_attn_bwd(
        ctypes.c_int64(b), ctypes.c_int64(sq), ctypes.c_int64(sk), ctypes.c_int(h), ctypes.c_int(hk), ctypes.c_int(d),
        _native.ptr(q), _strides3(q), _native.ptr(k), _strides3(k), _native.ptr(v), _strides3(v), _native.ptr(o), _strides3(o),
        _native.ptr(do), _strides3(do), _native.ptr(lse), _native.ptr(dq), _strides3(dq), _native.ptr(dk), _strides3(dk),
        _native.ptr(dv), _strides3(dv), _native.ptr(dq_acc), _native.ptr(delta), ctypes.c_float(scale),
        ctypes.c_int(1 if causal else 0), _native.ptr(mask8), _native.ptr(lens32), ctypes.c_int(_DT[q.dtype]),
        _native.stream_handle()), "fused attention backward")
    return dq, dk, dv


def _softmax_args(mask, kv_lens):
    m = None if mask is None else (mask.contiguous().view(torch.uint8) if mask.dtype == torch.bool else mask.to(torch.uint8).contiguous())
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
        m8, l32 = _softmax_args(mask, kv_lens)
        ctx.scale, ctx.group, ctx.causal = scale, group, causal
        if flash_usable(q, k, v):
            o, lse = flash_forward(q, k, v, scale, causal, m8, l32)
            # nothing of size sq x sk is kept: backward rebuilds the probabilities tile by tile from q, k and lse
            ctx.save_for_backward(q, k, v, o, lse, m8, l32)
            ctx.fused = True
            return o
        assert d % 8 == 0, "head dimension must be a multiple of 8"
        p = AttentionFunction._probabilities(lib, q, k, scale, causal, m8, l32, group)
        o = torch.empty(b, sq, h, d, dtype=q.dtype, device=q.device)
        _bgemm_heads(lib, "pv", sq, d, sk, p, v, o, b, h, group, 1.0)
        ctx.save_for_backward(q, k, v, p)
        ctx.fused = False
        return o

    @staticmethod
    def _probabilities(lib, q, k, scale, causal, m8, l32, group):
        """(b, h, sq, sk) masked softmax of the scaled scores (row pitch padded to 8 elements for TMA)."""
        b, sq, h, d = q.shape
        sk = k.shape[1]
        skp = (sk + 7) // 8 * 8
        p = torch.empty(b, h, sq, skp, dtype=q.dtype, device=q.device)[..., :sk]
        _bgemm_heads(lib, "nt", sq, sk, d, q, k, p, b, h, group, scale)
        _native.check(lib.bmt_masked_softmax(
            ctypes.c_int64(b), ctypes.c_int64(h), ctypes.c_int64(sq), ctypes.c_int64(sk), ctypes.c_int64(p.stride(2)), _native.ptr(p),
            ctypes.c_int(_DT[q.dtype]), ctypes.c_int(1 if causal else 0), _native.ptr(m8), _native.ptr(l32),
            _native.stream_handle()), "masked softmax kernel")
        return p

    @staticmethod
    def backward(ctx, do):
        lib = _native.cuda_lib()
        if ctx.fused:
            q, k, v, o, lse, m8, l32 = ctx.saved_tensors
            do = do.contiguous()
            if do.data_ptr() % 16:
                do = do.clone()
            dq, dk, dv = flash_backward(q, k, v, o, lse, do, ctx.scale, ctx.causal, m8, l32)
            return dq, dk, dv, None, None, None, None
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
