"""Whole pre-LN GPT block as one autograd node on the native block executor (``csrc/block_exec.cu``).

Forward issues 9 kernel launches and backward 21 from C++ in a single call each, all contractions on the tcgen05
GEMM with fused epilogues (bias, ReLU, residual add, ReLU-mask on dgrad).  The big weight gradients are written
straight into ``param.grad`` when a gradient buffer of the right dtype is already attached (as the ZeRO block
does before backward), which removes the separate accumulate pass.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import torch

from . import _native
from . import gemm as _gemm

_c_void_p, _i64, _int, _f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int, ctypes.c_float


class _Block(ctypes.Structure):
    _fields_ = [
        ("batch", _i64), ("seq", _i64), ("d_model", _i64), ("n_heads", _i64), ("d_head", _i64), ("d_ff", _i64),
        ("dtype", _int), ("act", _int), ("eps", _f32), ("causal", _int), ("mask", _c_void_p),
        ("ln1_w", _c_void_p), ("ln1_b", _c_void_p), ("qkv_w", _c_void_p), ("qkv_b", _c_void_p), ("out_w", _c_void_p),
        ("out_b", _c_void_p), ("ln2_w", _c_void_p), ("ln2_b", _c_void_p), ("fc1_w", _c_void_p), ("fc1_b", _c_void_p),
        ("fc2_w", _c_void_p), ("fc2_b", _c_void_p),
        ("x", _c_void_p), ("y", _c_void_p),
        ("ln1", _c_void_p), ("stats1", _c_void_p), ("qkv", _c_void_p), ("probs", _c_void_p), ("probs_ld", _i64),
        ("ctx", _c_void_p), ("h1", _c_void_p), ("ln2", _c_void_p), ("stats2", _c_void_p), ("ff", _c_void_p), ("pre", _c_void_p),
        ("lse", _c_void_p),
    ]


class _Grad(ctypes.Structure):
    _fields_ = [
        ("dy", _c_void_p), ("dx", _c_void_p),
        ("d_ln1_w", _c_void_p), ("d_ln1_b", _c_void_p), ("d_qkv_w", _c_void_p), ("d_qkv_b", _c_void_p),
        ("d_out_w", _c_void_p), ("d_out_b", _c_void_p), ("d_ln2_w", _c_void_p), ("d_ln2_b", _c_void_p),
        ("d_fc1_w", _c_void_p), ("d_fc1_b", _c_void_p), ("d_fc2_w", _c_void_p), ("d_fc2_b", _c_void_p),
        ("acc_w", _int),
        ("d_ff", _c_void_p), ("d_ln2", _c_void_p), ("d_h1", _c_void_p), ("d_ctx", _c_void_p), ("d_probs", _c_void_p),
        ("d_qkv", _c_void_p), ("norm_partial", _c_void_p), ("nblk", _int),
        ("dq_acc", _c_void_p), ("delta", _c_void_p),
        ("acc_small", _int), ("colsum_scratch", _c_void_p), ("colsum_scratch_bytes", ctypes.c_int64),
    ]


_PARAM_NAMES = ("ln1_w", "ln1_b", "qkv_w", "qkv_b", "out_w", "out_b", "ln2_w", "ln2_b", "fc1_w", "fc1_b", "fc2_w", "fc2_b")
_WEIGHTS = ("qkv_w", "out_w", "fc1_w", "fc2_w")


def _as_bytes(mask: torch.Tensor) -> torch.Tensor:
    """A boolean mask as bytes without a conversion pass (bool tensors are stored as one 0/1 byte per element)."""
    if mask.dtype == torch.bool:
        return mask.contiguous().view(torch.uint8)
    return mask.to(torch.uint8).contiguous()


def _fill(blk: _Block, x, y, mask, params, saved, n_heads, d_head, act, eps, causal):
    b, s, d = x.shape
    blk.batch, blk.seq, blk.d_model, blk.n_heads, blk.d_head = b, s, d, n_heads, d_head
    blk.d_ff = params[8].shape[0]
    blk.dtype = 0 if x.dtype == torch.float16 else 1
    blk.act = 1 if act == "relu" else 2
    blk.eps, blk.causal = eps, 1 if causal else 0
    blk.mask = None if mask is None else mask.data_ptr()
    for name, p in zip(_PARAM_NAMES, params):
        setattr(blk, name, p.data_ptr())
    blk.x, blk.y = x.data_ptr(), y.data_ptr()
    for name in ("ln1", "stats1", "qkv", "ctx", "h1", "ln2", "stats2", "ff"):
        setattr(blk, name, saved[name].data_ptr())
    if saved.get("lse") is not None:
        # fused attention: scores and probabilities never reach memory, one log-sum-exp per row is kept instead
        blk.lse, blk.probs, blk.probs_ld = saved["lse"].data_ptr(), None, 0
    else:
        blk.lse, blk.probs, blk.probs_ld = None, saved["probs"].data_ptr(), saved["probs"].stride(2)
    blk.pre = saved["pre"].data_ptr() if saved.get("pre") is not None else None


class GPTBlockFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, mask, n_heads, d_head, act, eps, causal, deferred, *params):
        lib = _native.cuda_lib()
        x = x.contiguous()
        b, s, d = x.shape
        T, hd, dff = b * s, n_heads * d_head, params[8].shape[0]
        dev, dt = x.device, x.dtype
        sp = (s + 7) // 8 * 8
        mask8 = None if mask is None else _as_bytes(mask)
        import os

        fused_attn = d_head % 16 == 0 and d_head <= 128 and os.environ.get("BMT_FLASH_ATTN", "1") != "0"
        saved = {
            "ln1": torch.empty(T, d, dtype=dt, device=dev), "stats1": torch.empty(2, T, dtype=torch.float32, device=dev),
            "qkv": torch.empty(T, 3 * hd, dtype=dt, device=dev),
            "probs": None if fused_attn else torch.empty(b, n_heads, s, sp, dtype=dt, device=dev),
            "lse": torch.empty(b, n_heads, s, dtype=torch.float32, device=dev) if fused_attn else None,
            "ctx": torch.empty(T, hd, dtype=dt, device=dev), "h1": torch.empty(T, d, dtype=dt, device=dev),
            "ln2": torch.empty(T, d, dtype=dt, device=dev), "stats2": torch.empty(2, T, dtype=torch.float32, device=dev),
            "ff": torch.empty(T, dff, dtype=dt, device=dev),
            "pre": torch.empty(T, dff, dtype=dt, device=dev) if act == "gelu" else None,
        }
        y = torch.empty_like(x)
        blk = _Block()
        _fill(blk, x, y, mask8, params, saved, n_heads, d_head, act, eps, causal)
        if deferred is None:
            _native.check(lib.bmt_gpt_block_forward(ctypes.byref(blk), _native.stream_handle()), "GPT block forward")
        else:
            # the block's parameters are still on their way: norms and biases first; the QKV weight is gathered by the GEMM
            # that consumes it; the other big weights travel on the peer stream and have the attention core's duration to
            # arrive before the output projection.  They start together with the GEMM ("before") or when it is done
            # ("after", so that the QKV weight has the links to itself): BMT_REST_PUSH, default by group size.
            import os

            from ..parallel import fused_ops

            cur = torch.cuda.current_stream()
            cur.wait_event(deferred["ev_small"])
            _native.check(lib.bmt_gpt_block_forward_steps(ctypes.byref(blk), 1, 1, _native.stream_handle()), "GPT block forward")
            when = os.environ.get("BMT_REST_PUSH") or ("before" if deferred["bucket"].comm.size <= 2 else "after")
            if when == "before":
                ev_rest = deferred["push_rest"]()
                fused_ops.zero_gather_gemm(saved["ln1"], saved["qkv"], params[3], deferred)
            else:
                fused_ops.zero_gather_gemm(saved["ln1"], saved["qkv"], params[3], deferred)
                ev_gemm = torch.cuda.Event()
                ev_gemm.record(cur)
                ev_rest = deferred["push_rest"](ev_gemm)
            _native.check(lib.bmt_gpt_block_forward_steps(ctypes.byref(blk), 3, 5, _native.stream_handle()), "GPT block forward")
            cur.wait_event(ev_rest)
            _native.check(lib.bmt_gpt_block_forward_steps(ctypes.byref(blk), 6, 9, _native.stream_handle()), "GPT block forward")
        ctx.saved, ctx.x, ctx.mask8, ctx.params = saved, x, mask8, params
        ctx.cfg = (n_heads, d_head, act, eps, causal)
        return y

    @staticmethod
    def backward(ctx, dy):
        lib = _native.cuda_lib()
        x, saved, params = ctx.x, ctx.saved, ctx.params
        n_heads, d_head, act, eps, causal = ctx.cfg
        b, s, d = x.shape
        T, hd, dff = b * s, n_heads * d_head, params[8].shape[0]
        dev, dt = x.device, x.dtype
        dy = dy.contiguous()
        blk = _Block()
        y_dummy = dy  # forward output pointer is not read by backward
        _fill(blk, x, y_dummy, ctx.mask8, params, saved, n_heads, d_head, act, eps, causal)
        g = _Grad()
        dx = torch.empty_like(x)
        g.dy, g.dx = dy.data_ptr(), dx.data_ptr()
        # gradients of the parameters: accumulate in place when the owner already attached same-dtype gradient buffers (no
        # tensor goes back to autograd for them, so no add kernel per parameter either)
        def attached(p):
            return p.is_leaf and p.requires_grad and p.grad is not None and p.grad.dtype == dt and p.grad.is_contiguous()

        acc_w = all(attached(p) for name, p in zip(_PARAM_NAMES, params) if name in _WEIGHTS)
        acc_small = all(attached(p) for name, p in zip(_PARAM_NAMES, params) if name not in _WEIGHTS)
        grads = {}
        for name, p in zip(_PARAM_NAMES, params):
            if acc_w if name in _WEIGHTS else acc_small:
                setattr(g, "d_" + name, p.grad.data_ptr())
            else:
                grads[name] = torch.empty_like(p)
                setattr(g, "d_" + name, grads[name].data_ptr())
        g.acc_w = 1 if acc_w else 0
        g.acc_small = 1 if acc_small else 0
        scratch = _gemm.colsum_scratch(dev)
        g.colsum_scratch, g.colsum_scratch_bytes = scratch.data_ptr(), scratch.numel() * 4
        nblk = min(T, 296)
        work = {
            "d_ff": torch.empty(T, dff, dtype=dt, device=dev), "d_ln2": torch.empty(T, d, dtype=dt, device=dev),
            "d_h1": torch.empty(T, d, dtype=dt, device=dev), "d_ctx": torch.empty(T, hd, dtype=dt, device=dev),
            "d_probs": None if saved["probs"] is None else torch.empty_like(saved["probs"]),
            "d_qkv": torch.empty(T, 3 * hd, dtype=dt, device=dev),
            "norm_partial": torch.empty(2, nblk, d, dtype=torch.float32, device=dev),
            "dq_acc": torch.empty(T * hd, dtype=torch.float32, device=dev) if saved["probs"] is None else None,
            "delta": torch.empty(b * n_heads * s, dtype=torch.float32, device=dev) if saved["probs"] is None else None,
        }
        for name, t in work.items():
            setattr(g, name, None if t is None else t.data_ptr())
        g.nblk = nblk
        _native.check(lib.bmt_gpt_block_backward(ctypes.byref(blk), ctypes.byref(g), _native.stream_handle()), "GPT block backward")
        ctx.saved = None
        out = [grads.get(name) if p.requires_grad else None for name, p in zip(_PARAM_NAMES, params)]
        return (dx, None, None, None, None, None, None, None) + tuple(out)


def gpt_block(x: torch.Tensor, mask: Optional[torch.Tensor], n_heads: int, d_head: int, act: str, eps: float, causal: bool,
              ln1_w, ln1_b, qkv_w, qkv_b, out_w, out_b, ln2_w, ln2_b, fc1_w, fc1_b, fc2_w, fc2_b, deferred=None) -> torch.Tensor:
    """``x`` (batch, seq, d_model) -> same shape.  ``mask``: optional bool (batch, seq, seq), True = attend.
    ``deferred``: gather-in-progress description from the owning ZeRO block (see ``Block._try_deferred_gather``)."""
    return GPTBlockFunction.apply(x, mask, n_heads, d_head, act, eps, causal, deferred, ln1_w, ln1_b, qkv_w, qkv_b, out_w, out_b,
                                  ln2_w, ln2_b, fc1_w, fc1_b, fc2_w, fc2_b)
