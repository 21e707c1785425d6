"""Dense GEMMs of the transformer blocks.

Three operand layouts cover a linear layer (reference does all of them through
cuBLAS: ``bmtrain/nn/linear.py:10-24``):

* ``gemm_nt(a[M,K], b[N,K])``  -> ``a @ b.T``   forward  (x, W)
* ``gemm_nn(a[M,K], b[K,N])``  -> ``a @ b``     dgrad    (grad_out, W)
* ``gemm_tn(a[K,M], b[K,N])``  -> ``a.T @ b``   wgrad    (grad_out, x)

On a B200 all three run the hand-written tcgen05 kernel (``csrc/gemm_sm100.cu``:
TMA-fed shared-memory pipeline, accumulators in tensor memory, persistent tile
scheduler) with optional fused epilogues (bias add, GELU/ReLU, accumulate into
an existing tensor).  CPU tensors take the PyTorch definition.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import torch

from . import _native

ACT_NONE, ACT_RELU, ACT_GELU = 0, 1, 2
_ACT = {None: ACT_NONE, "none": ACT_NONE, "relu": ACT_RELU, "gelu": ACT_GELU}
_DT = {torch.float16: 0, torch.bfloat16: 1}

# operand major-ness as seen by the kernel: 0 = reduction dim contiguous, 1 = output dim contiguous
_K_MAJOR, _MN_MAJOR = 0, 1


def _apply_act(x: torch.Tensor, act) -> torch.Tensor:
    if act in (None, "none"):
        return x
    if act == "relu":
        return torch.relu(x)
    if act == "gelu":
        return torch.nn.functional.gelu(x)
    raise ValueError(act)


def _launch(a, b, out, m, n, k, a_major, b_major, bias, act, accumulate, lda, ldb):
    lib = _native.cuda_lib()
    assert a.dtype == b.dtype and a.dtype in _DT, "tensor-core GEMM takes fp16 or bf16 operands"
    out_dt = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[out.dtype]
    status = lib.bmt_gemm(
        ctypes.c_int64(m), ctypes.c_int64(n), ctypes.c_int64(k),
        _native.ptr(a), ctypes.c_int64(lda), ctypes.c_int(a_major),
        _native.ptr(b), ctypes.c_int64(ldb), ctypes.c_int(b_major),
        _native.ptr(out), ctypes.c_int64(out.stride(0)), ctypes.c_int(out_dt),
        _native.ptr(bias), ctypes.c_int(_ACT[act]), ctypes.c_int(1 if accumulate else 0),
        ctypes.c_int(_DT[a.dtype]), _native.stream_handle())
    _native.check(status, f"tcgen05 GEMM (m={m}, n={n}, k={k})")


def _use_torch(t: torch.Tensor) -> bool:
    return (not t.is_cuda) or os.environ.get("BMT_GEMM_DEBUG_TORCH", "0") == "1"


def _rowmajor(t: torch.Tensor) -> torch.Tensor:
    """A view TMA can read: unit inner stride, 16-byte aligned base and row pitch (pads a copy when needed)."""
    if t.stride(-1) == 1 and t.stride(0) >= t.shape[1] and t.stride(0) % 8 == 0 and t.data_ptr() % 16 == 0:
        return t
    if t.shape[1] % 8 == 0:
        return t.contiguous()
    padded = torch.zeros(t.shape[0], (t.shape[1] + 7) // 8 * 8, dtype=t.dtype, device=t.device)
    padded[:, : t.shape[1]].copy_(t)
    return padded[:, : t.shape[1]]


def gemm_nt(a: torch.Tensor, b: torch.Tensor, bias: Optional[torch.Tensor] = None, act=None,
            out: Optional[torch.Tensor] = None, accumulate: bool = False, out_dtype=None) -> torch.Tensor:
    """``act(a @ b.T + bias)``; ``a`` (M, K), ``b`` (N, K), both with contiguous K."""
    m, k = a.shape
    n = b.shape[0]
    assert b.shape[1] == k
    if _use_torch(a):
        r = torch.matmul(a.float(), b.float().t()) if a.dtype != torch.float32 else torch.matmul(a, b.t())
        if bias is not None:
            r = r + bias.float()
        r = _apply_act(r, act)
        if out is not None:
            out.copy_(out.float() + r if accumulate else r)
            return out
        return r.to(out_dtype or a.dtype)
    a, b = _rowmajor(a), _rowmajor(b)
    if out is None:
        assert not accumulate
        out = torch.empty(m, n, dtype=out_dtype or a.dtype, device=a.device)
    _launch(a, b, out, m, n, k, _K_MAJOR, _K_MAJOR, bias, act, accumulate, a.stride(0), b.stride(0))
    return out


def gemm_nn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
            out_dtype=None) -> torch.Tensor:
    """``a @ b``; ``a`` (M, K) with contiguous K, ``b`` (K, N) with contiguous N."""
    m, k = a.shape
    n = b.shape[1]
    assert b.shape[0] == k
    if _use_torch(a):
        r = torch.matmul(a.float(), b.float()) if a.dtype != torch.float32 else torch.matmul(a, b)
        if out is not None:
            out.copy_(out.float() + r if accumulate else r)
            return out
        return r.to(out_dtype or a.dtype)
    a, b = _rowmajor(a), _rowmajor(b)
    if out is None:
        assert not accumulate
        out = torch.empty(m, n, dtype=out_dtype or a.dtype, device=a.device)
    _launch(a, b, out, m, n, k, _K_MAJOR, _MN_MAJOR, None, None, accumulate, a.stride(0), b.stride(0))
    return out


def gemm_tn(a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None, accumulate: bool = False,
            out_dtype=None) -> torch.Tensor:
    """``a.T @ b``; ``a`` (K, M) with contiguous M, ``b`` (K, N) with contiguous N."""
    k, m = a.shape
    n = b.shape[1]
    assert b.shape[0] == k
    if _use_torch(a):
        r = torch.matmul(a.float().t(), b.float()) if a.dtype != torch.float32 else torch.matmul(a.t(), b)
        if out is not None:
            out.copy_(out.float() + r if accumulate else r)
            return out
        return r.to(out_dtype or a.dtype)
    a, b = _rowmajor(a), _rowmajor(b)
    if out is None:
        assert not accumulate
        out = torch.empty(m, n, dtype=out_dtype or a.dtype, device=a.device)
    _launch(a, b, out, m, n, k, _MN_MAJOR, _MN_MAJOR, None, None, accumulate, a.stride(0), b.stride(0))
    return out


_scratch = {}


def colsum_scratch(dev) -> torch.Tensor:
    """Work space of the row-split column sums (4 KB of ticket counters + partial sums), one per device and stream, zeroed
    once: the kernel leaves the counters at zero, and calls that share it are ordered on their stream."""
    key = (str(dev), torch.cuda.current_stream(dev).cuda_stream)
    buf = _scratch.get(key)
    if buf is None:
        buf = _scratch[key] = torch.zeros(1024 + 2 * 1024 * 1024, dtype=torch.float32, device=dev)
    return buf


def bias_grad(grad_out: torch.Tensor) -> torch.Tensor:
    """Column sums of ``grad_out`` (M, N), accumulated in fp32, returned in the input dtype."""
    if not grad_out.is_cuda:
        return grad_out.float().sum(0).to(grad_out.dtype)
    lib = _native.cuda_lib()
    g = grad_out.contiguous()
    m, n = g.shape
    out = torch.empty(n, dtype=g.dtype, device=g.device)
    dt = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[g.dtype]
    scratch = colsum_scratch(g.device)
    _native.check(lib.bmt_colsum_ex(ctypes.c_int64(m), ctypes.c_int64(n), _native.ptr(g), ctypes.c_int(dt), _native.ptr(out),
                                    ctypes.c_int(0), _native.ptr(scratch), ctypes.c_int64(scratch.numel() * 4),
                                    _native.stream_handle()), "column-sum kernel")
    return out


class LinearFunction(torch.autograd.Function):
    """``y = act(x W^T + b)`` with explicit dgrad / wgrad / bgrad GEMMs (activation only when no grad through it is needed: ``act`` must be None for training)."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        x2 = x.reshape(-1, x.shape[-1])
        y = gemm_nt(x2, weight, bias)
        return y.view(*x.shape[:-1], weight.shape[0])

    @staticmethod
    def backward(ctx, grad_output):
        x, weight = ctx.saved_tensors
        g2 = grad_output.reshape(-1, grad_output.shape[-1])
        x2 = x.reshape(-1, x.shape[-1])
        grad_x = grad_w = grad_b = None
        if ctx.needs_input_grad[0]:
            grad_x = gemm_nn(g2, weight).view(x.shape)
        if ctx.needs_input_grad[1]:
            grad_w = gemm_tn(g2, x2)
        if ctx.has_bias and ctx.needs_input_grad[2]:
            grad_b = bias_grad(g2)
        return grad_x, grad_w, grad_b


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Differentiable ``x @ weight.T + bias`` on the framework's GEMM kernels."""
    if x.dtype == torch.float32 and not x.is_cuda:
        return torch.nn.functional.linear(x, weight, bias)
    return LinearFunction.apply(x, weight, bias)
