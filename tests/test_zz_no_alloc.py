"""The allocation-free norm backward (``bmt_norm_bwd_noalloc``), called through its exported C symbol.

Some users of the kernel library cannot allocate device memory when they need the norm backward (no PyTorch
allocator around, or an up-front memory budget); for them the library carries the partial-sum scratch itself.
This test drives that entry point with ctypes exactly as such a caller would -- inputs and outputs are plain
device pointers -- and compares it with the regular entry point (caller-provided scratch) twice in a row, the
second time with different data, because the built-in scratch is shared between calls and keeps old contents.

The file name sorts last on purpose: a run that stops at the first failure has then already run everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from bmtrain_b200.ops import _native

    lib = _native.cuda_lib()
    lib.bmt_norm_bwd_noalloc.restype = ctypes.c_int
    return lib, _native


def _run_both(lib, _native, rows, d, dtype, rms, seed):
    torch.manual_seed(seed)
    dev = torch.device("cuda")
    dt_code = 0 if dtype == torch.float16 else 1
    x = torch.randn(rows, d, device=dev, dtype=dtype)
    w = (1 + 0.1 * torch.randn(d, device=dev)).to(dtype)
    b = None if rms else (0.1 * torch.randn(d, device=dev)).to(dtype)
    dy = torch.randn(rows, d, device=dev, dtype=dtype)
    y = torch.empty_like(x)
    stats = torch.empty(2, rows, dtype=torch.float32, device=dev)
    stream = _native.stream_handle()
    assert lib.bmt_norm_fwd(ctypes.c_int64(rows), ctypes.c_int64(d), _native.ptr(x), _native.ptr(w), _native.ptr(b),
                            ctypes.c_float(1e-5), ctypes.c_int(int(rms)), ctypes.c_int(dt_code), _native.ptr(y),
                            _native.ptr(stats), stream) == 0

    # regular entry point: the caller brings the scratch
    nblk = min(rows, 296)
    partial = torch.empty(2, nblk, d, dtype=torch.float32, device=dev)
    dx_a, dw_a = torch.empty_like(x), torch.empty_like(w)
    db_a = None if rms else torch.empty_like(w)
    assert lib.bmt_norm_bwd(ctypes.c_int64(rows), ctypes.c_int64(d), _native.ptr(x), _native.ptr(dy), _native.ptr(w),
                            _native.ptr(stats), ctypes.c_int(int(rms)), ctypes.c_int(dt_code), ctypes.c_int(nblk),
                            _native.ptr(dx_a), _native.ptr(partial), _native.ptr(dw_a), _native.ptr(db_a), stream) == 0

    # allocation-free entry point: outputs are pre-allocated here, nothing is allocated inside the call
    dx_b, dw_b = torch.empty_like(x), torch.empty_like(w)
    db_b = None if rms else torch.empty_like(w)
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    rc = lib.bmt_norm_bwd_noalloc(ctypes.c_int64(rows), ctypes.c_int64(d), _native.ptr(x), _native.ptr(dy), _native.ptr(w),
                                  _native.ptr(stats), ctypes.c_int(int(rms)), ctypes.c_int(dt_code),
                                  _native.ptr(dx_b), _native.ptr(dw_b), _native.ptr(db_b), stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before

    def rel(a, ref):
        return ((a.float() - ref.float()).abs().max() / (ref.float().abs().max() + 1e-6)).item()

    tol = 2e-2 if dtype == torch.bfloat16 else 3e-3  # same tolerance as the norm tests
    assert rel(dx_b, dx_a) < tol
    assert rel(dw_b, dw_a) < tol
    if not rms:
        assert rel(db_b, db_a) < tol
    # and against a plain PyTorch fp32 definition
    xr, wr = x.float().requires_grad_(), w.float().requires_grad_()
    if rms:
        yr = xr * torch.rsqrt(xr.pow(2).mean(-1, keepdim=True) + 1e-5) * wr
    else:
        br = b.float().requires_grad_()
        yr = torch.nn.functional.layer_norm(xr, (d,), wr, br, 1e-5)
    yr.backward(dy.float())
    assert rel(dx_b, xr.grad) < tol and rel(dw_b, wr.grad) < tol


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_noalloc_norm_backward_twice(bmt_gpu, dtype):
    lib, _native = _lib()
    # two calls in a row on the shared scratch: different sizes and data, LayerNorm then RMSNorm
    _run_both(lib, _native, rows=300, d=2560, dtype=dtype, rms=False, seed=11)
    _run_both(lib, _native, rows=77, d=4096, dtype=dtype, rms=True, seed=12)
    _run_both(lib, _native, rows=1000, d=256, dtype=dtype, rms=False, seed=13)


def test_noalloc_rejects_oversize(bmt_gpu):
    lib, _native = _lib()
    dev = torch.device("cuda")
    d = 4096 + 8
    x = torch.zeros(4, d, device=dev, dtype=torch.float16)
    stats = torch.zeros(2, 4, device=dev)
    w = torch.ones(d, device=dev, dtype=torch.float16)
    rc = lib.bmt_norm_bwd_noalloc(ctypes.c_int64(4), ctypes.c_int64(d), _native.ptr(x), _native.ptr(x), _native.ptr(w),
                                  _native.ptr(stats), ctypes.c_int(0), ctypes.c_int(0), _native.ptr(x), _native.ptr(w),
                                  _native.ptr(None), _native.stream_handle())
    assert rc == -100
