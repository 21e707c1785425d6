"""All-gather -> GEMM and GEMM -> reduce-scatter as single operators.

These are the tensor-parallel hot pairs of ``ColumnParallelLinear`` /
``RowParallelLinear`` (reference: chunked NCCL + cuBLAS overlap in
``bmtrain/nn/parallel_linear_func.py:26-105``).  On NVLink-connected B200s
each pair is one kernel working on peer memory (``csrc/gemm_sm100.cu``, fused modes 1 and 2); on other
setups (CPU ranks, or peer access unavailable) the collective and the GEMM run
back to back.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from ..comm import Communicator
from ..ops import gemm as _gemm


def _fused_available(x: torch.Tensor, comm: Communicator) -> bool:
    if not x.is_cuda or comm.size == 1:
        return False
    # With ZeRO groups larger than one, kernels of the data-parallel dimension that wait for other ranks run next to the
    # tensor-parallel ones.  The fused kernels have a non-spinning form for that layout (``symm.no_spin``: pusher CTAs are
    # the first of their grid, GEMM -> reduce-scatter leaves waiting and summing to separate small launches), which is
    # verified kernel by kernel on two GPUs; the one full-size run of tensor parallel 2 x ZeRO 4 on eight GPUs with them
    # did not get through its first optimizer step (one tensor-parallel pair fell behind the others and every rank ended
    # up waiting in an all-gather).  Until that has been understood on hardware, this layout takes NCCL + separate GEMMs
    # unless BMT_TP_FUSED_WITH_ZERO=1 asks for the fused kernels.
    from ..global_var import config
    from . import symm

    zero = config.get("pp_tp_zero_comm") if config.get("pipe_size", 1) > 1 else config.get("tp_zero_comm")
    if zero is not None and zero.size > 1 and os.environ.get("BMT_TP_FUSED_WITH_ZERO", "0") != "1":
        return False
    return symm.peer_runtime_ready(comm)


def all_gather_gemm(x_local: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], comm: Communicator,
                    b_is_kn: bool = False, return_gathered: bool = False):
    """``gather_tokens(x_local) @ W^T`` (or ``@ W`` when ``b_is_kn``: W is (K, N)).

    Returns the (size*m, N) product, and the gathered input as well when asked.
    """
    if _fused_available(x_local, comm):
        from . import fused_ops

        res = fused_ops.ag_gemm(x_local, weight, bias, comm, b_is_kn, return_gathered)
        if res is not None:
            return res
    x_local = x_local.contiguous()
    x_all = torch.empty((comm.size * x_local.shape[0], x_local.shape[1]), dtype=x_local.dtype, device=x_local.device)
    comm.all_gather_into(x_all, x_local)
    out = _gemm.gemm_nn(x_all, weight) if b_is_kn else _gemm.gemm_nt(x_all, weight, bias)
    return (out, x_all) if return_gathered else out


def gemm_reduce_scatter(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor], comm: Communicator,
                        b_is_kn: bool = False) -> torch.Tensor:
    """``reduce_scatter_tokens(x @ W^T)`` (+ bias on the scattered result); ``b_is_kn``: ``x @ W``."""
    if _fused_available(x, comm):
        from . import fused_ops

        res = fused_ops.gemm_rs(x, weight, bias, comm, b_is_kn)
        if res is not None:
            return res
    full = _gemm.gemm_nn(x, weight) if b_is_kn else _gemm.gemm_nt(x, weight)
    out = torch.empty((full.shape[0] // comm.size, full.shape[1]), dtype=full.dtype, device=full.device)
    comm.reduce_scatter_into(out, full, "sum")
    if bias is not None:
        out = out + bias
    return out
