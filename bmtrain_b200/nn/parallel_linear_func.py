"""Tensor-parallel linear core (reference: ``bmtrain/nn/parallel_linear_func.py:10-352``).

``OpParallelLinear.apply(input, weight, bias, gather_input, gather_output,
split_input, reduce_output_type, async_gather_chunks)`` covers every
column/row-parallel variant:

==================  =================================================================
gather_input        all-gather the token dim (dim 0) of ``input`` over the TP group
split_input         keep this rank's slice of the feature dim of ``input``
gather_output       all-gather the feature dim of the output
reduce_output_type  ``ALL_REDUCE`` (sum in place) or ``REDUCE_SCATTER`` (sum, keep
                    this rank's slice of the token dim)
==================  =================================================================

Tokens are laid out rank-major: after a gather, rows ``[j*m, (j+1)*m)`` are rank
``j``'s tokens, and a reduce-scatter hands rank ``j`` those rows back.

Where a GEMM is adjacent to its collective (all-gather -> GEMM, GEMM ->
reduce-scatter) the pair is handed to ``bmtrain_b200.parallel.tp_fused``, which
on NVLink-connected B200s runs them as one kernel over peer memory and otherwise
falls back to collective + GEMM.  ``async_gather_chunks`` is accepted for API
compatibility; the fused kernels overlap at tile granularity instead of chunking.
"""
from __future__ import annotations

from enum import Enum

import torch

from ..global_var import config
from ..ops import gemm as _gemm
from ..parallel import tp_fused


class ReduceType(Enum):
    ALL_REDUCE = 1
    REDUCE_SCATTER = 2


def _gather_tokens(x: torch.Tensor) -> torch.Tensor:
    comm = config["tp_comm"]
    x = x.contiguous()
    out = torch.empty((comm.size * x.shape[0],) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    comm.all_gather_into(out, x)
    return out


def _scatter_tokens_sum(x: torch.Tensor) -> torch.Tensor:
    comm = config["tp_comm"]
    x = x.contiguous()
    out = torch.empty((x.shape[0] // comm.size,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
    comm.reduce_scatter_into(out, x, "sum")
    return out


def _split_features(x: torch.Tensor) -> torch.Tensor:
    return x.chunk(config["tp_size"], dim=-1)[config["topology"].tp_id]


def preprocess_input(input, gather_input, split_input):
    if gather_input:
        input = _gather_tokens(input)
    if split_input:
        input = _split_features(input)
    return input


def async_all_gather_linear_func(input, weight, bias, async_chunks=2):
    """``all_gather_tokens(input) @ weight^T + bias`` (reference: ``bmtrain/nn/parallel_linear_func.py:26-61``, which
    overlaps by cutting the tokens into ``async_chunks`` rounds; here the fused kernel overlaps tile by tile)."""
    tp = config["tp_size"]
    x2 = input.reshape(-1, input.shape[-1])
    out = tp_fused.all_gather_gemm(x2, weight, bias, config["tp_comm"])
    return out.view(input.shape[0] * tp, *input.shape[1:-1], weight.shape[0])


def async_reduce_scatter_linear_func(input, weight, bias, async_chunks=2):
    """``reduce_scatter_tokens(input @ weight^T) + bias`` (reference: ``bmtrain/nn/parallel_linear_func.py:64-105``)."""
    tp = config["tp_size"]
    x2 = input.reshape(-1, input.shape[-1])
    out = tp_fused.gemm_reduce_scatter(x2, weight, bias, config["tp_comm"])
    return out.view(input.shape[0] // tp, *input.shape[1:-1], weight.shape[0])


def async_all_gather_linear_backward_func(grad_out, input, weight, bias, async_chunks=2):
    """Backward of the row-parallel GEMM -> reduce-scatter: the output gradient is all-gathered over the tokens, then
    ``grad_input = G @ W``, ``grad_weight = G^T @ input``, ``grad_bias = sum(G)``
    (reference: ``bmtrain/nn/parallel_linear_func.py:108-200``)."""
    comm = config["tp_comm"]
    x2 = input.reshape(-1, input.shape[-1])
    g_local = grad_out.reshape(-1, grad_out.shape[-1])
    grad_input = grad_weight = grad_bias = None
    if input.requires_grad:
        gx, g_all = tp_fused.all_gather_gemm(g_local, weight, None, comm, b_is_kn=True, return_gathered=True)
        grad_input = gx.view(input.shape)
    else:
        g_all = _gather_tokens(g_local)
    if weight.requires_grad:
        grad_weight = _gemm.gemm_tn(g_all, x2)
    if bias is not None and bias.requires_grad:
        grad_bias = _gemm.bias_grad(g_all)
    return grad_input, grad_weight, grad_bias


class OpParallelLinear(torch.autograd.Function):
    """Linear layer with the tensor-parallel collectives folded in (see the module docstring)."""

    @staticmethod
    def forward(ctx, input, weight, bias=None, gather_input=False, gather_output=False, split_input=False,
                reduce_output_type=None, async_gather_chunks=2):
        if reduce_output_type is not None:
            reduce_output_type = ReduceType(reduce_output_type)
        tp = config["tp_size"]
        ctx.save_for_backward(input, weight, bias)
        ctx.flags = (gather_input, gather_output, split_input, reduce_output_type)

        lead = input.shape[:-1]
        if tp == 1:
            out = _gemm.gemm_nt(input.reshape(-1, input.shape[-1]), weight, bias)
            return out.view(*lead, weight.shape[0])

        if gather_input and not split_input:
            x2 = input.reshape(-1, input.shape[-1])
            out = tp_fused.all_gather_gemm(x2, weight, bias, config["tp_comm"])
            out = out.view(lead[0] * tp, *lead[1:], weight.shape[0])
        elif reduce_output_type == ReduceType.REDUCE_SCATTER:
            x = preprocess_input(input, gather_input, split_input)
            x2 = x.reshape(-1, x.shape[-1])
            out = tp_fused.gemm_reduce_scatter(x2, weight, bias, config["tp_comm"])
            return out.view(x.shape[0] // tp, *x.shape[1:-1], weight.shape[0])
        else:
            x = preprocess_input(input, gather_input, split_input)
            out = _gemm.gemm_nt(x.reshape(-1, x.shape[-1]), weight, bias).view(*x.shape[:-1], weight.shape[0])

        if gather_output:
            comm = config["tp_comm"]
            stacked = torch.empty((tp,) + tuple(out.shape), dtype=out.dtype, device=out.device)
            comm.all_gather_into(stacked, out.contiguous())
            out = torch.cat(list(stacked.unbind(0)), dim=-1)

        if reduce_output_type is None:
            return out
        if reduce_output_type == ReduceType.ALL_REDUCE:
            config["tp_comm"].all_reduce(out, "sum")
            return out
        raise AssertionError(f"no support reduce type{reduce_output_type}")

    @staticmethod
    def backward(ctx, grad_output):
        input, weight, bias = ctx.saved_tensors
        gather_input, gather_output, split_input, reduce_type = ctx.flags
        tp = config["tp_size"]
        comm = config["tp_comm"]
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        need_b = bias is not None and ctx.needs_input_grad[2]
        grad_input = grad_weight = grad_bias = None
        none5 = (None,) * 5

        if tp == 1:
            g2 = grad_output.reshape(-1, grad_output.shape[-1])
            x2 = input.reshape(-1, input.shape[-1])
            if need_x:
                grad_input = _gemm.gemm_nn(g2, weight).view(input.shape)
            if need_w:
                grad_weight = _gemm.gemm_tn(g2, x2)
            if need_b:
                grad_bias = _gemm.bias_grad(g2)
            return (grad_input, grad_weight, grad_bias) + none5

        if reduce_type == ReduceType.REDUCE_SCATTER:
            # forward was GEMM -> reduce-scatter(tokens): backward is all-gather(grad) -> dgrad / wgrad
            x = preprocess_input(input, gather_input, split_input)
            x2 = x.reshape(-1, x.shape[-1])
            g_local = grad_output.reshape(-1, grad_output.shape[-1])
            if need_x:
                gx, g_all = tp_fused.all_gather_gemm(g_local, weight, None, comm, b_is_kn=True, return_gathered=True)
                grad_input = gx.view(x.shape)
                if split_input:
                    stacked = torch.empty((tp,) + tuple(grad_input.shape), dtype=gx.dtype, device=gx.device)
                    comm.all_gather_into(stacked, grad_input.contiguous())
                    grad_input = torch.cat(list(stacked.unbind(0)), dim=-1)
            else:
                g_all = _gather_tokens(g_local)
            if need_w:
                grad_weight = _gemm.gemm_tn(g_all, x2)
            if need_b:
                grad_bias = _gemm.bias_grad(g_all)
            return (grad_input, grad_weight, grad_bias) + none5

        if gather_output:
            grad_output = grad_output.chunk(tp, dim=-1)[config["topology"].tp_id].contiguous()
        g2 = grad_output.reshape(-1, grad_output.shape[-1])

        if need_x:
            if gather_input and not split_input:
                # dgrad GEMM -> reduce-scatter over tokens (mirror of the forward all-gather)
                gx = tp_fused.gemm_reduce_scatter(g2, weight, None, comm, b_is_kn=True)
                grad_input = gx.view(input.shape)
            else:
                gx = _gemm.gemm_nn(g2, weight)
                if gather_input:
                    gx = _scatter_tokens_sum(gx)
                elif reduce_type is None:
                    comm.all_reduce(gx, "sum")
                lead = grad_output.shape[:-1] if not gather_input else input.shape[:-1]
                grad_input = gx.view(*lead, gx.shape[-1])
                if split_input:
                    stacked = torch.empty((tp,) + tuple(grad_input.shape), dtype=gx.dtype, device=gx.device)
                    comm.all_gather_into(stacked, grad_input.contiguous())
                    grad_input = torch.cat(list(stacked.unbind(0)), dim=-1)
                    if gather_input:
                        grad_input = grad_input.view(input.shape)
        if need_w:
            x = preprocess_input(input, gather_input, split_input)
            grad_weight = _gemm.gemm_tn(g2, x.reshape(-1, x.shape[-1]))
        if need_b:
            grad_bias = _gemm.bias_grad(g2)
        return (grad_input, grad_weight, grad_bias) + none5
