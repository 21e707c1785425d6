"""Fused cross-entropy losses (reference: ``bmtrain/loss/cross_entropy.py:7-260``).

``FusedCrossEntropy`` takes half-precision logits ``(N, C)`` and returns an fp32
loss.  With ``parallel=True`` the class dimension is sharded over the
tensor-parallel group (``(N, C / tp)`` per rank) and the per-row statistics of
all ranks (maximum, sum of exponentials, target logit) travel in ONE small
all-gather and are combined locally, where the reference issues three all-reduces
(``bmtrain/loss/cross_entropy.py:46,65,71``).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..global_var import config
from ..ops import cross_entropy as _ce


class OpFusedCrossEntropy(torch.autograd.Function):
    """Per-row cross entropy over dim 1; rows whose target equals ``ignore_index`` give 0."""

    @staticmethod
    def forward(ctx, x: torch.Tensor, target: torch.Tensor, ignore_index: int):
        assert x.ndim == 2
        x = x.contiguous()
        mx, se, tl = _ce.row_stats(x, target)
        lse = mx + torch.log(se + 1e-10)
        loss = torch.where(target == ignore_index, torch.zeros_like(lse), lse - tl)
        ctx.ignore_index = ignore_index
        ctx.save_for_backward(x, target, lse)
        return loss

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        x, target, lse = ctx.saved_tensors
        grad = _ce.ce_backward(x, target, lse, grad_output.contiguous(), 0, ctx.ignore_index)
        return grad, None, None


class VPFusedCrossEntropy(torch.autograd.Function):
    """Cross entropy over a vocabulary sharded across the tensor-parallel group."""

    @staticmethod
    def forward(ctx, logits: torch.Tensor, target: torch.Tensor):
        comm = config["tp_comm"]
        rank = config["tp_rank"]
        shape = target.shape
        n = logits.size(-1)
        x = logits.reshape(-1, n).contiguous()
        t = target.reshape(-1)
        start = rank * n
        mx, se, tl = _ce.row_stats(x, t, start)
        if comm is not None and comm.size > 1:
            # one collective: every rank's (max, sum-exp, target logit) rows; the combination is the usual rescaling of
            # partial sums to the common maximum (a rank that does not own the target contributes a target logit of 0)
            mine = torch.stack([mx, se, tl])
            every = mine.new_zeros((comm.size,) + tuple(mine.shape))
            comm.all_gather_into(every, mine)
            gmax = every[:, 0].max(dim=0).values
            total = (every[:, 1] * torch.exp(every[:, 0] - gmax)).sum(dim=0)
            tl = every[:, 2].sum(dim=0)
        else:
            gmax, total = mx, se
        lse = gmax + torch.log(total + 1e-10)
        loss = lse - tl
        ctx.start = start
        ctx.save_for_backward(x, t, lse)
        ctx.logits_shape = logits.shape
        return loss.view(shape)

    @staticmethod
    def backward(ctx, grad_output: torch.Tensor):
        x, t, lse = ctx.saved_tensors
        # an index no target can take: ignored rows are zeroed by the caller's weights
        grad = _ce.ce_backward(x, t, lse, grad_output.reshape(-1).contiguous(), ctx.start, -(1 << 62))
        return grad.view(ctx.logits_shape), None


class FusedCrossEntropy(torch.nn.Module):
    """Drop-in for ``nn.CrossEntropyLoss`` on half-precision logits; always returns fp32.

    Args:
        weight: optional per-class weights (1-D, length C).
        ignore_index: targets with this value do not contribute.
        reduction: ``"none"`` | ``"mean"`` | ``"sum"``.
        label_smoothing: only 0.0 is supported by the fused path.
        parallel: the class dimension is sharded over the tensor-parallel group.
    """

    def __init__(self, weight: Optional[torch.Tensor] = None, ignore_index: int = -100, reduction: str = "mean",
                 label_smoothing: float = 0.0, parallel: bool = False) -> None:
        super().__init__()
        self.weight = weight
        self.ignore_index = ignore_index
        self.reduction = reduction
        self.label_smoothing = label_smoothing
        self.parallel = parallel

    def forward(self, input: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        if self.parallel:
            ret = VPFusedCrossEntropy.apply(input, target.long())
        else:
            if input.dtype == torch.float32 and not input.is_cuda:
                return torch.nn.functional.cross_entropy(
                    input, target.long(), weight=self.weight, ignore_index=self.ignore_index,
                    reduction=self.reduction, label_smoothing=self.label_smoothing)
            if self.label_smoothing != 0.0:
                raise NotImplementedError("label_smoothing is not supported by the fused cross entropy")
            ret = OpFusedCrossEntropy.apply(input, target.long(), self.ignore_index)

        ignored = target == self.ignore_index
        if self.weight is not None:
            classes = input.size(1) * (config["tp_size"] if self.parallel else 1)
            if self.weight.dim() != 1 or self.weight.size(0) != classes:
                raise ValueError("weight should be a 1D tensor of size C")
            w = self.weight[torch.where(ignored, torch.zeros_like(target), target)].float()
            w = w.masked_fill(ignored, 0)
        else:
            w = (~ignored).float()
        ret = w * ret
        if self.reduction == "none":
            return ret
        if self.reduction == "sum":
            return ret.sum()
        if self.reduction == "mean":
            return ret.sum() / w.sum().float()
        raise ValueError(f"unknown reduction {self.reduction}")
