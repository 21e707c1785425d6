"""Kernel entry points with the reference's names (``bmtrain/loss/_function.py:7-182``)."""
import torch

from ..ops import cross_entropy as _ce
from ..ops.infnan import has_inf_nan  # noqa: F401  (re-export)


def cross_entropy_forward(m: int, n: int, input: torch.Tensor, target: torch.Tensor, softmax: torch.Tensor,
                          output: torch.Tensor, ignore_index: int) -> None:
    """Fill ``softmax`` (m, n) and the per-row ``output`` loss (0 where ``target == ignore_index``)."""
    mx, se, tl = _ce.row_stats(input.view(m, n), target.view(m))
    lse = mx + torch.log(se + 1e-10)
    loss = lse - tl
    loss = torch.where(target.view(m) == ignore_index, torch.zeros_like(loss), loss)
    output.copy_(loss)
    softmax.copy_(torch.exp(input.view(m, n).float() - lse[:, None]))


def cross_entropy_backward_inplace(m: int, n: int, grad_output: torch.Tensor, target: torch.Tensor,
                                   x: torch.Tensor, ignore_index: int) -> None:
    """``x`` holds a softmax on entry and ``(softmax - onehot) * grad_output`` on return."""
    sm = x.view(m, n).float()
    t = target.view(m).long()
    valid = t != ignore_index
    rows = torch.nonzero(valid, as_tuple=True)[0]
    sm[rows, t[rows]] -= 1.0
    sm = sm * grad_output.view(m, 1).float()
    sm[~valid] = 0
    x.view(m, n).copy_(sm)


def fused_sumexp(logits: torch.Tensor, max_logits: torch.Tensor) -> torch.Tensor:
    """``sum_j exp(logits[i, j] - max_logits[i])`` in fp32."""
    mx, se, _ = _ce.row_stats(logits, torch.zeros(logits.size(0), dtype=torch.int64, device=logits.device))
    return se * torch.exp(mx - max_logits.float())


def fused_softmax_inplace(logits: torch.Tensor, max_logits: torch.Tensor, sum_exp_logits: torch.Tensor) -> None:
    """``logits <- exp(logits - max) / sum`` in place."""
    logits.copy_(torch.exp(logits.float() - max_logits[:, None].float()) / sum_exp_logits[:, None].float())


def is_bf16_supported() -> bool:
    """bf16 kernels are always built here (the reference probes its CUDA version: ``csrc/cuda/has_inf_nan.cu:139-145``)."""
    return True
