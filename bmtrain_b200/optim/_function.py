"""Launch shims with the reference's names (``bmtrain/optim/_function.py:7-218``)."""
import torch

from ..ops import adam as _adam


def bf16_from_fp32(param_fp32: torch.Tensor, param_bf16: torch.Tensor) -> None:
    _adam.half_from_fp32(param_fp32, param_bf16)


def fp16_from_fp32(param_fp32: torch.Tensor, param_fp16: torch.Tensor) -> None:
    _adam.half_from_fp32(param_fp32, param_fp16)


def adam_cpu(param_fp32, param_fp16, delta_info, g_fp16, m_fp32, v_fp32, beta1, beta2, eps, lr, scale, weight_decay, step):
    _adam.adam_cpu(param_fp32, param_fp16, delta_info, g_fp16, m_fp32, v_fp32, beta1, beta2, eps, lr, scale, weight_decay, step)


def adam_fp16(param_fp32, param_fp16, g_fp16, m_fp16, v_fp32, beta1, beta2, eps, lr, scale, weight_decay, step):
    assert param_fp16.dtype == torch.float16 and m_fp16.dtype == torch.float16
    _adam.adam_half_multi([(param_fp32, param_fp16, g_fp16, m_fp16, v_fp32)], beta1, beta2, eps, lr, scale, weight_decay, step)


def adam_bf16(param_fp32, param_bf16, g_bf16, m_fp32, v_fp32, beta1, beta2, eps, lr, scale, weight_decay, step):
    assert param_bf16.dtype == torch.bfloat16 and m_fp32.dtype == torch.float32
    _adam.adam_half_multi([(param_fp32, param_bf16, g_bf16, m_fp32, v_fp32)], beta1, beta2, eps, lr, scale, weight_decay, step)
