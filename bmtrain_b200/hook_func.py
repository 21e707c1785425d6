"""Forward / backward hooks of a ZeRO block under their reference names (``bmtrain/hook_func.py:6-121``).

The reference wraps every block in two identity autograd functions (``PreHookFunc`` / ``PostHookFunc``) whose forward
and backward call these four hooks, plus ``OneStepNoGradFunc`` for blocks whose inputs need no gradient.  Here a block is
a single autograd node (``block_layer._BlockFunction``) that calls ``Block._enter_forward`` / ``_exit_forward`` /
``_enter_backward`` / ``_exit_backward`` itself; the functions below expose the same four moments for code written
against the reference, and the two identity functions are kept so such code can still bracket a module by hand.
"""
from __future__ import annotations

import torch

from .block_layer import _BlockFunction


def zero_pre_forward(module, inputs):
    """Parameters of ``module`` (a ``Block``) are gathered, the next block's gather is started."""
    module._enter_forward(inputs if isinstance(inputs, tuple) else (inputs,))


def zero_post_forward(module, inputs, outputs):
    """Parameters are released (ZeRO-3) or kept for backward (ZeRO-2)."""
    module._exit_forward()


def zero_pre_backward(module, grad_outputs):
    """Parameters are gathered again and full-size gradient buffers attached."""
    module._enter_backward()


def zero_post_backward(module, grad_inputs, grad_outputs):
    """Gradients are reduce-scattered into the local partitions, parameters released."""
    module._exit_backward()


class PreHookFunc(torch.autograd.Function):
    """Identity whose forward runs ``zero_pre_forward`` and whose backward runs ``zero_post_backward``."""

    @staticmethod
    def forward(ctx, module, *x):
        ctx.module = module
        zero_pre_forward(module, x)
        return x

    @staticmethod
    def backward(ctx, *grads):
        zero_post_backward(ctx.module, grads, None)
        return (None,) + grads


class PostHookFunc(torch.autograd.Function):
    """Identity whose forward runs ``zero_post_forward`` and whose backward runs ``zero_pre_backward``."""

    @staticmethod
    def forward(ctx, module, *out):
        ctx.module = module
        zero_post_forward(module, None, out)
        return out

    @staticmethod
    def backward(ctx, *grads):
        zero_pre_backward(ctx.module, grads)
        return (None,) + grads


# Blocks whose inputs need no gradient run through the same autograd node as every other block: it executes the forward
# without building a graph and rebuilds it in backward (with the RNG state restored), which is what the reference's
# OneStepNoGradFunc does for that special case only.
OneStepNoGradFunc = _BlockFunction
