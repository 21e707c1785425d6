"""``ZeroContext``: a block's parameters gathered for the duration of a ``with`` body.

In the reference (``bmtrain/zero_context.py:7-203``) this class *is* the ZeRO engine: ``enter`` all-gathers every bucket
on the load stream and re-points the parameters, ``exit`` reduce-scatters the gradients and points them back.  Here the
engine lives in ``Block`` (``block_layer.py``: ``_ensure_gathered`` / ``_prepare_grads`` / ``_scatter_grads`` /
``_release_params``, driven by one autograd node per block); this class keeps the reference's entry points on top of
those methods for code that gathers a block by hand, e.g. to read full parameters or to call the inner module directly::

    with ZeroContext(block):
        out = block._module(x)          # full-size parameters are in place

Flags follow the reference: 0 = gather and drop afterwards (ZeRO-3), 1 = gather and keep the gathered buffers at exit
(ZeRO-2 forward), 2 = reuse kept buffers.
"""
from __future__ import annotations

from typing import Optional


class ZeroContext:
    def __init__(self, block, ctx_dict: Optional[dict] = None, pipe: bool = False) -> None:
        self.block = block
        self.ctx_dict = ctx_dict
        self.pipe = pipe
        self._entered = False

    def enter(self, flag: int = 0, requires_grad: bool = False) -> None:
        """Gather the block's parameters (no-op when they are resident); with ``requires_grad`` full-size gradient
        buffers are attached as well, as before a backward pass."""
        if self._entered:
            return
        self._entered = True
        self._was_resident = self.block._resident
        self.block._ensure_gathered()
        if requires_grad:
            self.block._prepare_grads()

    def exit(self, flag: int = 0, backward: bool = False) -> None:
        """Give the gathered parameters up again; after a backward pass (``backward``) the gradients are reduce-scattered
        into the local partitions first.  ``flag == 1`` keeps the gathered buffers for a later ``enter(flag=2)``."""
        if not self._entered:
            return
        self._entered = False
        if backward:
            self.block._scatter_grads()
        if flag == 1:
            self.block._point_to_local()
            self.block._resident = False
        elif not self._was_resident:
            self.block._release_params()

    def __enter__(self):
        self.enter()
        return self

    def __exit__(self, exc_type, exc_val, exc_tb):
        self.exit()
