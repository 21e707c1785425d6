"""Building-block modules on sharded parameters: embedding, LayerNorm, RMSNorm.

The reference keeps these in its example (``example/layers/embedding.py``,
``example/layers/layernorm.py``); they are part of the package here because
they sit on the framework's own kernels.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..layer import DistributedModule
from ..ops import embedding as _emb
from ..ops import gemm as _gemm
from ..ops import norm as _norm
from ..parameter import DistributedParameter, ParameterInitializer


class Embedding(DistributedModule):
    """Token embedding; ``forward(x, projection=True)`` multiplies by the transposed table (tied LM head)."""

    def __init__(self, num_embeddings: int, embedding_dim: int, dtype=None, init_mean: float = 0.0, init_std: float = 1.0):
        super().__init__()
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.weight = DistributedParameter(
            torch.empty(num_embeddings, embedding_dim, dtype=dtype, device="meta"),
            init_method=ParameterInitializer(torch.nn.init.normal_, mean=init_mean, std=init_std))

    def forward(self, input: torch.Tensor, projection: bool = False) -> torch.Tensor:
        if projection:
            return _gemm.linear(input, self.weight)
        return _emb.embedding(input, self.weight)

    def extra_repr(self) -> str:
        return f"{self.num_embeddings}, {self.embedding_dim}"


class LayerNorm(DistributedModule):
    """LayerNorm over the last dimension."""

    def __init__(self, normalized_shape: int, eps: float = 1e-5, elementwise_affine: bool = True, dtype=None):
        super().__init__()
        if not isinstance(normalized_shape, int):
            (normalized_shape,) = tuple(normalized_shape)
        self.normalized_shape = (normalized_shape,)
        self.eps = eps
        self.elementwise_affine = elementwise_affine
        assert elementwise_affine, "LayerNorm without affine parameters is not provided"
        self.weight = DistributedParameter(torch.empty(normalized_shape, dtype=dtype, device="meta"),
                                           init_method=torch.nn.init.ones_)
        self.bias = DistributedParameter(torch.empty(normalized_shape, dtype=dtype, device="meta"),
                                         init_method=torch.nn.init.zeros_)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return _norm.layer_norm(input, self.weight, self.bias, self.eps)

    def extra_repr(self) -> str:
        return f"{self.normalized_shape}, eps={self.eps}"


Layernorm = LayerNorm


class RMSNorm(DistributedModule):
    """Root-mean-square norm over the last dimension (Llama style)."""

    def __init__(self, dim: int, eps: float = 1e-6, dtype=None):
        super().__init__()
        self.dim = dim
        self.eps = eps
        self.weight = DistributedParameter(torch.empty(dim, dtype=dtype, device="meta"), init_method=torch.nn.init.ones_)

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        return _norm.rms_norm(input, self.weight, self.eps)

    def extra_repr(self) -> str:
        return f"{self.dim}, eps={self.eps}"
