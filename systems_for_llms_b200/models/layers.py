"""Basic modules of the decoder: Linear, Embedding, SwiGLU, RMSNorm.

These are the portable (CPU / fp32 / any-shape) definitions and the holders of
the fp32 parameters; their construction order and initialisers match the
reference (src/llmlab/model/layers.py:6-141) so the same seed gives the same
weights and ``state_dict`` keys.  On a B200 with bf16 autocast the transformer
block bypasses these ``forward`` methods and runs the fused sm_100a path over the
same parameters (see models/fused.py).
"""

from __future__ import annotations

import math

import torch
from torch import nn


def _truncated_normal(shape, std: float, device, dtype) -> nn.Parameter:
    weight = torch.empty(*shape, device=device, dtype=dtype)
    nn.init.trunc_normal_(weight, mean=0.0, std=std, a=-3 * std, b=3 * std)
    return nn.Parameter(weight)


class Linear(nn.Module):
    """Bias-free ``y = x W^T`` with ``W`` stored ``[out_features, in_features]``."""

    def __init__(self, in_features: int, out_features: int, device=None, dtype=None):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.weight = _truncated_normal((out_features, in_features),
                                        math.sqrt(2 / (in_features + out_features)), device, dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return torch.nn.functional.linear(x, self.weight)


class Embedding(nn.Module):
    """Row lookup into a ``[num_embeddings, embedding_dim]`` table."""

    def __init__(self, num_embeddings: int, embedding_dim: int, device=None, dtype=None):
        super().__init__()
        self.num_embeddings = num_embeddings
        self.embedding_dim = embedding_dim
        self.weight = _truncated_normal((num_embeddings, embedding_dim), 1.0, device, dtype)

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        return self.weight[token_ids]


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def default_d_ff(d_model: int) -> int:
    """8/3 of the model width, rounded up to a multiple of 64."""
    return 64 * math.ceil(int(8 * d_model / 3) / 64)


class SwiGLU(nn.Module):
    """``w2(silu(w1 x) * w3 x)``."""

    def __init__(self, d_model: int, d_ff: int | None = None, device=None, dtype=None):
        super().__init__()
        self.d_model = d_model
        self.d_ff = default_d_ff(d_model) if d_ff is None else d_ff
        # w1, w2, w3 in this order: the initialiser consumes the RNG per module.
        self.w1 = Linear(d_model, self.d_ff, device=device, dtype=dtype)
        self.w2 = Linear(self.d_ff, d_model, device=device, dtype=dtype)
        self.w3 = Linear(d_model, self.d_ff, device=device, dtype=dtype)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.w2(silu(self.w1(x)) * self.w3(x))


class RMSNorm(nn.Module):
    """fp32 ``x / sqrt(mean(x^2) + eps) * weight``, returned in the input dtype."""

    def __init__(self, d_model: int, eps: float = 1e-5, device=None, dtype=None):
        super().__init__()
        self.d_model = d_model
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(d_model, device=device, dtype=dtype))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        wide = x.to(torch.float32)
        rms = torch.sqrt(torch.mean(wide * wide, dim=-1, keepdim=True) + self.eps)
        return ((wide / rms) * self.weight).to(x.dtype)
