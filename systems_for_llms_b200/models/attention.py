"""Rotary embedding, reference softmax attention and multi-head self-attention.

Portable definitions with the numerics of the reference
(src/llmlab/model/attention.py:10-203): interleaved-pair RoPE with tables cast
to the activation dtype, fp32 softmax for 16-bit scores, separate q/k/v/output
projections (so ``state_dict`` keys match) and an ``eager`` or ``sdpa`` backend.
The fused sm_100a path (models/fused.py) reads the same parameters.
"""

from __future__ import annotations

import math

import torch
from torch import nn
from torch.nn import functional as F

from .layers import Linear


class RotaryPositionalEmbedding(nn.Module):
    """cos/sin tables ``[max_seq_len, d_k/2]``; rotates lanes (2i, 2i+1) together."""

    def __init__(self, theta: float, d_k: int, max_seq_len: int, device=None):
        super().__init__()
        if d_k <= 0 or d_k % 2:
            raise ValueError("d_k must be positive and even because RoPE rotates dimension pairs")
        if not math.isfinite(theta) or theta <= 0:
            raise ValueError("theta must be finite and positive")
        if max_seq_len <= 0:
            raise ValueError("max_seq_len must be positive")
        self.theta, self.d_k, self.max_seq_len = theta, d_k, max_seq_len
        positions = torch.arange(max_seq_len, device=device)
        exponents = torch.arange(0, d_k, 2, device=device) / d_k
        angles = positions[:, None] * (1.0 / (theta ** exponents))[None, :]
        self.register_buffer("cos", torch.cos(angles), persistent=False)
        self.register_buffer("sin", torch.sin(angles), persistent=False)

    def forward(self, x: torch.Tensor, token_positions: torch.Tensor) -> torch.Tensor:
        cos = self.cos[token_positions].to(x.dtype)
        sin = self.sin[token_positions].to(x.dtype)
        even, odd = x[..., 0::2], x[..., 1::2]
        rotated = torch.empty_like(x)
        rotated[..., 0::2] = even * cos - odd * sin
        rotated[..., 1::2] = even * sin + odd * cos
        return rotated


def softmax(x: torch.Tensor, dim: int) -> torch.Tensor:
    shifted = x - torch.max(x, dim=dim, keepdim=True).values
    weights = torch.exp(shifted)
    return weights / torch.sum(weights, dim=dim, keepdim=True)


def scaled_dot_product_attention(query, key, value, mask=None):
    """Materialised attention; ``mask`` is True where attention is allowed."""
    scores = torch.matmul(query, key.transpose(-1, -2)) / math.sqrt(query.shape[-1])
    if mask is not None:
        scores = scores.masked_fill(~mask, float("-inf"))
    wide = scores.float() if scores.dtype in (torch.bfloat16, torch.float16) else scores
    weights = softmax(wide, dim=-1).to(scores.dtype)
    return torch.matmul(weights, value)


class MultiHeadSelfAttention(nn.Module):
    def __init__(self, d_model: int, num_heads: int, theta: float | None = None,
                 max_seq_len: int | None = None, device=None, dtype=None,
                 attention_backend: str = "eager"):
        super().__init__()
        if d_model <= 0 or num_heads <= 0:
            raise ValueError("d_model and num_heads must be positive")
        if d_model % num_heads:
            raise ValueError("d_model must be divisible by num_heads")
        if attention_backend not in ("eager", "sdpa"):
            raise ValueError("attention_backend must be 'eager' or 'sdpa'")
        if (theta is None) != (max_seq_len is None):
            raise ValueError("theta and max_seq_len must be provided together")
        self.d_model, self.num_heads = d_model, num_heads
        self.d_k = d_model // num_heads
        self.attention_backend = attention_backend
        self.max_seq_len = max_seq_len
        self.q_proj = Linear(d_model, d_model, device=device, dtype=dtype)
        self.k_proj = Linear(d_model, d_model, device=device, dtype=dtype)
        self.v_proj = Linear(d_model, d_model, device=device, dtype=dtype)
        self.output_proj = Linear(d_model, d_model, device=device, dtype=dtype)
        self.rope = (RotaryPositionalEmbedding(theta, self.d_k, max_seq_len, device=device)
                     if theta is not None else None)

    def _split_heads(self, x: torch.Tensor) -> torch.Tensor:
        return x.unflatten(-1, (self.num_heads, self.d_k)).transpose(-3, -2)

    def forward(self, x: torch.Tensor, token_positions: torch.Tensor | None = None):
        if x.ndim < 2 or x.shape[-1] != self.d_model:
            raise ValueError("x must have shape (..., sequence_length, d_model)")
        seq_len = x.shape[-2]
        if seq_len == 0:
            raise ValueError("sequence length must be positive")
        if self.max_seq_len is not None and seq_len > self.max_seq_len:
            raise ValueError("sequence length exceeds max_seq_len")
        if token_positions is None:
            token_positions = torch.arange(seq_len, device=x.device)
        query = self._split_heads(self.q_proj(x))
        key = self._split_heads(self.k_proj(x))
        value = self._split_heads(self.v_proj(x))
        if self.rope is not None:
            query = self.rope(query, token_positions)
            key = self.rope(key, token_positions)
        if self.attention_backend == "sdpa":
            attended = F.scaled_dot_product_attention(query, key, value, is_causal=True,
                                                      dropout_p=0.0)
        else:
            causal = torch.ones(seq_len, seq_len, device=x.device, dtype=torch.bool).tril()
            attended = scaled_dot_product_attention(query, key, value, mask=causal)
        merged = attended.transpose(-3, -2).flatten(-2)
        return self.output_proj(merged)
