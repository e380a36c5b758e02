"""Pre-norm decoder block and language model.

Module tree, constructor signature, validation and ``state_dict`` keys follow
the reference (src/llmlab/model/transformer.py:8-139).  ``forward`` has two
implementations chosen per call:

* the portable path - plain PyTorch modules, any device / dtype / shape, with
  ``torch.utils.checkpoint`` for ``activation_checkpointing="block"``;
* the fused sm_100a path - used on a B200 under bf16 autocast when the shapes fit
  the kernels (models/fused.py): flat fp32 parameters with a bf16 shadow, one
  autograd node per block, tcgen05 GEMMs with fused RoPE / SwiGLU / residual
  epilogues, flash attention, and block recomputation done inside the node.

``loss(input_ids, targets, scale)`` is the training entry point: on the fused
path it never materialises fp32 logits (vocabulary projection, log-sum-exp, loss
and the logit gradient are produced together).
"""

from __future__ import annotations

import torch
from torch import nn
from torch.utils.checkpoint import checkpoint

from .attention import MultiHeadSelfAttention
from .layers import Embedding, Linear, RMSNorm, SwiGLU


class TransformerBlock(nn.Module):
    def __init__(self, d_model: int, num_heads: int, d_ff: int, theta: float, max_seq_len: int,
                 device=None, dtype=None, attention_backend: str = "eager"):
        super().__init__()
        self.attn_norm = RMSNorm(d_model, device=device, dtype=dtype)
        self.attn = MultiHeadSelfAttention(d_model=d_model, num_heads=num_heads, theta=theta,
                                           max_seq_len=max_seq_len, device=device, dtype=dtype,
                                           attention_backend=attention_backend)
        self.ffn_norm = RMSNorm(d_model, device=device, dtype=dtype)
        self.ffn = SwiGLU(d_model=d_model, d_ff=d_ff, device=device, dtype=dtype)

    def forward(self, x: torch.Tensor, token_positions: torch.Tensor | None = None):
        x = x + self.attn(self.attn_norm(x), token_positions)
        return x + self.ffn(self.ffn_norm(x))


class TransformerLM(nn.Module):
    def __init__(self, vocab_size: int, context_length: int, d_model: int, num_layers: int,
                 num_heads: int, d_ff: int, rope_theta: float, device=None, dtype=None,
                 attention_backend: str = "eager", activation_checkpointing: str = "none"):
        super().__init__()
        sizes = dict(vocab_size=vocab_size, context_length=context_length, d_model=d_model,
                     num_layers=num_layers, num_heads=num_heads, d_ff=d_ff)
        for name, value in sizes.items():
            if not isinstance(value, int) or value <= 0:
                raise ValueError(f"{name} must be a positive integer")
        if activation_checkpointing not in ("none", "block"):
            raise ValueError("activation_checkpointing must be 'none' or 'block'")
        for name, value in sizes.items():
            setattr(self, name, value)
        self.theta = rope_theta
        self.attention_backend = attention_backend
        self.activation_checkpointing = activation_checkpointing
        self.token_embeddings = Embedding(vocab_size, d_model, device=device, dtype=dtype)
        self.layers = nn.ModuleList([
            TransformerBlock(d_model, num_heads, d_ff, rope_theta, context_length, device=device,
                             dtype=dtype, attention_backend=attention_backend)
            for _ in range(num_layers)])
        self.ln_final = RMSNorm(d_model, device=device, dtype=dtype)
        self.lm_head = Linear(d_model, vocab_size, device=device, dtype=dtype)
        self._fused = None          # models.fused.FusedEngine, created on first use
        self._fused_disabled = False

    # ------------------------------------------------------------ fused path --
    def fused_engine(self):
        """The sm_100a engine if this call can use it, else ``None``."""
        if self._fused_disabled:
            return None
        from . import fused
        if self._fused is None:
            if not fused.eligible(self):
                return None
            self._fused = fused.FusedEngine(self)
        return self._fused if fused.autocast_bf16_active() else None

    def disable_fused(self) -> None:
        """Force the portable PyTorch path (used by parity tests)."""
        self._fused_disabled = True

    def _check_ids(self, input_ids: torch.Tensor) -> None:
        if input_ids.ndim < 1:
            raise ValueError("input_ids must have a sequence dimension")
        if not 0 < input_ids.shape[-1] <= self.context_length:
            raise ValueError("sequence length must be between 1 and context_length")

    def _recompute_blocks(self) -> bool:
        return (self.activation_checkpointing == "block" and self.training
                and torch.is_grad_enabled())

    def hidden_states(self, input_ids: torch.Tensor) -> torch.Tensor:
        """Portable path up to (not including) the final norm."""
        x = self.token_embeddings(input_ids)
        positions = torch.arange(input_ids.shape[-1], device=input_ids.device)
        for layer in self.layers:
            if self._recompute_blocks():
                x = checkpoint(layer, x, positions, use_reentrant=False)
            else:
                x = layer(x, positions)
        return x

    def forward(self, input_ids: torch.Tensor) -> torch.Tensor:
        self._check_ids(input_ids)
        engine = self.fused_engine() if input_ids.is_cuda else None
        if engine is not None:
            return engine.logits(input_ids)
        return self.lm_head(self.ln_final(self.hidden_states(input_ids)))

    def loss(self, input_ids: torch.Tensor, targets: torch.Tensor,
             scale: float = 1.0) -> torch.Tensor:
        """``scale * mean cross-entropy`` of next-token prediction (fp32 scalar)."""
        self._check_ids(input_ids)
        engine = self.fused_engine() if input_ids.is_cuda else None
        if engine is not None:
            return engine.loss(input_ids, targets, scale)
        from ..training.loss import cross_entropy
        logits = self.lm_head(self.ln_final(self.hidden_states(input_ids)))
        loss = cross_entropy(logits.float(), targets)
        if scale == 1.0:
            return loss
        # Divide when the scale is 1/n so accumulation rounds like ``loss / n``.
        inverse = round(1.0 / scale)
        return loss / inverse if inverse > 0 and inverse * scale == 1.0 else loss * scale
