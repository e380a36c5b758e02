"""Cross-entropy and perplexity over the last dimension (portable path).

Numerically stable log-sum-exp form, mean over all positions, as in the reference
(src/llmlab/training/loss.py:4-29).  The fused sm_100a equivalent is
``ops.functional.cross_entropy_rows``.
"""

import torch


def cross_entropy(inputs: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    shifted = inputs - inputs.amax(dim=-1, keepdim=True)
    log_normalizer = shifted.exp().sum(dim=-1).log()
    picked = shifted.gather(-1, targets.unsqueeze(-1)).squeeze(-1)
    return (log_normalizer - picked).mean()


def perplexity(inputs: torch.Tensor, targets: torch.Tensor) -> torch.Tensor:
    return cross_entropy(inputs, targets).exp()
