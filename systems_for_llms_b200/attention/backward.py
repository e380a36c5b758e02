"""Differentiable block-sparse attention: ``training_attention``.

Autograd wrapper over the sm_100a forward and backward kernels with the
interface of the reference (attention_lab/backward.py:180-218): inputs
``[B, H, N, D]`` fp16/bf16, a ``MaskSpec`` plus optional document labels,
``implementation`` in {"auto", "csr", "interval"} (auto = CSR when documents are
involved, interval otherwise), first derivatives only.  Forward saves
(q, k, v, o, lse); backward computes delta = rowsum(O dO), dQ over the forward
schedule and dK/dV over its transpose, each written once in the input dtype.
A caller-supplied ``schedule`` (for example a strided block pattern) is honoured
in both directions.
"""

from __future__ import annotations

import torch
from torch.autograd.function import once_differentiable

from . import flash
from .masks import BlockSchedule, MaskSpec


class StructuredAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, mask, scale):
        B, H, N, D = q.shape
        out = torch.empty_like(q)
        lse = torch.empty(B, H, N, dtype=torch.float32, device=q.device)
        flash.flash_fwd(q, k, v, out, lse, mask, scale)
        ctx.save_for_backward(q, k, v, out, lse)
        ctx.mask, ctx.scale = mask, scale
        return out

    @staticmethod
    @once_differentiable
    def backward(ctx, upstream):
        q, k, v, out, lse = ctx.saved_tensors
        upstream = upstream.contiguous()
        dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
        flash.flash_bwd(q, k, v, out, upstream, lse, dq, dk, dv, ctx.mask, ctx.scale)
        return dq, dk, dv, None, None


def training_attention(q, k, v, spec: MaskSpec = MaskSpec(), document_ids=None, *,
                       block_q: int = 128, block_k: int = 128, implementation: str = "auto",
                       schedule: BlockSchedule | None = None, scale: float | None = None,
                       num_warps: int = 4, num_stages: int = 2):
    """Attention output with gradients for q, k and v.

    ``block_q`` / ``block_k`` set the granularity at which a CSR schedule is
    compiled when none is given; the kernels always walk 128 x 128 tiles and keep
    finer structure in per-tile bitmaps.  ``num_warps`` / ``num_stages`` exist for
    signature compatibility and are ignored.
    """
    flash._check_inputs(q, k, v, allow_grad=True)
    if implementation not in ("auto", "csr", "interval"):
        raise ValueError("implementation must be 'auto', 'csr' or 'interval'")
    if implementation == "auto":
        implementation = "csr" if (spec.same_document or schedule is not None) else "interval"
    if schedule is None and implementation == "csr":
        from .masks import compile_mask
        schedule = compile_mask(q.shape[2], spec, block_q, block_k, flash._doc_list(document_ids))
    mask = flash.prepare_mask(q, schedule, spec, document_ids, implementation)
    D = q.shape[-1]
    return StructuredAttention.apply(q, k, v, mask, D ** -0.5 if scale is None else scale)
