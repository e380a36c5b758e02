"""CPU validation of the mask compiler: schedules against dense masks, and a
block-schedule interpreter against dense attention in fp64.

Two checks, as in the reference's validator (attention_lab/validate.py:15-122):

* ``semantic_cases`` - for a grid of specs, lengths and tile shapes, the compiled
  schedule must list exactly the tiles that contain an allowed (q, k) pair and
  flag exactly the tiles in which every pair is allowed;
* ``interpreter_cases`` - ``interpret_schedule`` evaluates attention tile by tile
  the way the GPU kernels do (online softmax, full tiles unmasked, partial tiles
  through the scalar predicate) with differentiable fp64 tensor ops; output and
  input gradients must match masked dense attention to round-off.

Runs without a GPU: ``python -m systems_for_llms_b200.attention.validate``.
"""

from __future__ import annotations

import itertools
import json
import math
import random

import torch

from .masks import MaskSpec, allows, compile_mask


def dense_allowed(length: int, spec: MaskSpec, documents=None) -> list[list[bool]]:
    return [[allows(q, k, spec, documents) for k in range(length)] for q in range(length)]


def semantic_cases() -> dict:
    specs = [MaskSpec(), MaskSpec(causal=True), MaskSpec(causal=True, window_left=7),
             MaskSpec(window_left=5, window_right=3), MaskSpec(window_right=0),
             MaskSpec(causal=True, window_left=0), MaskSpec(causal=True, same_document=True),
             MaskSpec(window_left=9, same_document=True)]
    rng = random.Random(0)
    checked = 0
    for spec, length, (bq, bk) in itertools.product(specs, (5, 16, 31, 40, 64),
                                                    ((4, 4), (8, 4), (4, 16), (16, 16), (8, 32))):
        documents = [rng.randrange(3) for _ in range(length)] if spec.same_document else None
        mask = dense_allowed(length, spec, documents)
        schedule = compile_mask(length, spec, bq, bk, documents)
        for row in range(-(-length // bq)):
            stored = dict(zip(schedule.col_idx[schedule.row_ptr[row]:schedule.row_ptr[row + 1]],
                              schedule.full_blocks[schedule.row_ptr[row]:schedule.row_ptr[row + 1]]))
            for col in range(-(-length // bk)):
                cells = [mask[q][k] for q in range(row * bq, min(length, (row + 1) * bq))
                         for k in range(col * bk, min(length, (col + 1) * bk))]
                if (col in stored) != any(cells) or (col in stored and stored[col] != all(cells)):
                    raise AssertionError(f"schedule mismatch: {spec} N={length} tile {bq}x{bk} "
                                         f"({row}, {col})")
        checked += 1
    return {"semantic_cases": checked}


def interpret_schedule(q, k, v, schedule, spec: MaskSpec, documents=None) -> torch.Tensor:
    """Tile-by-tile attention over a schedule with online softmax (differentiable)."""
    length, dim = q.shape[-2], q.shape[-1]
    scale = dim ** -0.5
    rows = []
    for row in range(len(schedule.row_ptr) - 1):
        q_lo, q_hi = row * schedule.block_q, min(length, (row + 1) * schedule.block_q)
        q_tile = q[..., q_lo:q_hi, :]
        running_max = torch.full(q_tile.shape[:-1], -math.inf, dtype=q.dtype)
        normalizer = torch.zeros(q_tile.shape[:-1], dtype=q.dtype)
        accumulator = torch.zeros_like(q_tile)
        for entry in range(schedule.row_ptr[row], schedule.row_ptr[row + 1]):
            col = schedule.col_idx[entry]
            k_lo, k_hi = col * schedule.block_k, min(length, (col + 1) * schedule.block_k)
            scores = q_tile @ k[..., k_lo:k_hi, :].transpose(-1, -2) * scale
            if not schedule.full_blocks[entry]:
                keep = torch.tensor([[allows(a, b, spec, documents) for b in range(k_lo, k_hi)]
                                     for a in range(q_lo, q_hi)])
                scores = scores.masked_fill(~keep, -math.inf)
            new_max = torch.maximum(running_max, scores.amax(-1))
            safe = torch.where(torch.isinf(new_max), torch.zeros_like(new_max), new_max)
            alpha = torch.exp(running_max - safe)
            alpha = torch.where(torch.isinf(running_max), torch.zeros_like(alpha), alpha)
            weights = torch.exp(scores - safe[..., None])
            normalizer = normalizer * alpha + weights.sum(-1)
            accumulator = accumulator * alpha[..., None] + weights @ v[..., k_lo:k_hi, :]
            running_max = new_max
        denominator = torch.where(normalizer > 0, normalizer, torch.ones_like(normalizer))
        rows.append(accumulator / denominator[..., None])
    return torch.cat(rows, dim=-2)


def interpreter_cases() -> dict:
    specs = [MaskSpec(causal=True), MaskSpec(causal=True, window_left=6),
             MaskSpec(window_left=4, window_right=4), MaskSpec(causal=True, same_document=True)]
    worst_out = worst_grad = 0.0
    count = 0
    generator = torch.Generator().manual_seed(0)
    for spec, length, (bq, bk) in itertools.product(specs, (19, 32), ((4, 8), (8, 8), (16, 4))):
        documents = [i * 3 // length for i in range(length)] if spec.same_document else None
        q, k, v = (torch.randn(2, length, 8, dtype=torch.float64, generator=generator,
                               requires_grad=True) for _ in range(3))
        schedule = compile_mask(length, spec, bq, bk, documents)
        got = interpret_schedule(q, k, v, schedule, spec, documents)
        mask = torch.tensor(dense_allowed(length, spec, documents))
        scores = (q @ k.transpose(-1, -2) * 8 ** -0.5).masked_fill(~mask, -math.inf)
        want = torch.softmax(scores, -1) @ v
        upstream = torch.randn(got.shape, dtype=torch.float64, generator=generator)
        grads_got = torch.autograd.grad(got, (q, k, v), upstream, retain_graph=True)
        grads_want = torch.autograd.grad(want, (q, k, v), upstream)
        worst_out = max(worst_out, (got - want).abs().max().item())
        worst_grad = max(worst_grad, max((a - b).abs().max().item()
                                         for a, b in zip(grads_got, grads_want)))
        count += 1
    if worst_out > 1e-12 or worst_grad > 1e-12:
        raise AssertionError(f"interpreter mismatch: out {worst_out}, grad {worst_grad}")
    return {"interpreter_cases": count, "max_output_error": worst_out,
            "max_gradient_error": worst_grad}


def main() -> None:
    report = {**semantic_cases(), **interpreter_cases()}
    print(json.dumps(report, indent=2))


if __name__ == "__main__":
    main()
