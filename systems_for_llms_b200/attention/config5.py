"""Block-sparse flash attention forward+backward table against dense-causal SDPA.

One process measures, for batch 8, 16 heads, head dimension 64, bf16 and sequence
lengths 1024 / 4096 / 16384:

* this library's forward and backward kernels under three block masks - causal,
  causal sliding window (the interval schedule) and strided (a CSR schedule that
  keeps every ``period``-th key tile plus a local band),
* PyTorch ``scaled_dot_product_attention(is_causal=True)`` forward and
  forward+backward on the same device as the dense-causal yardstick.

Every mask is first checked at batch 1, 2 heads against a dense fp32 oracle
(output, dQ, dK, dV; tolerances of the reference harness,
attention_lab/backward_study.py:47).  Timing follows the reference's method
(attention_lab/benchmark.py:42-84: CUDA-graph replay, median of event-timed
repeats) with one change: the graph cycles through enough independent input sets
that consecutive calls never find their operands in the 126 MB L2.

FLOP accounting: a forward pass is ``4 B H N^2 D x density`` and a backward pass
2.5 times that (five products against two), where density is the fraction of the
N x N score matrix the mask keeps; "dense-causal equivalent" uses density 0.5
whatever the mask keeps, i.e. it is the rate a dense-causal kernel would need to
finish in the same time.

    python -m systems_for_llms_b200.attention.config5 --output config5.json
"""

from __future__ import annotations

import argparse
import json
import math
import statistics
from pathlib import Path

L2_BYTES = 126 * 1024 * 1024
LENGTHS = (1024, 4096, 16384)
MASKS = ("causal", "window", "strided")
BACKWARD_TOLERANCE = (0.025, 0.035)     # bf16 atol, rtol


def mask_for(name: str, length: int, window: int = 1023):
    """``(spec, schedule, implementation)`` of a named mask."""
    from .masks import MaskSpec, strided_schedule
    if name == "causal":
        return MaskSpec(causal=True), None, "interval"
    if name == "window":
        return MaskSpec(causal=True, window_left=min(window, length - 1)), None, "interval"
    if name == "strided":
        schedule, spec = strided_schedule(length, 128, 4, 2)
        return spec, schedule, "csr"
    raise ValueError(f"unknown mask {name!r}")


def flops(batch: int, heads: int, length: int, dim: int, density: float) -> float:
    return 4.0 * batch * heads * length * length * dim * density


def input_sets(working_set_bytes: int) -> int:
    """Independent operand sets needed so that a call's data was evicted from L2."""
    return max(1, min(16, math.ceil(2 * L2_BYTES / max(1, working_set_bytes))))


def time_graph(calls, *, repeats: int = 15, warmup: int = 2) -> dict:
    """Median milliseconds per call of a CUDA graph that runs every callable once."""
    import torch
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            for call in calls:
                call()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for call in calls:
                call()
        graph.replay()
        stream.synchronize()
        samples = []
        for _ in range(repeats):
            begin, end = (torch.cuda.Event(enable_timing=True) for _ in range(2))
            begin.record(stream)
            graph.replay()
            end.record(stream)
            end.synchronize()
            samples.append(begin.elapsed_time(end) / len(calls))
    torch.cuda.current_stream().wait_stream(stream)
    return {"median_ms": statistics.median(samples), "min_ms": min(samples),
            "max_ms": max(samples), "calls_per_replay": len(calls), "repeats": repeats}


def check_mask(name: str, length: int, dim: int, seed: int = 5) -> dict:
    """Output and gradients at batch 1, 2 heads against the dense fp32 oracle."""
    import torch
    from .backward import training_attention
    from .benchmark import dense_mask
    spec, schedule, implementation = mask_for(name, length)
    generator = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(1, 2, length, dim, generator=generator).to(torch.bfloat16).cuda()
               .requires_grad_() for _ in range(3))
    upstream = torch.randn(1, 2, length, dim, generator=generator).to(torch.bfloat16).cuda()
    out = training_attention(q, k, v, spec, None, block_q=128, block_k=128,
                             implementation=implementation, schedule=schedule)
    grads = torch.autograd.grad(out, (q, k, v), upstream)
    mask = dense_mask(length, spec, None, schedule).cuda()
    qf, kf, vf = (t.detach().float().requires_grad_() for t in (q, k, v))
    want_grads = [torch.zeros_like(qf) for _ in range(3)]
    want_out = torch.empty_like(qf)
    chunk = 2048
    for start in range(0, length, chunk):          # query chunks bound the score matrix
        scores = qf[:, :, start:start + chunk] @ kf.transpose(-1, -2) * dim ** -0.5
        scores = scores.masked_fill(~mask[start:start + chunk], float("-inf"))
        part = torch.nan_to_num(torch.softmax(scores, -1), 0.0) @ vf
        want_out[:, :, start:start + chunk] = part.detach()
        for total, piece in zip(want_grads, torch.autograd.grad(
                part, (qf, kf, vf), upstream[:, :, start:start + chunk].float())):
            total += piece
    atol, rtol = BACKWARD_TOLERANCE
    errors = {}
    for label, got, want in zip(("out", "dq", "dk", "dv"), (out, *grads),
                                (want_out, *want_grads)):
        errors[label] = {"max_abs_error": (got.float() - want).abs().max().item(),
                         "correct": bool(torch.allclose(got.float(), want, atol=atol, rtol=rtol))}
    return {"mask": name, "length": length, "density": mask.float().mean().item(),
            "errors": errors, "correct": all(e["correct"] for e in errors.values())}


def time_case(name: str, length: int, *, batch: int, heads: int, dim: int, seed: int = 0) -> dict:
    """Forward and backward latency of this library's kernels under one mask."""
    import torch
    from . import flash
    spec, schedule, implementation = mask_for(name, length)
    element = 2
    tensor_bytes = batch * heads * length * dim * element
    sets = input_sets(9 * tensor_bytes)     # q k v o do dq dk dv (+ statistics)
    generator = torch.Generator(device="cuda").manual_seed(seed)
    shape = (batch, heads, length, dim)

    def fresh():
        return torch.randn(shape, generator=generator, device="cuda", dtype=torch.bfloat16)

    data = []
    for _ in range(sets):
        q, k, v, upstream = fresh(), fresh(), fresh(), fresh()
        out = torch.empty_like(q)
        lse = torch.empty(batch, heads, length, dtype=torch.float32, device="cuda")
        grads = tuple(torch.empty_like(q) for _ in range(3))
        data.append((q, k, v, out, lse, upstream, grads))
    prepared = flash.prepare_mask(data[0][0], schedule, spec, None, implementation)
    scale = dim ** -0.5
    forward = [lambda s=s: flash.flash_fwd(s[0], s[1], s[2], s[3], s[4], prepared, scale)
               for s in data]
    for call in forward:
        call()
    backward = [lambda s=s: flash.flash_bwd(s[0], s[1], s[2], s[3], s[5], s[4], *s[6], prepared,
                                            scale) for s in data]
    fwd = time_graph(forward)
    bwd = time_graph(backward)
    return {"mask": name, "length": length, "batch": batch, "heads": heads, "dim": dim,
            "input_sets": sets, "forward_ms": fwd["median_ms"], "backward_ms": bwd["median_ms"],
            "forward_timing": fwd, "backward_timing": bwd}


def time_sdpa(length: int, *, batch: int, heads: int, dim: int, seed: int = 0) -> dict:
    """Dense-causal ``scaled_dot_product_attention`` forward and forward+backward."""
    import torch
    import torch.nn.functional as F
    tensor_bytes = batch * heads * length * dim * 2
    sets = input_sets(9 * tensor_bytes)
    generator = torch.Generator(device="cuda").manual_seed(seed)
    shape = (batch, heads, length, dim)
    data = []
    for _ in range(sets):
        q, k, v = (torch.randn(shape, generator=generator, device="cuda", dtype=torch.bfloat16)
                   .requires_grad_() for _ in range(3))
        upstream = torch.randn(shape, generator=generator, device="cuda", dtype=torch.bfloat16)
        data.append((q, k, v, upstream))

    def forward_only(s):
        with torch.no_grad():
            return F.scaled_dot_product_attention(s[0], s[1], s[2], is_causal=True)

    def forward_backward(s):
        out = F.scaled_dot_product_attention(s[0], s[1], s[2], is_causal=True)
        return torch.autograd.grad(out, (s[0], s[1], s[2]), s[3])

    fwd = time_graph([lambda s=s: forward_only(s) for s in data])
    both = time_graph([lambda s=s: forward_backward(s) for s in data])
    return {"length": length, "input_sets": sets, "forward_ms": fwd["median_ms"],
            "forward_backward_ms": both["median_ms"], "forward_timing": fwd,
            "forward_backward_timing": both}


def tabulate(records: dict, *, batch: int, heads: int, dim: int) -> str:
    """Markdown table from the ``run`` result (pure function of its argument)."""
    lines = ["| N | mask | density | fwd ms | fwd+bwd ms | fwd TFLOP/s | fwd+bwd TFLOP/s | "
             "dense-causal-equivalent fwd+bwd TFLOP/s | SDPA dense causal fwd / fwd+bwd ms | "
             "SDPA time / ours: fwd, fwd+bwd |",
             "|---:|---|---:|---:|---:|---:|---:|---:|---:|---:|"]
    sdpa = {row["length"]: row for row in records["sdpa"]}
    checks = {(row["mask"], row["length"]): row for row in records["checks"]}
    for row in records["cases"]:
        length, name = row["length"], row["mask"]
        density = checks[(name, length)]["density"]
        both = row["forward_ms"] + row["backward_ms"]
        work = flops(batch, heads, length, dim, density)
        base = sdpa[length]
        lines.append(
            f"| {length} | {name} | {density:.3f} | {row['forward_ms']:.3f} | {both:.3f} | "
            f"{work / row['forward_ms'] / 1e9:.0f} | {3.5 * work / both / 1e9:.0f} | "
            f"{3.5 * flops(batch, heads, length, dim, 0.5) / both / 1e9:.0f} | "
            f"{base['forward_ms']:.3f} / {base['forward_backward_ms']:.3f} | "
            f"{base['forward_ms'] / row['forward_ms']:.2f}, "
            f"{base['forward_backward_ms'] / both:.2f} |")
    return "\n".join(lines)


def run(*, lengths=LENGTHS, masks=MASKS, batch: int = 8, heads: int = 16, dim: int = 64,
        check=check_mask, time_ours=time_case, time_baseline=time_sdpa) -> dict:
    """Checks, times and tabulates; the three workers can be replaced for testing."""
    records = {"batch": batch, "heads": heads, "dim": dim, "dtype": "bf16",
               "checks": [], "cases": [], "sdpa": []}
    for length in lengths:
        for name in masks:
            verdict = check(name, length, dim)
            records["checks"].append(verdict)
            if not verdict["correct"]:
                raise RuntimeError(f"mask {name} at N={length} failed its correctness check: "
                                   f"{verdict['errors']}")
    for length in lengths:
        records["sdpa"].append(time_baseline(length, batch=batch, heads=heads, dim=dim))
        for name in masks:
            records["cases"].append(time_ours(name, length, batch=batch, heads=heads, dim=dim))
    records["table"] = tabulate(records, batch=batch, heads=heads, dim=dim)
    return records


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--output", type=Path, default=None)
    parser.add_argument("--lengths", type=int, nargs="+", default=list(LENGTHS))
    parser.add_argument("--masks", nargs="+", choices=MASKS, default=list(MASKS))
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--heads", type=int, default=16)
    parser.add_argument("--dim", type=int, default=64, choices=(64, 128))
    args = parser.parse_args()
    import torch
    from ..ops.gemm import check_status
    records = run(lengths=tuple(args.lengths), masks=tuple(args.masks), batch=args.batch,
                  heads=args.heads, dim=args.dim)
    torch.cuda.synchronize()
    check_status()
    records["gpu"] = torch.cuda.get_device_name()
    if args.output is not None:
        args.output.parent.mkdir(parents=True, exist_ok=True)
        args.output.write_text(json.dumps(records, indent=2) + "\n")
    print(records["table"])


if __name__ == "__main__":
    main()
