"""Correctness-gated timing of the attention kernels against PyTorch baselines.

Harness in the spirit of the reference's (attention_lab/benchmark.py:190-466):
``run_case`` draws q, k, v from a seeded CPU generator, builds the dense oracle
mask for the spec (and for any dropped schedule blocks), computes a chunked fp32
reference, checks the kernel's output against it (fp16: atol 0.005 / rtol 0.01,
bf16: 0.02 / 0.02) and that the inputs were left untouched, and only then times
the kernel and the baselines - native causal / dense SDPA where the mask allows,
SDPA with an explicit boolean mask otherwise.  ``time_cuda`` captures
``inner_repeats`` calls in a CUDA graph and reports the median of ``repeats``
event-timed replays, so launch overhead is excluded the same way for every
contestant.  FlexAttention (PyTorch's compiled block-mask attention) is an
optional third baseline, requested with ``include_flex``; it is library code
that is only ever timed against, and a failure to compile it is recorded in
the result rather than raised.
"""

from __future__ import annotations

import argparse
import json
import math
import statistics
import time

import torch

from . import flash
from .backward import training_attention
from .masks import BlockSchedule, MaskSpec, compile_mask

TOLERANCE = {torch.float16: (0.005, 0.01), torch.bfloat16: (0.02, 0.02)}
DTYPES = {"fp16": torch.float16, "bf16": torch.bfloat16}


def dense_mask(length: int, spec: MaskSpec, document_ids=None,
               schedule: BlockSchedule | None = None) -> torch.Tensor:
    q = torch.arange(length)[:, None]
    k = torch.arange(length)[None, :]
    mask = torch.ones(length, length, dtype=torch.bool)
    if spec.causal:
        mask &= k <= q
    if spec.window_left is not None:
        mask &= k >= q - spec.window_left
    if spec.window_right is not None:
        mask &= k <= q + spec.window_right
    if spec.same_document:
        labels = torch.as_tensor(list(document_ids))
        mask &= labels[:, None] == labels[None, :]
    if schedule is not None:
        present = torch.zeros(length, length, dtype=torch.bool)
        for row in range(len(schedule.row_ptr) - 1):
            for entry in range(schedule.row_ptr[row], schedule.row_ptr[row + 1]):
                col = schedule.col_idx[entry]
                present[row * schedule.block_q:(row + 1) * schedule.block_q,
                        col * schedule.block_k:(col + 1) * schedule.block_k] = True
        mask &= present
    return mask


def reference_attention(q, k, v, mask, chunk: int = 1024) -> torch.Tensor:
    """fp32 softmax(QK^T/sqrt(D) + mask)V, query-chunked to bound memory."""
    scale = q.shape[-1] ** -0.5
    out = torch.empty(q.shape, dtype=torch.float32, device=q.device)
    kf, vf = k.float(), v.float()
    for start in range(0, q.shape[2], chunk):
        scores = q[:, :, start:start + chunk].float() @ kf.transpose(-1, -2) * scale
        scores = scores.masked_fill(~mask[start:start + chunk], float("-inf"))
        out[:, :, start:start + chunk] = torch.nan_to_num(torch.softmax(scores, -1), 0.0) @ vf
    return out


def time_cuda(function, *, repeats: int = 20, inner_repeats: int = 10, warmup: int = 3) -> dict:
    """Median milliseconds per call over CUDA-graph replays of ``inner_repeats`` calls."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(warmup):
            function()
    torch.cuda.current_stream().wait_stream(stream)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(inner_repeats):
            function()
    samples = []
    for _ in range(repeats):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        graph.replay()
        end.record()
        end.synchronize()
        samples.append(begin.elapsed_time(end) / inner_repeats)
    return {"median_ms": statistics.median(samples), "min_ms": min(samples),
            "max_ms": max(samples), "samples_ms": samples, "mode": "cuda_graph",
            "repeats": repeats, "inner_repeats": inner_repeats}


_FLEX_CACHE: dict = {}


def flex_baseline(q, k, v, spec: MaskSpec, document_ids, want, tolerance, *, contiguous=False,
                  repeats=20, inner_repeats=10) -> dict:
    """Time compiled FlexAttention on the same inputs; never raises.

    The mask predicate is written from the spec alone (it never reads a block
    schedule).  ``contiguous`` hands the library the same fact the interval
    kernel uses - for causal/window masks the key blocks of a query block form
    one contiguous run - through its ``BLOCKS_ARE_CONTIGUOUS`` kernel option
    (reference: attention_lab/benchmark.py:93-102); it is refused for document masks.
    """
    record = {"status": "failed", "correct": False, "contiguous_hint": bool(contiguous)}
    try:
        if contiguous and spec.same_document:
            raise ValueError("the contiguous-block hint needs a mask without documents")
        options = {"BLOCKS_ARE_CONTIGUOUS": True} if contiguous else {}
        from torch.nn.attention.flex_attention import create_block_mask, flex_attention
        length = q.shape[2]
        labels = (None if document_ids is None
                  else torch.as_tensor(list(document_ids), device=q.device))

        def predicate(b, h, qi, ki):
            ok = qi >= 0
            if spec.causal:
                ok = ok & (ki <= qi)
            if spec.window_left is not None:
                ok = ok & (ki >= qi - spec.window_left)
            if spec.window_right is not None:
                ok = ok & (ki <= qi + spec.window_right)
            if spec.same_document:
                ok = ok & (labels[qi] == labels[ki])
            return ok

        begin = time.perf_counter()
        block = create_block_mask(predicate, None, None, length, length, device=q.device,
                                  BLOCK_SIZE=128)
        compiled = _FLEX_CACHE.setdefault("fn", torch.compile(flex_attention, dynamic=False))
        out = compiled(q, k, v, block_mask=block, kernel_options=options)
        torch.cuda.synchronize()
        record["first_call_ms"] = (time.perf_counter() - begin) * 1000
        atol, rtol = tolerance
        record["max_abs_error"] = (out.float() - want).abs().max().item()
        record["correct"] = bool(torch.allclose(out.float(), want, atol=atol, rtol=rtol))
        if record["correct"]:
            timing = time_cuda(lambda: compiled(q, k, v, block_mask=block,
                                                kernel_options=options), repeats=repeats,
                               inner_repeats=inner_repeats)
            record.update(status="passed", latency_ms=timing["median_ms"], timing=timing)
        else:
            record["error"] = "FlexAttention output outside tolerance"
    except Exception as error:
        record.update(error_type=type(error).__name__, error=str(error)[:2000])
    return record


def attention_flops(batch: int, heads: int, length: int, dim: int, mask_fraction: float) -> float:
    return 4.0 * batch * heads * length * length * dim * mask_fraction


def run_case(*, batch: int = 1, heads: int = 8, length: int = 1024, dim: int = 64,
             dtype: str = "bf16", spec: MaskSpec = MaskSpec(causal=True), document_ids=None,
             schedule: BlockSchedule | None = None, implementation: str = "interval",
             block_q: int = 128, block_k: int = 128, use_full_blocks: bool = True, seed: int = 0,
             backward: bool = False, repeats: int = 20, inner_repeats: int = 10,
             warmup: int = 3, time_baselines: bool = True, include_flex: bool = False,
             flex_contiguous: bool = False, device: str = "cuda",
             pipeline: str | None = None) -> dict:
    torch_dtype = DTYPES[dtype]
    generator = torch.Generator().manual_seed(seed)
    q, k, v = (torch.randn(batch, heads, length, dim, generator=generator).to(torch_dtype)
               .to(device) for _ in range(3))
    if implementation == "csr" and schedule is None:
        schedule = compile_mask(length, spec, block_q, block_k,
                                None if document_ids is None else list(document_ids))
    mask = dense_mask(length, spec, document_ids, schedule).to(device)
    before = [t.clone() for t in (q, k, v)]
    torch.cuda.synchronize()
    first_call = time.perf_counter()
    out = flash.attention(q, k, v, schedule, spec, document_ids=document_ids,
                          implementation=implementation, use_full_blocks=use_full_blocks,
                          pipeline=pipeline)
    torch.cuda.synchronize()
    first_call_ms = (time.perf_counter() - first_call) * 1000
    want = reference_attention(q, k, v, mask)
    atol, rtol = TOLERANCE[torch_dtype]
    error = (out.float() - want).abs().max().item()
    correct = bool(torch.allclose(out.float(), want, atol=atol, rtol=rtol)
                   and all(torch.equal(a, b) for a, b in zip(before, (q, k, v))))
    fraction = mask.float().mean().item()
    result = {"batch": batch, "heads": heads, "length": length, "dim": dim, "dtype": dtype,
              "spec": {"causal": spec.causal, "window_left": spec.window_left,
                       "window_right": spec.window_right, "same_document": spec.same_document},
              "implementation": implementation, "block_q": block_q, "block_k": block_k,
              "use_full_blocks": use_full_blocks, "pipeline": pipeline or "default", "seed": seed,
              "correct": correct,
              "max_abs_error": error, "mask_density": fraction, "first_call_ms": first_call_ms,
              "status": "passed" if correct else "failed_correctness"}
    if not correct:
        result["error"] = "kernel output outside tolerance or inputs modified"
        return result
    prepared = flash.prepare_mask(q, schedule, spec, document_ids, implementation, use_full_blocks)
    output = torch.empty_like(q)
    lse = torch.empty(batch, heads, length, dtype=torch.float32, device=device)
    scale = dim ** -0.5
    timing = time_cuda(lambda: flash.flash_fwd(q, k, v, output, lse, prepared, scale, pipeline),
                       repeats=repeats, inner_repeats=inner_repeats, warmup=warmup)
    flops = attention_flops(batch, heads, length, dim, fraction)
    result.update(latency_ms=timing["median_ms"], timing=timing,
                  tflops_effective=flops / timing["median_ms"] / 1e9,
                  tflops_dense_causal_equivalent=(attention_flops(batch, heads, length, dim, 0.5)
                                                  / timing["median_ms"] / 1e9))
    if backward:
        upstream = torch.randn_like(output)
        dq, dk, dv = (torch.empty_like(q) for _ in range(3))
        back = time_cuda(lambda: flash.flash_bwd(q, k, v, output, upstream, lse, dq, dk, dv,
                                                 prepared, scale),
                         repeats=repeats, inner_repeats=max(1, inner_repeats // 2))
        result.update(backward_latency_ms=back["median_ms"],
                      backward_tflops_effective=2.5 * flops / back["median_ms"] / 1e9)
    if time_baselines:
        sdpa = torch.nn.functional.scaled_dot_product_attention
        plain_causal = spec == MaskSpec(causal=True) and schedule is None
        dense = spec == MaskSpec() and schedule is None
        if plain_causal or dense:
            base = time_cuda(lambda: sdpa(q, k, v, is_causal=plain_causal), repeats=repeats,
                             inner_repeats=inner_repeats)
            result["baseline"] = "sdpa_native"
        else:
            base = time_cuda(lambda: sdpa(q, k, v, attn_mask=mask), repeats=repeats,
                             inner_repeats=inner_repeats)
            result["baseline"] = "sdpa_bool_mask"
        result.update(baseline_latency_ms=base["median_ms"],
                      baseline_over_custom=base["median_ms"] / timing["median_ms"])
    if include_flex:
        result["flex"] = flex_baseline(q, k, v, spec, document_ids, want, (atol, rtol),
                                       contiguous=flex_contiguous, repeats=repeats,
                                       inner_repeats=inner_repeats)
    return result


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--heads", type=int, default=16)
    parser.add_argument("--length", type=int, default=4096)
    parser.add_argument("--dim", type=int, default=64, choices=[64, 128])
    parser.add_argument("--dtype", choices=list(DTYPES), default="bf16")
    parser.add_argument("--mask", choices=["causal", "window", "strided", "dense"], default="causal")
    parser.add_argument("--window", type=int, default=255)
    parser.add_argument("--backward", action="store_true")
    parser.add_argument("--seed", type=int, default=0)
    args = parser.parse_args()
    schedule, implementation = None, "interval"
    if args.mask == "causal":
        spec = MaskSpec(causal=True)
    elif args.mask == "window":
        spec = MaskSpec(causal=True, window_left=args.window)
    elif args.mask == "dense":
        spec = MaskSpec()
    else:
        from .masks import strided_schedule
        schedule, spec = strided_schedule(args.length, 128, 4, 2)
        implementation = "csr"
    print(json.dumps(run_case(batch=args.batch, heads=args.heads, length=args.length, dim=args.dim,
                              dtype=args.dtype, spec=spec, schedule=schedule,
                              implementation=implementation, backward=args.backward,
                              seed=args.seed), indent=2))


if __name__ == "__main__":
    main()
