"""Correctness sweep and bounded, paired measurements of the split-KV decode kernel.

Same two stages as the reference's decode study
(attention_lab/cuda_decode/study.py:73-261):

``smoke``   for every kernel variant, 2 dtypes x D in {64, 128} x GQA ratio in
            {1, 2, 4, 8} x cache length in {1, 31, 32, 33, 127, 513} x splits in
            {1, 3, 8} on a ragged batch (lengths 0, 1, half, full), plus three
            special cases: 128 splits with a custom scale, launch on a caller's
            non-default stream, and CUDA-graph replay after the lengths tensor was
            edited in place: 288 + 3 checks per variant - 582 for the two
            CUDA-core schedules the reference has, 873 with the tensor-core one.
``study``   the smoke sweep as a pre-flight, then ten serving-like shapes x three
            input seeds: every (variant, splits) combination is checked against
            an fp32 oracle and timed by CUDA-graph replay, next to SDPA (flash
            backend, GQA enabled) as the library baseline; operator order rotates
            with the seed.  The best observed split is reported per case together
            with the effective KV-cache bandwidth; no claim about a dispatch rule
            on unseen shapes.
"""

from __future__ import annotations

import argparse
import gc
import json
import math
import platform
import statistics
import sys
import time
from pathlib import Path

from .decode import prepare
from .study import write_json

REFERENCE_VARIANTS = ("token", "tile")      # softmax schedules on the CUDA cores
VARIANTS = REFERENCE_VARIANTS + ("mma",)     # + scores and P V on the tensor cores
SMOKE_LENGTHS = (1, 31, 32, 33, 127, 513)
SMOKE_SPLITS = (1, 3, 8)
STUDY_SPLITS = (1, 2, 4, 8, 16, 32)
STUDY_SEEDS = (211, 212, 213)
STUDY_CASES = ((1, 32, 8, 1024, 128), (1, 32, 8, 4096, 128), (1, 32, 8, 16384, 128),
               (1, 32, 8, 65536, 128), (8, 32, 8, 4096, 128), (8, 32, 8, 16384, 128),
               (32, 32, 8, 4096, 128), (1, 16, 1, 16384, 64), (1, 32, 4, 4096, 64),
               (8, 32, 4, 4096, 64))
PAIRED_BASELINES = ("cuda_token_split_1", "cuda_tile_split_1", "sdpa_flash")


def smoke_case_count() -> int:
    """Checks one variant contributes: the grid plus the three special cases."""
    return 2 * 2 * 4 * len(SMOKE_LENGTHS) * len(SMOKE_SPLITS) + 3


def reference(q, k, v, lengths, *, scale=None):
    """fp32 token-level attention that never materialises repeated KV heads."""
    import torch
    batch, heads, dim = q.shape
    kv_heads, capacity = k.shape[1:3]
    queries = q.float().reshape(batch, kv_heads, heads // kv_heads, dim)
    scores = torch.einsum("bhgd,bhnd->bhgn", queries, k.float())
    scores = scores * (dim ** -0.5 if scale is None else scale)
    visible = torch.arange(capacity, device=q.device)[None, :] < lengths[:, None]
    scores = scores.masked_fill(~visible[:, None, None, :], -torch.inf)
    weights = torch.softmax(scores, dim=-1).nan_to_num(0.0)
    return torch.einsum("bhgn,bhnd->bhgd", weights, v.float()).reshape_as(q)


def make_inputs(batch, query_heads, groups, length, dim, dtype, seed, *, ragged=False):
    import torch
    generator = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn(batch, query_heads, dim, device="cuda", dtype=dtype, generator=generator)
    shape = (batch, query_heads // groups, length, dim)
    k = torch.randn(shape, device="cuda", dtype=dtype, generator=generator)
    v = torch.randn(shape, device="cuda", dtype=dtype, generator=generator)
    sizes = [length] * batch
    if ragged:
        if batch != 4:
            raise ValueError("the ragged fixture uses a batch of four")
        sizes = [min(length, value) for value in (0, 1, max(1, length // 2), length)]
    return q, k, v, torch.tensor(sizes, device="cuda", dtype=torch.int32)


def check(actual, expected, dtype) -> dict:
    import torch
    tolerance = 0.02 if dtype == torch.bfloat16 else 0.004
    torch.testing.assert_close(actual.float(), expected, atol=tolerance, rtol=tolerance)
    delta = actual.float() - expected
    return {"max_abs_error": delta.abs().max().item(),
            "rms_error": delta.square().mean().sqrt().item(),
            "finite": bool(torch.isfinite(actual).all().item()), "atol": tolerance,
            "rtol": tolerance}


def smoke_variant(output: Path, deadline: float, variant: str):
    import torch
    records = []
    for dtype in (torch.float16, torch.bfloat16):
        for dim in (64, 128):
            for groups in (1, 2, 4, 8):
                for length in SMOKE_LENGTHS:
                    if time.monotonic() >= deadline:
                        return records, "time_budget_exhausted"
                    inputs = make_inputs(4, 8, groups, length, dim, dtype, 2027, ragged=True)
                    expected = reference(*inputs)
                    for splits in SMOKE_SPLITS:
                        operation = prepare(*inputs, splits=splits, variant=variant)
                        records.append({"dtype": str(dtype), "dim": dim, "groups": groups,
                                        "length": length, "splits": splits,
                                        **check(operation(), expected, dtype)})
                write_json(output / "correctness.json", records)
    # every merge lane and the custom-scale path: most of the 128 partitions are
    # empty and one request is empty altogether
    inputs = make_inputs(4, 8, 2, 33, 128, torch.float16, 93, ragged=True)
    operation = prepare(*inputs, splits=128, scale=0.37, variant=variant)
    records.append({"case": "maximum_splits_custom_scale", "splits": 128, "scale": 0.37,
                    **check(operation(), reference(*inputs, scale=0.37), inputs[0].dtype)})
    # the launch must land on the caller's stream; the event dependency makes the
    # check independent of default-stream synchronisation
    inputs = make_inputs(4, 8, 4, 513, 64, torch.bfloat16, 91, ragged=True)
    operation = prepare(*inputs, splits=8, variant=variant)
    expected = reference(*inputs)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        result = operation().clone()
    torch.cuda.current_stream().wait_stream(stream)
    records.append({"case": "non_default_stream", **check(result, expected, inputs[0].dtype)})
    # replay after editing the lengths in place: captured launches must read the
    # metadata at run time, including all-empty and partly filled partitions
    with torch.cuda.stream(stream):
        operation()
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        operation()
    inputs[3].copy_(torch.tensor([513, 256, 0, 3], device="cuda", dtype=torch.int32))
    graph.replay()
    torch.cuda.synchronize()
    records.append({"case": "graph_replay_changed_lengths",
                    **check(operation.output, reference(*inputs), inputs[0].dtype)})
    write_json(output / "correctness.json", records)
    return records, "completed"


def smoke(output: Path, deadline: float):
    records = []
    for variant in VARIANTS:
        cases, status = smoke_variant(output / variant, deadline, variant)
        records.extend({"variant": variant, **case} for case in cases)
        write_json(output / "correctness.json", records)
        if status != "completed":
            return records, status
    return records, "completed"


def geomean(values):
    values = list(values)
    return math.exp(statistics.mean(math.log(v) for v in values)) if values else None


L2_BYTES = 126 * 1024 * 1024


def cold_copies(cache_bytes: int) -> int:
    """Cache copies to rotate over so that no call finds its operands in L2."""
    return max(1, min(64, math.ceil(2 * L2_BYTES / max(1, cache_bytes))))


def time_cold(build, copies: int, *, repeats: int = 12) -> dict:
    """``build(i)`` returns the zero-argument operator for cache copy ``i``; one CUDA
    graph runs all copies back to back and the median per-call time is reported."""
    import torch
    operators = [build(i) for i in range(copies)]
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for _ in range(2):
            for operator in operators:
                operator()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for operator in operators:
                operator()
        graph.replay()
        stream.synchronize()
        samples = []
        for _ in range(repeats):
            begin, end = (torch.cuda.Event(enable_timing=True) for _ in range(2))
            begin.record(stream)
            graph.replay()
            end.record(stream)
            end.synchronize()
            samples.append(begin.elapsed_time(end) / copies)
    torch.cuda.current_stream().wait_stream(stream)
    return {"median_ms": statistics.median(samples), "min_ms": min(samples),
            "max_ms": max(samples), "copies": copies, "repeats": repeats, "mode": "cuda_graph_cold"}


def summarise_case(record: dict) -> None:
    """Best split overall and per variant, ratios, cache bandwidth - from recorded timings."""
    timings = record["timings"]
    ours = [name for name in timings if name.startswith("cuda_")]
    best = min(ours, key=lambda name: timings[name]["median_ms"])
    best_ms = timings[best]["median_ms"]
    by_variant = {variant: min((n for n in ours if n.startswith(f"cuda_{variant}_")),
                               key=lambda name: timings[name]["median_ms"])
                  for variant in VARIANTS
                  if any(n.startswith(f"cuda_{variant}_") for n in ours)}
    record.update({
        "best_observed": best, "best_observed_by_variant": by_variant,
        "best_tile_over_best_token": (timings[by_variant["token"]]["median_ms"]
                                      / timings[by_variant["tile"]]["median_ms"]),
        "tile_over_token_same_split": {
            str(s): (timings[f"cuda_token_split_{s}"]["median_ms"]
                     / timings[f"cuda_tile_split_{s}"]["median_ms"])
            for s in STUDY_SPLITS if f"cuda_token_split_{s}" in timings
            and f"cuda_tile_split_{s}" in timings},
        "speedups": {name: timing["median_ms"] / best_ms for name, timing in timings.items()
                     if name in PAIRED_BASELINES},
        "effective_kv_bandwidth_gbs": record["cache_bytes"] / (best_ms * 1e6)})


def benchmark(output: Path, deadline: float):
    import torch
    import torch.nn.functional as F
    from torch.nn.attention import SDPBackend, sdpa_kernel

    from .benchmark import time_cuda

    write_json(output / "plan.json", {
        "cases": STUDY_CASES, "seeds": STUDY_SEEDS, "splits": STUDY_SPLITS, "variants": VARIANTS,
        "baselines": {"sdpa_flash": "scaled_dot_product_attention, flash backend, enable_gqa"},
        "selection": "best observed split per case; no claim about dispatch on unseen shapes"})
    records = []
    for index, (batch, heads, groups, length, dim) in enumerate(STUDY_CASES):
        for seed in STUDY_SEEDS:
            if time.monotonic() >= deadline:
                return records, "time_budget_exhausted"
            inputs = make_inputs(batch, heads, groups, length, dim, torch.bfloat16, seed)
            q, k, v, _ = inputs
            expected = reference(*inputs)
            record = {"batch": batch, "query_heads": heads, "kv_heads": heads // groups,
                      "groups": groups, "length": length, "dim": dim, "seed": seed,
                      "dtype": "torch.bfloat16", "timings": {}, "checks": {}, "setup": {},
                      "cache_bytes": (k.numel() + v.numel()) * k.element_size()}
            operators = {}
            for variant in VARIANTS:
                for splits in STUDY_SPLITS:
                    torch.cuda.synchronize()
                    begin = time.perf_counter()
                    operation = prepare(*inputs, splits=splits, variant=variant)
                    torch.cuda.synchronize()
                    prepared = time.perf_counter()
                    result = operation()
                    torch.cuda.synchronize()
                    name = f"cuda_{variant}_split_{splits}"
                    record["setup"][name] = {"prepare_ms": (prepared - begin) * 1000,
                                             "first_call_ms": (time.perf_counter() - prepared) * 1000}
                    record["checks"][name] = check(result, expected, q.dtype)
                    operators[name] = operation

            def flash():
                with sdpa_kernel(SDPBackend.FLASH_ATTENTION):
                    return F.scaled_dot_product_attention(q.unsqueeze(2), k, v,
                                                          enable_gqa=True).squeeze(2)

            try:
                record["checks"]["sdpa_flash"] = check(flash(), expected, q.dtype)
                operators["sdpa_flash"] = flash
            except (RuntimeError, NotImplementedError, AssertionError) as error:
                record.setdefault("unsupported_baselines", {})["sdpa_flash"] = str(error)
            names = list(operators)
            offset = seed % len(names)          # no operator always runs first
            for name in names[offset:] + names[:offset]:
                record["timings"][name] = time_cuda(operators[name], warmup=3, repeats=12,
                                                    inner_repeats=10)
            record["scratch_bytes"] = min(
                (operators[n] for n in names if n.startswith("cuda_")),
                key=lambda op: record["timings"][f"cuda_{op.variant}_split_{op.splits}"]
                ["median_ms"]).scratch_bytes
            summarise_case(record)
            # cold-L2 figures for the best split of each variant and the baseline
            copies = cold_copies(record["cache_bytes"])
            caches = [(k, v)] + [(torch.randn_like(k), torch.randn_like(v))
                                 for _ in range(copies - 1)]
            lengths = inputs[3]
            record["cold_timings"] = {}
            for variant, name in record["best_observed_by_variant"].items():
                splits = operators[name].splits
                record["cold_timings"][name] = time_cold(
                    lambda i, s=splits, w=variant: prepare(q, *caches[i], lengths, splits=s,
                                                           variant=w), copies)
            if "sdpa_flash" in operators:
                def flash_on(i):
                    kc, vc = caches[i]

                    def call():
                        with sdpa_kernel(SDPBackend.FLASH_ATTENTION):
                            return F.scaled_dot_product_attention(q.unsqueeze(2), kc, vc,
                                                                  enable_gqa=True).squeeze(2)
                    return call
                record["cold_timings"]["sdpa_flash"] = time_cold(flash_on, copies)
            cold_best = min((n for n in record["cold_timings"] if n.startswith("cuda_")),
                            key=lambda n: record["cold_timings"][n]["median_ms"])
            cold_ms = record["cold_timings"][cold_best]["median_ms"]
            record.update(cold_best=cold_best,
                          cold_kv_bandwidth_gbs=record["cache_bytes"] / (cold_ms * 1e6))
            if "sdpa_flash" in record["cold_timings"]:
                record["cold_sdpa_flash_over_best"] = (
                    record["cold_timings"]["sdpa_flash"]["median_ms"] / cold_ms)
            del caches
            records.append(record)
            write_json(output / "cases" / f"case-{index:02d}-seed-{seed}.json", record)
            write_json(output / "benchmark.json", records)
            del operators, operation, inputs, q, k, v, expected
            gc.collect()
            torch.cuda.empty_cache()
    return records, "completed"


def study_summary(records: list[dict]) -> dict:
    paired = {}
    for baseline in PAIRED_BASELINES:
        cases = [case for case in records if baseline in case["speedups"]]
        paired[baseline] = {
            "paired_cases": len(cases), "unpaired_completed_cases": len(records) - len(cases),
            "distinct_shapes": len({(c["batch"], c["query_heads"], c["groups"], c["length"],
                                     c["dim"]) for c in cases}),
            "geomean_speedup": geomean(c["speedups"][baseline] for c in cases)}
    return {"planned_cases": len(STUDY_CASES) * len(STUDY_SEEDS),
            "geomean_best_tile_over_best_token": geomean(c["best_tile_over_best_token"]
                                                         for c in records),
            "geomean_effective_kv_bandwidth_gbs": geomean(c["effective_kv_bandwidth_gbs"]
                                                          for c in records),
            "paired_baselines_best_observed": paired}


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--stage", choices=("smoke", "study"), default="smoke")
    parser.add_argument("--output-dir", type=Path, required=True)
    parser.add_argument("--time-budget-seconds", type=int, default=600)
    parser.add_argument("--execute", action="store_true")
    args = parser.parse_args()
    if args.time_budget_seconds <= 0:
        parser.error("time budget must be positive")
    if not args.execute:
        print(json.dumps({"stage": args.stage, "output_dir": str(args.output_dir),
                          "time_budget_seconds": args.time_budget_seconds, "execute": False,
                          "smoke_checks": len(VARIANTS) * smoke_case_count()}))
        return
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("CUDA GPU required")
    args.output_dir.mkdir(parents=True, exist_ok=True)
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    started = time.monotonic()
    deadline = started + args.time_budget_seconds
    write_json(args.output_dir / "environment.json", {
        "python": platform.python_version(), "torch": torch.__version__,
        "cuda": torch.version.cuda, "gpu": torch.cuda.get_device_name(),
        "timing_scope": ("warmed CUDA graphs; all scratch traffic and the split merge included; "
                         "Python dispatch and workspace allocation excluded"),
        "attention_scope": ("one query token, bf16/fp16 contiguous KV, per-request valid lengths, "
                            "GQA without repeating KV heads")})
    planned_smoke = len(VARIANTS) * smoke_case_count()
    try:
        preflight = None
        if args.stage == "smoke":
            records, status = smoke(args.output_dir, deadline)
        else:
            checks, status = smoke(args.output_dir / "preflight", deadline)
            preflight = {"status": status, "cases": len(checks), "planned_cases": planned_smoke,
                         "max_abs_error": max((c["max_abs_error"] for c in checks), default=None)}
            write_json(args.output_dir / "preflight" / "summary.json", preflight)
            records = []
            if status == "completed":
                records, status = benchmark(args.output_dir, deadline)
        summary = {"status": status, "stage": args.stage, "cases": len(records),
                   "wall_seconds": time.monotonic() - started}
        if args.stage == "study":
            summary.update(preflight=preflight, **study_summary(records))
        else:
            summary.update(planned_cases=planned_smoke,
                           max_abs_error=max((c["max_abs_error"] for c in records), default=None))
        write_json(args.output_dir / "summary.json", summary)
        print(json.dumps(summary))
        if status != "completed":
            sys.exit(2)      # partial records are kept but never read as a pass
    except Exception as error:
        write_json(args.output_dir / "summary.json", {
            "status": "failed", "stage": args.stage, "error": f"{type(error).__name__}: {error}",
            "wall_seconds": time.monotonic() - started})
        raise


if __name__ == "__main__":
    main()
