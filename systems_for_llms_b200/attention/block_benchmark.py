"""Attention substitutions measured inside one inference Transformer block.

Every variant runs the same surrounding operators on the same weights: LayerNorm,
QKV projection, attention, output projection + residual, LayerNorm, GELU MLP +
residual, all bf16 without bias - the block of the reference's study
(attention_lab/block_benchmark.py:25-304).  Only the attention call changes:
this package's interval kernel, PyTorch SDPA, and (optionally) compiled
FlexAttention.  Each variant is first checked against the block computed with
explicit-mask math attention, then the whole block and the attention call alone
are timed as CUDA-graph replays; the Amdahl figure derived from the two is an
illustration, not a prediction for a whole model.

Configurations are frozen before anything is measured - the winner of the
matching tuning workload, or the fixed default - and block measurements never
select a configuration.  ``run_block_study`` accepts an ``evaluate`` callable so
its bookkeeping can be tested without a GPU.
"""

from __future__ import annotations

import argparse
import json
import math
import platform
import random
import time
from dataclasses import asdict, replace
from datetime import datetime, timezone
from pathlib import Path

from .masks import MaskSpec
from .search import KernelConfig, default_configs
from .study import DEFAULT, is_fatal, load_winners, source_hashes, write_json

REQUIRED_VARIANTS = ("custom_interval_split", "sdpa")
SCOPE = "One bf16 inference Transformer block; same weights and operators for every variant."


def build_block_plan(winners: dict | None = None, *, seed: int = 211) -> dict:
    winners = winners or {}
    cases = []
    for length in (1024, 4096):
        for dim in (64, 128):
            for pattern in ("causal", "window"):
                family = "tune-causal" if pattern == "causal" else "tune-window128"
                winner = winners.get(family)
                config = KernelConfig(**winner["config"]) if winner else DEFAULT
                if config not in default_configs(64) + default_configs(128):
                    raise ValueError("selected config must belong to the declared tuning space")
                if dim == 128:         # one forward pipeline exists at this head dimension
                    config = replace(config, pipeline="one_stream")
                spec = MaskSpec(causal=True, window_left=127 if pattern == "window" else None)
                cases.append({
                    "case_id": f"block-n{length}-d{dim}-{pattern}-s{seed}", "length": length,
                    "dim": dim, "heads": 8, "batch": 1, "dtype": "bfloat16", "seed": seed,
                    "pattern": pattern, "mask": asdict(spec), "config": asdict(config),
                    "selection": {"policy": "training_family_transfer" if winner else "fixed_default",
                                  "source_workload": family if winner else None,
                                  "source_case_id": winner.get("case_id") if winner else None,
                                  "block_results_used_for_selection": False}})
    return {"stage": "block", "cases": cases, "scope": SCOPE,
            "selection_policy": ("Configurations are frozen from training-workload winners or the "
                                 "fixed default; block measurements never select one.")}


def training_winners(directory) -> dict:
    plan = json.loads((Path(directory) / "plan.json").read_text())
    if plan.get("stage") != "tuning":
        raise ValueError("--tuning-dir must hold a tuning-stage run, not held-out measurements")
    return load_winners(directory)


def _positive(value) -> bool:
    return (isinstance(value, (int, float)) and not isinstance(value, bool)
            and math.isfinite(value) and value > 0)


def passed_measurement(measurement: dict, required=REQUIRED_VARIANTS) -> bool:
    if (measurement.get("status") != "passed" or measurement.get("correct") is not True
            or measurement.get("reference_finite") is not True
            or measurement.get("inputs_weights_unchanged") is not True):
        return False
    for name in required:
        variant = measurement.get("variants", {}).get(name, {})
        if (variant.get("status") != "passed" or variant.get("correct") is not True
                or not _positive(variant.get("block_latency_ms"))):
            return False
    return True


def run_block_case(case: dict, *, device: str = "cuda", warmup: int = 5, repeats: int = 20,
                   inner_repeats: int = 5, include_flex: bool = False) -> dict:
    import torch
    import torch.nn.functional as F
    from torch.nn.attention import SDPBackend, sdpa_kernel

    from . import flash
    from .benchmark import dense_mask, time_cuda

    if not torch.cuda.is_available():
        raise RuntimeError("A CUDA GPU is required; no Transformer block was run")
    spec = MaskSpec(**case["mask"])
    length, dim, heads, batch = (case[k] for k in ("length", "dim", "heads", "batch"))
    width = heads * dim
    result = {"status": "running", "correct": False, "variants": {},
              "hardware": {"name": torch.cuda.get_device_name()},
              "software": {"python": platform.python_version(), "torch": torch.__version__,
                           "cuda_runtime": torch.version.cuda},
              "architecture": {"width": width, "heads": heads, "head_dim": dim,
                               "mlp_width": 4 * width, "activation": "GELU exact", "bias": False,
                               "order": ("LN -> QKV -> attention -> output projection + residual "
                                         "-> LN -> MLP + residual")},
              "timing_scope": ("CUDA-graph replay of one whole inference block, per call; Python "
                               "dispatch, mask set-up and graph capture are excluded."),
              "reference": "same bf16 block with explicit-mask math SDPA in query chunks of 256",
              "tolerances": {"atol": 0.03, "rtol": 0.03}}
    with torch.inference_mode():
        generator = torch.Generator().manual_seed(case["seed"])

        def normal(shape, scale=1.0):
            return (torch.randn(shape, generator=generator) * scale).to(device, torch.bfloat16)

        x = normal((batch, length, width))
        weights = {"qkv": normal((3 * width, width), width ** -0.5),
                   "output": normal((width, width), width ** -0.5),
                   "up": normal((4 * width, width), width ** -0.5),
                   "down": normal((width, 4 * width), (4 * width) ** -0.5),
                   "ln1": torch.ones(width, dtype=torch.bfloat16, device=device),
                   "ln2": torch.ones(width, dtype=torch.bfloat16, device=device)}
        originals = [t.clone() for t in (x, *weights.values())]
        mask = dense_mask(length, spec).to(device)
        native_causal = spec == MaskSpec(causal=True)

        def project(value):
            normed = F.layer_norm(value, (width,), weight=weights["ln1"], eps=1e-5)
            qkv = F.linear(normed, weights["qkv"]).reshape(batch, length, 3, heads, dim)
            return tuple(t.contiguous() for t in qkv.permute(2, 0, 3, 1, 4).unbind(0))

        def block(attend):
            q, k, v = project(x)
            y = attend(q, k, v).transpose(1, 2).contiguous().reshape(batch, length, width)
            residual = x + F.linear(y, weights["output"])
            normed = F.layer_norm(residual, (width,), weight=weights["ln2"], eps=1e-5)
            return residual + F.linear(F.gelu(F.linear(normed, weights["up"])), weights["down"])

        def oracle(q, k, v):
            with sdpa_kernel(SDPBackend.MATH):
                return torch.cat([F.scaled_dot_product_attention(
                    q[:, :, start:start + 256], k, v, attn_mask=mask[start:start + 256])
                    for start in range(0, length, 256)], dim=2)

        reference = block(oracle)
        result["reference_finite"] = bool(torch.isfinite(reference).all().item())
        if not result["reference_finite"]:
            raise RuntimeError("the reference block produced non-finite values")
        q0, k0, v0 = project(x)
        prepared = flash.prepare_mask(q0, None, spec, None, "interval", True)
        out_buffer = torch.empty_like(q0)
        lse = torch.empty(batch, heads, length, dtype=torch.float32, device=device)
        scale = dim ** -0.5

        def custom(q, k, v):
            flash.flash_fwd(q, k, v, out_buffer, lse, prepared, scale)
            return out_buffer

        def sdpa(q, k, v):
            return F.scaled_dot_product_attention(q, k, v, is_causal=native_causal,
                                                  attn_mask=None if native_causal else mask)

        variants = {"custom_interval_split": custom, "sdpa": sdpa}
        if include_flex:
            try:
                from torch.nn.attention.flex_attention import create_block_mask, flex_attention
                left = spec.window_left

                def predicate(b, h, qi, ki):
                    ok = ki <= qi
                    return ok if left is None else ok & (ki >= qi - left)

                block_mask = create_block_mask(predicate, None, None, length, length, device=device)
                compiled = torch.compile(flex_attention, dynamic=False)
                variants["flex"] = lambda q, k, v: compiled(q, k, v, block_mask=block_mask)
            except Exception as error:
                result["variants"]["flex"] = {"status": "failed", "correct": False,
                                              "error": str(error), "error_type": type(error).__name__}
        order = list(variants)
        random.Random(case["seed"] + length + dim).shuffle(order)
        result["measurement_order"] = order
        for name in order:
            attend = variants[name]
            measured = result["variants"][name] = {"status": "running", "correct": False}
            try:
                torch.cuda.synchronize()
                begin = time.perf_counter()
                output = block(attend)
                torch.cuda.synchronize()
                measured["first_block_call_ms"] = (time.perf_counter() - begin) * 1000
                measured["max_abs_error"] = (output.float() - reference.float()).abs().max().item()
                measured["correct"] = bool(torch.allclose(output.float(), reference.float(),
                                                          atol=0.03, rtol=0.03))
                if measured["correct"]:
                    timing = time_cuda(lambda: block(attend), warmup=warmup, repeats=repeats,
                                       inner_repeats=inner_repeats)
                    measured.update(block_timing=timing, block_latency_ms=timing["median_ms"])
                    timing = time_cuda(lambda: attend(q0, k0, v0), warmup=warmup, repeats=repeats,
                                       inner_repeats=inner_repeats)
                    measured.update(attention_timing=timing,
                                    attention_latency_ms=timing["median_ms"])
                measured["status"] = "passed" if measured["correct"] else "failed_correctness"
            except Exception as error:
                measured.update(status="failed", correct=False, error=str(error),
                                error_type=type(error).__name__)
        result["inputs_weights_unchanged"] = all(
            torch.equal(t, o) for t, o in zip((x, *weights.values()), originals))
    wanted = REQUIRED_VARIANTS + (("flex",) if include_flex else ())
    ok = result["inputs_weights_unchanged"] and all(
        result["variants"].get(name, {}).get("status") == "passed" for name in wanted)
    result.update(correct=ok, status="passed" if ok else "failed")
    add_speedups(result)
    return result


def add_speedups(result: dict) -> None:
    """Block and attention ratios against each baseline, with the Amdahl illustration."""
    candidate = result["variants"].get("custom_interval_split", {})
    if candidate.get("status") != "passed" or not result.get("inputs_weights_unchanged"):
        return
    for name, baseline in result["variants"].items():
        if name == "custom_interval_split" or baseline.get("status") != "passed":
            continue
        attention = baseline["attention_latency_ms"] / candidate["attention_latency_ms"]
        fraction = baseline["attention_latency_ms"] / baseline["block_latency_ms"]
        result[f"speedup_vs_{name}"] = baseline["block_latency_ms"] / candidate["block_latency_ms"]
        result[f"attention_speedup_vs_{name}"] = attention
        result[f"isolated_attention_fraction_{name}"] = fraction
        if 0 <= fraction <= 1:
            result[f"amdahl_estimate_vs_{name}"] = 1 / (1 - fraction + fraction / attention)
    result["amdahl_scope"] = ("Illustration from separately timed attention and block; assumes "
                              "nothing about cache behaviour and predicts no whole-model speedup.")


def run_block_study(output_dir, *, tuning_dir=None, winners=None, device="cuda", seed=211,
                    warmup=5, repeats=20, inner_repeats=5, time_budget_seconds=360,
                    include_flex=False, evaluate=None) -> dict:
    if tuning_dir is not None and winners is not None:
        raise ValueError("Supply either tuning_dir or winners, not both")
    if not math.isfinite(time_budget_seconds) or time_budget_seconds <= 0:
        raise ValueError("time budget must be finite and positive")
    if warmup < 0 or repeats < 1 or inner_repeats < 1:
        raise ValueError("warmup must be nonnegative and timing repetitions positive")
    winners = training_winners(tuning_dir) if tuning_dir is not None else winners
    plan = build_block_plan(winners, seed=seed)
    plan.update(warmup=warmup, repeats=repeats, inner_repeats=inner_repeats,
                include_flex=include_flex)
    output = Path(output_dir)
    (output / "cases").mkdir(parents=True, exist_ok=True)
    if any((output / "cases").iterdir()):
        raise FileExistsError("Block cases directory must be empty; use a new run directory")
    write_json(output / "plan.json", plan)
    planned = len(plan["cases"])
    summary = {"schema_version": 1, "stage": "block", "status": "running",
               "created_utc": datetime.now(timezone.utc).isoformat(), "planned_cases": planned,
               "completed_cases": 0, "passed_cases": 0, "failed_cases": 0,
               "not_run_cases": planned, "source_sha256": source_hashes(), "scope": SCOPE,
               "time_budget_seconds": time_budget_seconds}
    if evaluate is None:
        import torch
        if not torch.cuda.is_available():
            summary.update(status="not_run", error="A CUDA GPU is required; nothing was measured")
            write_json(output / "summary.json", summary)
            return summary
        evaluate = run_block_case
    required = REQUIRED_VARIANTS + (("flex",) if include_flex else ())
    started = time.monotonic()
    for case in plan["cases"]:
        if time.monotonic() - started >= time_budget_seconds:
            summary["status"] = "time_budget_exhausted"
            break
        begin = time.monotonic()
        try:
            measurement = evaluate(case, device=device, warmup=warmup, repeats=repeats,
                                   inner_repeats=inner_repeats, include_flex=include_flex)
        except Exception as error:
            measurement = {"status": "failed", "correct": False,
                           "error_type": type(error).__name__, "error": str(error)}
        write_json(output / "cases" / (case["case_id"] + ".json"),
                   {"case": case, "measurement": measurement,
                    "wall_seconds": time.monotonic() - begin})
        summary["completed_cases"] += 1
        key = "passed_cases" if passed_measurement(measurement, required) else "failed_cases"
        summary[key] += 1
        summary["elapsed_seconds"] = time.monotonic() - started
        summary["not_run_cases"] = planned - summary["completed_cases"]
        write_json(output / "summary.json", summary)
        print(json.dumps({"case": case["case_id"], "status": measurement.get("status"),
                          "progress": f"{summary['completed_cases']}/{planned}"}), flush=True)
        if is_fatal({"error": json.dumps(measurement)}):
            summary["status"] = "stopped_after_failure"
            break
    else:
        summary["status"] = "passed" if not summary["failed_cases"] else "completed_with_failures"
    summary["elapsed_seconds"] = time.monotonic() - started
    write_json(output / "summary.json", summary)
    return summary


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--output-dir", type=Path, required=True)
    parser.add_argument("--tuning-dir", type=Path)
    parser.add_argument("--seed", type=int, default=211)
    parser.add_argument("--warmup", type=int, default=5)
    parser.add_argument("--repeats", type=int, default=20)
    parser.add_argument("--inner-repeats", type=int, default=5)
    parser.add_argument("--time-budget-seconds", type=float, default=360)
    parser.add_argument("--include-flex", action="store_true")
    parser.add_argument("--execute", action="store_true")
    args = parser.parse_args(argv)
    if not args.execute:
        winners = training_winners(args.tuning_dir) if args.tuning_dir else None
        plan = build_block_plan(winners, seed=args.seed)
        write_json(args.output_dir / "plan.json", plan)
        print(json.dumps({"status": "dry_run", "stage": "block", "cases": len(plan["cases"])}))
        return 0
    result = run_block_study(args.output_dir, tuning_dir=args.tuning_dir, seed=args.seed,
                             warmup=args.warmup, repeats=args.repeats,
                             inner_repeats=args.inner_repeats, include_flex=args.include_flex,
                             time_budget_seconds=args.time_budget_seconds)
    print(json.dumps(result))
    return 0 if result["status"] == "passed" else 2


if __name__ == "__main__":
    raise SystemExit(main())
