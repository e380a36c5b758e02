"""Finite attention-kernel experiments: a plan of cases, one evidence file per case.

Stages and rules follow the reference's study runner (attention_lab/study.py:70-293):

* ``smoke``        small ragged shapes, both dtypes, every mask family; stops at
                   the first incorrect case.
* ``ablation``     N in {1024, 4096} x D in {64, 128} x {causal, window, document}
                   x 3 seeds over the four lowering variants (CSR or interval
                   schedule, with or without the full-tile fast path), run in a
                   seeded order so no variant always goes first.
* ``flex_hints``   the FlexAttention baseline once more, this time told that its
                   key blocks are contiguous - the fact interval lowering uses.
* ``tuning``       the whole declared configuration space on four training
                   workloads; afterwards the measured tables are replayed offline
                   through both search strategies (``replay_search``) and the
                   fastest correct configuration per workload is written out
                   (``load_winners``).
* ``confirmation`` held-out shapes measured with the default configuration and
                   with the winner transferred from the matching training
                   workload; held-out numbers never select anything.

``build_plan`` is pure (no imports of torch, no allocation).  ``run_study`` takes an
``evaluate`` callable so the orchestration is testable without a GPU; the time
budget is checked between cases, a hung call has to be bounded from outside.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import math
import platform
import random
import time
from collections import defaultdict
from dataclasses import asdict
from datetime import datetime, timezone
from pathlib import Path

from .masks import MaskSpec
from .search import CandidateResult, KernelConfig, default_configs, search

STAGES = ("smoke", "ablation", "flex_hints", "tuning", "confirmation")
DEFAULT = KernelConfig(128, 128, "interval", True)
VARIANTS = {"csr_masked": ("csr", False), "csr_full": ("csr", True),
            "interval_masked": ("interval", False), "interval_split": ("interval", True)}
_DTYPE = {"float16": "fp16", "bfloat16": "bf16"}
_FATAL = ("illegal memory access", "illegal instruction", "misaligned address",
          "device-side assert", "context is destroyed", "unspecified launch failure")


def write_json(path, value) -> None:
    path = Path(path)
    path.parent.mkdir(parents=True, exist_ok=True)
    scratch = path.with_suffix(path.suffix + ".tmp")
    scratch.write_text(json.dumps(value, indent=2, allow_nan=False) + "\n")
    scratch.replace(path)


def packed_documents(length: int) -> list[int]:
    """Document labels with irregular boundaries that never align with a tile."""
    sizes, labels, label = (97, 211, 53, 389), [], 0
    while len(labels) < length:
        labels.extend([label] * min(sizes[label % len(sizes)], length - len(labels)))
        label += 1
    return labels


def _workload(name, length, dim, pattern, *, dtype="bfloat16", heads=8, window=127) -> dict:
    spec = MaskSpec(causal=True, window_left=window if pattern == "window" else None,
                    same_document=pattern == "document")
    return {"workload_id": name, "length": length, "dim": dim, "batch": 1, "heads": heads,
            "dtype": dtype, "pattern": pattern, "spec": asdict(spec),
            "document_ids": packed_documents(length) if spec.same_document else None}


def _case(workload, seed, variant, block=(128, 128), *, flex=False, selection=None,
          pipeline=None) -> dict:
    implementation, full = VARIANTS[variant]
    pipeline = pipeline or ("two_stream" if workload["dim"] == 64 else "one_stream")
    config = asdict(KernelConfig(block[0], block[1], implementation, full, pipeline))
    tag = f"{block[0]}x{block[1]}"
    if pipeline != ("two_stream" if workload["dim"] == 64 else "one_stream"):
        tag += "-" + pipeline.replace("_", "")
    return {**workload, "case_id": f"{workload['workload_id']}-s{seed}-{variant}-{tag}",
            "seed": seed, "variant": variant, "config": config, "include_flex": flex,
            "selection": selection}


def _config_case(workload, seed, config: KernelConfig, *, flex=False, selection=None) -> dict:
    variant = next(name for name, pair in VARIANTS.items()
                   if pair == (config.implementation, config.use_full_blocks))
    # head dimension 128 has one forward pipeline whatever a transferred configuration says
    pipeline = "one_stream" if workload["dim"] == 128 else config.pipeline
    return _case(workload, seed, variant, (config.block_q, config.block_k), flex=flex,
                 selection=selection, pipeline=pipeline)


def _family_configs(pattern: str, dim: int = 64) -> list[KernelConfig]:
    """The space of one workload: the forward pipelines its head dimension has, and for
    document masks (which have no interval form) only the CSR configurations."""
    return [c for c in default_configs(dim) if pattern != "document" or c.implementation == "csr"]


def build_plan(stage: str, *, winners: dict | None = None) -> dict:
    cases = []
    if stage == "smoke":
        shapes = [(128, 64, "float16"), (257, 128, "float16"), (128, 128, "bfloat16"),
                  (257, 64, "bfloat16")]
        for index, (length, dim, dtype) in enumerate(shapes):
            for pattern in ("causal", "window", "document"):
                workload = _workload(f"smoke-{index}-{pattern}", length, dim, pattern, dtype=dtype,
                                     heads=2)
                names = ("csr_full",) if pattern == "document" else ("csr_full", "interval_split")
                for variant in names:
                    cases.append(_case(workload, 0, variant, (64, 64)))
    elif stage == "ablation":
        for length in (1024, 4096):
            for dim in (64, 128):
                for pattern in ("causal", "window", "document"):
                    workload = _workload(f"n{length}-d{dim}-{pattern}", length, dim, pattern)
                    names = list(VARIANTS)[:2] if pattern == "document" else list(VARIANTS)
                    for seed in (11, 12, 13):
                        order = list(names)
                        random.Random(seed).shuffle(order)
                        for variant in order:
                            cases.append(_case(workload, seed, variant, flex=variant == "csr_full"))
    elif stage == "flex_hints":
        for length in (1024, 4096):
            for dim in (64, 128):
                for pattern in ("causal", "window"):
                    workload = _workload(f"n{length}-d{dim}-{pattern}", length, dim, pattern)
                    for seed in (11, 12, 13):
                        case = _case(workload, seed, "interval_split", flex=True)
                        case["flex_contiguous"] = True
                        cases.append(case)
    elif stage == "tuning":
        for workload in (_workload("tune-causal", 4096, 64, "causal"),
                         _workload("tune-window128", 4096, 64, "window"),
                         _workload("tune-window512", 4096, 128, "window", window=511),
                         _workload("tune-document", 4096, 64, "document")):
            configs = _family_configs(workload["pattern"], workload["dim"])
            random.Random(2026).shuffle(configs)
            for index, config in enumerate(configs):
                cases.append(_config_case(workload, 23, config, flex=index == 0))
    elif stage == "confirmation":
        held_out = ((_workload("holdout-tail257", 257, 64, "window"), "tune-window128"),
                    (_workload("holdout-tail4097", 4097, 128, "window", window=511),
                     "tune-window512"),
                    (_workload("holdout-causal8192", 8192, 64, "causal"), "tune-causal"),
                    (_workload("holdout-document8192", 8192, 64, "document"), "tune-document"))
        for workload, source in held_out:
            default = (KernelConfig(128, 128, "csr", True) if workload["pattern"] == "document"
                       else DEFAULT)
            for seed in (101, 102, 103):
                base = _config_case(workload, seed, default, flex=True, selection="fixed_default")
                base["case_id"] += "-default"
                cases.append(base)
                if winners and source in winners:
                    tuned = _config_case(
                        workload, seed, KernelConfig(**winners[source]["config"]),
                        selection={"policy": "fastest_correct_training_configuration",
                                   "source_workload": source,
                                   "source_case_id": winners[source]["case_id"]})
                    tuned["case_id"] += "-transferred"
                    cases.append(tuned)
    else:
        raise ValueError("unknown study stage")
    identifiers = [case["case_id"] for case in cases]
    if len(set(identifiers)) != len(identifiers):
        raise ValueError("duplicate case identifiers")
    return {"schema_version": 1, "stage": stage, "cases": cases, "warmup": 5, "repeats": 20,
            "inner_repeats": 20, "timing_mode": "cuda_graph",
            "selection_policy": ("Confirmation transfers winners from the matching training "
                                 "workload; held-out measurements never select a configuration."),
            "baseline_reuse": ("A Flex result is paired only with cases of the identical workload "
                               "and input seed; SDPA is measured again in every case.")}


def eligible(measurement: dict) -> bool:
    return CandidateResult(measurement.get("status") == "passed"
                           and measurement.get("correct") is True,
                           measurement.get("latency_ms"),
                           error=measurement.get("error")).eligible


def load_winners(directory) -> dict:
    """Fastest correct case per workload among the evidence files of a run."""
    winners: dict = {}
    for path in sorted((Path(directory) / "cases").glob("*.json")):
        record = json.loads(path.read_text())
        case, measured = record["case"], record["measurement"]
        if not eligible(measured):
            continue
        held = winners.get(case["workload_id"])
        if held is None or measured["latency_ms"] < held["latency_ms"]:
            winners[case["workload_id"]] = {"case_id": case["case_id"], "config": case["config"],
                                            "latency_ms": measured["latency_ms"]}
    return winners


def replay_search(records, *, budgets=(4, 8, 12), seeds=20) -> dict:
    """Both strategies against the measured tables - no new GPU work, no timing noise."""
    groups = defaultdict(list)
    for record in records:
        groups[record["case"]["workload_id"]].append(record)
    reports = []
    for workload, group in sorted(groups.items()):
        table = {KernelConfig(**r["case"]["config"]): r["measurement"] for r in group}
        space = set(_family_configs(group[0]["case"]["pattern"], group[0]["case"]["dim"]))
        if set(table) != space:
            reports.append({"workload_id": workload, "status": "incomplete_table",
                            "measured_configs": len(table)})
            continue
        valid = [m["latency_ms"] for m in table.values() if eligible(m)]
        if not valid:
            reports.append({"workload_id": workload, "status": "no_correct_configuration"})
            continue
        oracle, trials = min(valid), []

        def lookup(config):
            measured = table[config]
            return CandidateResult(eligible(measured), measured.get("latency_ms"),
                                   error=measured.get("error"))

        for method in ("random", "descent"):
            for budget in budgets:
                for seed in range(seeds):
                    best = search(lookup, sorted(space, key=lambda c: astuple_key(c)),
                                  budget=min(budget, len(space)), method=method, seed=seed).best
                    latency = best.result.latency_ms if best else None
                    trials.append({"method": method, "budget": budget, "search_seed": seed,
                                   "best_latency_ms": latency,
                                   "relative_regret": latency / oracle - 1 if best else None,
                                   "best_config": asdict(best.config) if best else None})
        reports.append({"workload_id": workload, "status": "completed",
                        "oracle_latency_ms": oracle, "eligible_configurations": len(valid),
                        "trials": trials})
    return {"methodology": ("Offline replay of fixed measured latency tables: no new GPU calls; "
                            "timing noise, first-call cost, thermal and order effects and the "
                            "search's own overhead are all excluded."),
            "workloads": reports}


def astuple_key(config: KernelConfig) -> tuple:
    return (config.block_q, config.block_k, config.implementation, config.use_full_blocks,
            config.pipeline)


def is_fatal(measurement: dict) -> bool:
    text = (str(measurement.get("error", "")) + " "
            + str(measurement.get("flex", {}).get("error", ""))).lower()
    return any(marker in text for marker in _FATAL)


def case_arguments(case: dict, plan: dict) -> dict:
    arguments = {key: case[key] for key in ("length", "dim", "batch", "heads", "document_ids",
                                            "seed", "include_flex")}
    arguments["dtype"] = _DTYPE[case["dtype"]]
    arguments["flex_contiguous"] = case.get("flex_contiguous", False)
    arguments["spec"] = MaskSpec(**case["spec"])
    arguments.update(case["config"])
    arguments.update({key: plan[key] for key in ("warmup", "repeats", "inner_repeats")})
    return arguments


def source_hashes() -> dict:
    return {path.name: hashlib.sha256(path.read_bytes()).hexdigest()
            for path in sorted(Path(__file__).parent.glob("*.py"))}


def run_study(plan: dict, output_dir, *, time_budget_seconds: float = 900, evaluate=None) -> dict:
    if evaluate is None:
        from .benchmark import run_case as evaluate
    output = Path(output_dir)
    (output / "cases").mkdir(parents=True, exist_ok=True)
    if any((output / "cases").iterdir()):
        raise FileExistsError("Case output directory must be empty; use a new run directory")
    if not math.isfinite(time_budget_seconds) or time_budget_seconds <= 0:
        raise ValueError("time budget must be finite and positive")
    write_json(output / "plan.json", plan)
    started, records = time.monotonic(), []
    summary = {"schema_version": 1, "stage": plan["stage"], "status": "running",
               "created_utc": datetime.now(timezone.utc).isoformat(),
               "planned_cases": len(plan["cases"]), "completed_cases": 0, "passed_cases": 0,
               "failed_cases": 0, "flex_requested_cases": 0, "flex_passed_cases": 0,
               "flex_failed_cases": 0, "time_budget_seconds": time_budget_seconds,
               "python": platform.python_version(), "source_sha256": source_hashes()}
    smoke = plan["stage"] == "smoke"
    for case in plan["cases"]:
        if time.monotonic() - started >= time_budget_seconds:
            summary["status"] = "time_budget_exhausted"
            break
        begin = time.monotonic()
        try:
            measured = evaluate(**case_arguments(case, plan))
        except Exception as error:
            measured = {"status": "failed", "correct": False, "latency_ms": None,
                        "error_type": type(error).__name__, "error": str(error)}
        record = {"case": case, "measurement": measured, "wall_seconds": time.monotonic() - begin}
        write_json(output / "cases" / (case["case_id"] + ".json"), record)
        records.append(record)
        passed = eligible(measured)
        summary["completed_cases"] += 1
        summary["passed_cases" if passed else "failed_cases"] += 1
        flex_failed = case["include_flex"] and measured.get("flex", {}).get("status") != "passed"
        if case["include_flex"]:
            summary["flex_requested_cases"] += 1
            summary["flex_failed_cases" if flex_failed else "flex_passed_cases"] += 1
        summary["elapsed_seconds"] = time.monotonic() - started
        write_json(output / "summary.json", summary)
        print(json.dumps({"case": case["case_id"], "status": measured.get("status"),
                          "latency_ms": measured.get("latency_ms"),
                          "progress": f"{len(records)}/{len(plan['cases'])}"}), flush=True)
        if is_fatal(measured) or (smoke and not passed):
            summary["status"] = "stopped_after_failure"
            break
    else:
        summary["status"] = ("completed_with_failures" if summary["failed_cases"] else
                             "completed_with_baseline_failures" if summary["flex_failed_cases"]
                             else "passed")
    write_json(output / "baseline_pairs.json", pair_baselines(records))
    if plan["stage"] == "tuning":
        write_json(output / "search_replay.json", replay_search(records))
        write_json(output / "winners.json", load_winners(output))
    summary["elapsed_seconds"] = time.monotonic() - started
    summary["not_run_cases"] = summary["planned_cases"] - summary["completed_cases"]
    write_json(output / "summary.json", summary)
    return summary


def pair_baselines(records) -> list[dict]:
    """Attach the Flex timing measured on the same workload and input seed."""
    sources = {(r["case"]["workload_id"], r["case"]["seed"]): r for r in records
               if r["measurement"].get("flex", {}).get("status") == "passed"}
    pairs = []
    for record in records:
        case, measured = record["case"], record["measurement"]
        source = sources.get((case["workload_id"], case["seed"]))
        latency = source["measurement"]["flex"].get("latency_ms") if source else None
        usable = (eligible(measured) and isinstance(latency, (int, float)) and latency > 0)
        pairs.append({"case_id": case["case_id"],
                      "baseline_source_case_id": source["case"]["case_id"] if source else None,
                      "flex_latency_ms": latency,
                      "flex_speedup": latency / measured["latency_ms"] if usable else None,
                      "sdpa_speedup": measured.get("baseline_over_custom")})
    return pairs


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--stage", choices=STAGES, default="smoke")
    parser.add_argument("--output-dir", type=Path, required=True)
    parser.add_argument("--time-budget-seconds", type=float, default=900)
    parser.add_argument("--tuning-dir", type=Path)
    parser.add_argument("--execute", action="store_true")
    args = parser.parse_args(argv)
    winners = load_winners(args.tuning_dir) if args.tuning_dir else None
    plan = build_plan(args.stage, winners=winners)
    if not args.execute:
        write_json(args.output_dir / "plan.json", plan)
        print(json.dumps({"status": "dry_run", "stage": args.stage, "cases": len(plan["cases"]),
                          "plan": str(args.output_dir / "plan.json")}))
        return 0
    import torch
    if not torch.cuda.is_available():
        report = {"status": "not_run", "error": "A CUDA GPU is required; nothing was measured"}
        write_json(args.output_dir / "summary.json", report)
        print(json.dumps(report))
        return 2
    summary = run_study(plan, args.output_dir, time_budget_seconds=args.time_budget_seconds)
    print(json.dumps(summary, sort_keys=True))
    return 0 if summary["status"] == "passed" else 2


if __name__ == "__main__":
    raise SystemExit(main())
