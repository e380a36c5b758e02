"""Correctness-gated configuration search for one shape and mask on a local GPU.

Counterpart of the reference's single-workload search driver
(attention_lab/gpu_search.py:20-135).  Every candidate is measured by
``benchmark.run_case`` on the same seeded inputs and is eligible only if its
output matched the fp32 reference; the chosen configuration is then measured
once more on inputs from a fresh seed, outside the search budget, and the run
passes only if that confirmation is correct too.  Nothing here assumes a timing:
every number in the report comes from a call that ran.
"""

from __future__ import annotations

import argparse
import json
import time
from dataclasses import asdict
from datetime import datetime, timezone
from pathlib import Path

from . import benchmark
from .masks import MaskSpec
from .search import CandidateResult, default_configs, search

_CONFIG_FIELDS = ("block_q", "block_k", "implementation", "use_full_blocks", "pipeline")


def _as_result(measurement: dict) -> CandidateResult:
    return CandidateResult(correct=measurement.get("correct") is True,
                           latency_ms=measurement.get("latency_ms"),
                           compile_ms=measurement.get("first_call_ms"),
                           error=measurement.get("error"))


def _measure(case: dict, config) -> tuple[dict, float]:
    begin = time.perf_counter()
    try:
        measurement = benchmark.run_case(**case, **asdict(config))
    except Exception as error:
        measurement = {"correct": False, "latency_ms": None, "error_type": type(error).__name__,
                       "error": str(error)}
    return measurement, (time.perf_counter() - begin) * 1000


def run_experiment(*, budget: int = 12, method: str = "descent", search_seed: int = 0,
                   **case) -> dict:
    """``case`` holds the arguments of ``benchmark.run_case`` that are not searched."""
    candidates = default_configs(case.get("dim", 64))
    if type(budget) is not int or not 1 <= budget <= len(candidates):
        raise ValueError(f"budget must be between 1 and {len(candidates)}")
    if set(_CONFIG_FIELDS) & case.keys():
        raise ValueError("kernel configurations are selected by search")
    case.setdefault("time_baselines", False)
    measurements = []

    def evaluate(config):
        measurement, wall = _measure(case, config)
        measurements.append({"config": asdict(config), "measurement": measurement,
                             "wall_time_ms": wall})
        return _as_result(measurement)

    started = time.perf_counter()
    result = search(evaluate, candidates, budget=budget, method=method, seed=search_seed)
    search_wall = (time.perf_counter() - started) * 1000
    confirmation, confirmed = None, False
    if result.best is not None:
        fresh = {**case, "seed": case.get("seed", 0) + 1}
        measurement, wall = _measure(fresh, result.best.config)
        confirmation = {"config": asdict(result.best.config), "measurement": measurement,
                        "wall_time_ms": wall, "counts_toward_search_budget": False}
        confirmed = _as_result(measurement).eligible
    return {"schema_version": 1, "created_utc": datetime.now(timezone.utc).isoformat(),
            "status": "passed" if confirmed else "failed", "search": result.to_dict(),
            "measurements": measurements, "confirmation": confirmation,
            "search_wall_time_ms": search_wall,
            "total_wall_time_ms": (time.perf_counter() - started) * 1000,
            "scope": ("One shape and mask, forward only; the winner is confirmed on a fresh input "
                      "seed. Says nothing about other shapes or about which search method is "
                      "better.")}


def spec_for(mask: str, window_left: int, window_right: int) -> MaskSpec:
    windowed = mask in ("sliding", "combined")
    return MaskSpec(causal=mask in ("causal", "combined"),
                    window_left=window_left if windowed else None,
                    window_right=window_right if windowed else None,
                    same_document=mask in ("document", "combined"))


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--method", choices=["descent", "random"], default="descent")
    parser.add_argument("--budget", type=int, default=12)
    parser.add_argument("--search-seed", type=int, default=0)
    parser.add_argument("--input-seed", type=int, default=0)
    parser.add_argument("--length", type=int, default=4096)
    parser.add_argument("--dim", type=int, choices=[64, 128], default=64)
    parser.add_argument("--batch", type=int, default=1)
    parser.add_argument("--heads", type=int, default=4)
    parser.add_argument("--mask", default="sliding",
                        choices=["dense", "causal", "sliding", "document", "combined"])
    parser.add_argument("--window-left", type=int, default=127)
    parser.add_argument("--window-right", type=int, default=0)
    parser.add_argument("--document-length", type=int, default=97)
    parser.add_argument("--dtype", choices=list(benchmark.DTYPES), default="fp16")
    parser.add_argument("--repeats", type=int, default=30)
    parser.add_argument("--output", type=Path, required=True)
    args = parser.parse_args(argv)
    if min(args.length, args.batch, args.heads, args.document_length, args.repeats) < 1:
        parser.error("shape, document length and repeats must be positive")
    if min(args.window_left, args.window_right) < 0:
        parser.error("windows must be nonnegative")
    spec = spec_for(args.mask, args.window_left, args.window_right)
    documents = ([i // args.document_length for i in range(args.length)]
                 if spec.same_document else None)
    report = {"schema_version": 1, "status": "not_run"}
    try:
        import torch
        if not torch.cuda.is_available():
            raise RuntimeError("A CUDA GPU is required; no search was run")
        report = run_experiment(method=args.method, budget=args.budget,
                                search_seed=args.search_seed, length=args.length, dim=args.dim,
                                batch=args.batch, heads=args.heads, spec=spec,
                                document_ids=documents, dtype=args.dtype, seed=args.input_seed,
                                repeats=args.repeats)
    except Exception as error:
        report.update(error_type=type(error).__name__, error=str(error))
    args.output.parent.mkdir(parents=True, exist_ok=True)
    args.output.write_text(json.dumps(report, indent=2, allow_nan=False) + "\n")
    print(json.dumps({"status": report["status"], "output": str(args.output)}))
    return 0 if report["status"] == "passed" else 2


if __name__ == "__main__":
    raise SystemExit(main())
