"""Fixed-batch attention / memory pilot: plan first, execute only on request.

Same workflow and artefacts as the reference pilot (src/llmlab/pilot.py:39-433):
``make_plan`` resolves the factorial {eager, sdpa} x {none, block} x microbatches
x seeds (or an explicit ``backend:checkpoint:microbatch`` policy list) at a
constant effective batch into fully validated per-case configs, shuffles the
order with a seed and seals the plan with a hash; ``write_plan`` lays it out on
disk; ``execute_plan`` re-verifies plan and source identity, then runs each
untouched case as ``python -m llmlab.train`` with a timeout, never overwriting
evidence; ``summarize_case`` / ``aggregate_results`` turn run directories into
rows with strict evidence validation (warm-up exclusion, p90 by linear
interpolation, OOM / timeout classification) and a comparability verdict per
seed (same data identity and batch stream).
"""

from __future__ import annotations

import argparse
import hashlib
import json
import random
import re
import statistics
import sys
from collections import Counter
from dataclasses import replace
from pathlib import Path

import torch

from .config import TrainConfig, load_config
from .experiments import common
from .train import source_identity

POLICY = re.compile(r"(eager|sdpa):(none|block):([1-9][0-9]*)")
STATUS_RANK = {"completed": 0, "insufficient_samples": 1, "missing_output": 2, "invalid_output": 3}


def _require_positive_int(value, name: str) -> None:
    if type(value) is not int or value <= 0:
        raise ValueError(f"{name} must be a positive integer")


def _parse_policies(policies, microbatches) -> set | None:
    if policies is None:
        return None
    if not policies:
        raise ValueError("policies must not be empty")
    chosen = set()
    for policy in policies:
        match = POLICY.fullmatch(policy) if isinstance(policy, str) else None
        if match is None:
            raise ValueError("policies must use backend:checkpoint:microbatch, "
                             "for example sdpa:block:8")
        treatment = (match.group(1), match.group(2), int(match.group(3)))
        if treatment[2] not in microbatches:
            raise ValueError("every policy microbatch must belong to microbatches")
        if treatment in chosen:
            raise ValueError("duplicate policies would repeat the same case")
        chosen.add(treatment)
    return chosen


def make_plan(config: TrainConfig, *, microbatches: list[int], effective_batch_size: int,
              seeds: list[int], warmup_steps: int, device: str = "cuda",
              precision: str | None = None, order_seed: int = 0, timeout_seconds: float = 600,
              policies: list[str] | None = None) -> dict:
    """Resolve every case without loading data or starting training."""
    config.validate()
    _require_positive_int(effective_batch_size, "effective_batch_size")
    _require_positive_int(warmup_steps, "warmup_steps")
    if warmup_steps >= config.max_steps:
        raise ValueError("profiling warmup_steps must be less than max_steps")
    if not microbatches or not seeds:
        raise ValueError("microbatches and seeds must not be empty")
    if len(set(microbatches)) != len(microbatches) or len(set(seeds)) != len(seeds):
        raise ValueError("duplicate microbatches or seeds would repeat the same case")
    for microbatch in microbatches:
        _require_positive_int(microbatch, "microbatch")
        if effective_batch_size % microbatch:
            raise ValueError("every microbatch must divide effective_batch_size")
    chosen = _parse_policies(policies, microbatches)
    for seed in seeds:
        if type(seed) is not int or not 0 <= seed < 2 ** 63 - 1:
            raise ValueError("seeds must be integers in [0, 2**63 - 1)")
    if type(order_seed) is not int:
        raise ValueError("order_seed must be an integer")
    if device not in ("cuda", "cpu"):
        raise ValueError("pilot device must be cuda, or cpu for an explicit harness check")
    if not common.is_finite(timeout_seconds, positive=True):
        raise ValueError("timeout_seconds must be finite and positive")
    data = config.data
    absolute = replace(
        data,
        train_path=str(Path(data.train_path).resolve()) if data.train_path else None,
        valid_path=str(Path(data.valid_path).resolve()) if data.valid_path else None,
        tokenizer_files=tuple(str(Path(p).resolve()) for p in data.tokenizer_files))
    config = replace(config, data=absolute)
    source = source_identity()
    cases = []
    grid = [(seed, backend, ckpt, mb) for seed in sorted(seeds) for backend in ("eager", "sdpa")
            for ckpt in ("none", "block") for mb in sorted(microbatches)]
    for seed, backend, ckpt, microbatch in grid:
        if chosen is not None and (backend, ckpt, microbatch) not in chosen:
            continue
        accumulation = effective_batch_size // microbatch
        resolved = replace(config, seed=seed, device=device, batch_size=microbatch,
                           grad_accum_steps=accumulation,
                           precision=config.precision if precision is None else precision,
                           model=replace(config.model, attention_backend=backend,
                                         activation_checkpointing=ckpt))
        resolved.validate()
        case_id = f"{backend}-{ckpt}-mb{microbatch}-acc{accumulation}-seed{seed}"
        as_dict = resolved.to_dict()
        cases.append({
            "case_id": case_id,
            "labels": {"attention_backend": backend, "activation_checkpointing": ckpt,
                       "batch_size": microbatch, "grad_accum_steps": accumulation, "seed": seed,
                       "device": device, "precision": resolved.precision},
            "config": as_dict, "config_sha256": common.json_sha256(as_dict),
            "source_sha256": source["python_source_sha256"], "max_steps": resolved.max_steps,
            "tokens_per_step": effective_batch_size * resolved.model.context_length,
            "config_path": f"configs/{case_id}.json", "run_path": f"runs/{case_id}"})
    random.Random(order_seed).shuffle(cases)
    plan = {"format_version": 1, "source": source, "effective_batch_size": effective_batch_size,
            "warmup_steps": warmup_steps, "order_seed": order_seed,
            "timeout_seconds": timeout_seconds,
            "attention_dispatch": ("sdpa selects the sm_100a flash kernel on the fused path and "
                                   "PyTorch SDPA elsewhere"),
            "warmup_scope": ("exclude optimizer steps <= warmup_steps from timing statistics; "
                             "keep the training schedule unchanged"),
            "cases": cases}
    return common.seal(plan)


def write_plan(plan: dict, output_dir: str | Path) -> Path:
    root = Path(output_dir).resolve()
    root.mkdir(parents=True, exist_ok=False)
    (root / "configs").mkdir()
    for case in plan["cases"]:
        common.write_json(root / case["config_path"], case["config"])
    common.write_json(root / "manifest.json", plan)
    return root


class _CaseReport:
    """Accumulates the row of one case and the worst problem seen so far."""

    def __init__(self, case: dict, warmup_steps: int):
        labels = case["labels"]
        self.failed = False
        self.errors: list[str] = []
        self.row = {
            "case_id": case["case_id"], **labels, "config_sha256": case["config_sha256"],
            "status": "completed",
            "effective_batch_size": labels["batch_size"] * labels["grad_accum_steps"],
            "tokens_per_step": case["tokens_per_step"], "tokens_seen": None,
            "data_identity": None, "data_identity_sha256": None, "batch_stream_sha256": None,
            "measured_steps": 0, "expected_measured_steps": case["max_steps"] - warmup_steps,
            "step_seconds_median": None, "step_seconds_p90": None, "tokens_per_second": None,
            "last_train_loss": None, "valid_loss": None, "runner_times": {},
            "subprocess_wall_seconds": None, "peak_cuda_allocated_bytes": None,
            "peak_cuda_reserved_bytes": None}

    def problem(self, status: str, message: str) -> None:
        if not self.failed and STATUS_RANK[status] > STATUS_RANK.get(self.row["status"], 0):
            self.row["status"] = status
        self.errors.append(message)

    def fail(self, status: str, message: str) -> None:
        if not self.failed:
            self.row["status"] = status
        self.failed = True
        self.errors.append(message)

    def number(self, value, name: str, *, required=False, nonnegative=False):
        if value is None and not required:
            return None
        if not common.is_finite(value, nonnegative=nonnegative):
            self.problem("invalid_output", f"{name} must be finite"
                         + (" and nonnegative" if nonnegative else ""))
            return None
        return value


def _read_execution(report: _CaseReport, root: Path, case: dict) -> None:
    path = root / "execution" / f"{case['case_id']}.json"
    if not path.exists():
        return
    execution = common.read_json(path)
    report.row["returncode"] = execution.get("returncode")
    if execution.get("status") in ("failed", "timeout") or execution.get("returncode") not in (None, 0):
        report.fail("timeout" if execution.get("status") == "timeout" else "failed",
                    execution.get("error")
                    or f"process exited with code {execution.get('returncode')}")
    elif execution.get("status") != "completed":
        report.problem("insufficient_samples", "subprocess completion was not recorded")
    report.row["subprocess_wall_seconds"] = report.number(
        execution.get("wall_seconds"), "subprocess wall time", nonnegative=True)


def _read_summary(report: _CaseReport, run_dir: Path, case: dict) -> None:
    path = run_dir / "summary.json"
    if not path.exists():
        report.problem("missing_output", "summary.json is missing")
        return
    summary = common.read_json(path)
    status = summary.get("status")
    if status == "failed":
        report.fail("failed", summary.get("error", "runner failed"))
    elif status != "completed":
        report.problem("insufficient_samples", "runner did not complete its planned updates")
    else:
        if type(summary.get("step")) is not int or summary["step"] != case["max_steps"]:
            report.problem("invalid_output", "completed summary step does not match the plan")
        expected = case["max_steps"] * case["tokens_per_step"]
        if type(summary.get("tokens_seen")) is not int or summary["tokens_seen"] != expected:
            report.problem("invalid_output", "completed summary tokens_seen does not match the plan")
    row = report.row
    row["tokens_seen"] = report.number(summary.get("tokens_seen"), "summary tokens_seen",
                                       nonnegative=True)
    row["valid_loss"] = report.number(summary.get("valid_loss"), "validation loss",
                                      required=status == "completed")
    row["runner_times"] = {key: report.number(summary.get(key), key, nonnegative=True)
                           for key in ("setup_seconds", "train_seconds", "eval_seconds",
                                       "checkpoint_seconds", "wall_seconds")}
    for key in ("peak_cuda_allocated_bytes", "peak_cuda_reserved_bytes"):
        row[key] = report.number(summary.get(key), key, nonnegative=True)


def _read_metadata(report: _CaseReport, run_dir: Path, case: dict) -> None:
    path = run_dir / "metadata.json"
    if not path.exists():
        report.problem("missing_output", "metadata.json is missing")
        return
    metadata = common.read_json(path)
    if metadata.get("config_sha256") != case["config_sha256"]:
        report.problem("invalid_output", "metadata config identity does not match the plan")
    if metadata.get("source", {}).get("python_source_sha256") != case["source_sha256"]:
        report.problem("invalid_output", "metadata source identity does not match the plan")
    identity = metadata.get("data_identity")
    if isinstance(identity, dict) and identity:
        report.row["data_identity"] = identity
        report.row["data_identity_sha256"] = common.json_sha256(identity)
    report.row["gpu_name"] = metadata.get("gpu_name")
    report.row["gpu_count"] = report.number(metadata.get("gpu_count"), "gpu_count",
                                            nonnegative=True)
    report.row["workload"] = metadata.get("workload")


def _read_metrics(report: _CaseReport, run_dir: Path, case: dict, warmup_steps: int) -> None:
    path = run_dir / "metrics.jsonl"
    if not path.exists():
        report.problem("missing_output", "metrics.jsonl is missing")
        records = []
    else:
        records = common.read_jsonl(path)
    train = [r for r in records if r.get("event") == "train"]
    for index, record in enumerate(train, 1):
        if type(record.get("step")) is not int or record["step"] != index or index > case["max_steps"]:
            raise ValueError("training steps must be a unique consecutive sequence starting at 1")
        if not common.is_finite(record.get("step_seconds"), positive=True) \
                or not common.is_finite(record.get("loss")):
            raise ValueError("training duration must be positive and finite; loss must be finite")
        if type(record.get("tokens_seen")) is not int \
                or record["tokens_seen"] != index * case["tokens_per_step"]:
            raise ValueError("tokens_seen does not match the planned effective batch")
    measured = [r["step_seconds"] for r in train if r["step"] > warmup_steps]
    row = report.row
    row["measured_steps"] = len(measured)
    if measured:
        row["step_seconds_median"] = statistics.median(measured)
        row["step_seconds_p90"] = common.percentile_linear(measured, 0.9)
        row["tokens_per_second"] = case["tokens_per_step"] * len(measured) / sum(measured)
    if train:
        row["last_train_loss"] = train[-1]["loss"]
    hashes = [r.get("batch_start_sha256") for r in train]
    valid = len(hashes) == case["max_steps"] and all(
        isinstance(h, str) and re.fullmatch(r"[0-9a-f]{64}", h) for h in hashes)
    row["batch_stream_sha256"] = (hashlib.sha256("".join(hashes).encode()).hexdigest()
                                  if valid else None)
    if len(measured) < row["expected_measured_steps"] and row["status"] == "completed":
        report.problem("insufficient_samples", "fewer post-warmup training rows than planned")


def summarize_case(root: str | Path, case: dict, warmup_steps: int) -> dict:
    """One row per case; failures, partial and missing output stay visible."""
    root = Path(root)
    run_dir = root / "runs" / case["case_id"]
    report = _CaseReport(case, warmup_steps)
    try:
        _read_execution(report, root, case)
        _read_summary(report, run_dir, case)
        _read_metadata(report, run_dir, case)
        _read_metrics(report, run_dir, case, warmup_steps)
    except (OSError, ValueError, TypeError, AttributeError) as error:
        report.problem("invalid_output", str(error))
    row = report.row
    if report.errors:
        row["error"] = "; ".join(str(e) for e in report.errors)
    if row["status"] == "timeout":
        row["failure_kind"] = "timeout"
    elif row["status"] == "failed":
        log = root / "logs" / f"{case['case_id']}.log"
        try:
            tail = log.read_text(errors="replace")[-4000:] if log.exists() else ""
        except OSError:
            tail = ""
        row["failure_kind"] = common.classify_failure(row.get("error", "") + tail)
    return row


def aggregate_results(root: str | Path, plan: dict) -> dict:
    rows = [summarize_case(root, case, plan["warmup_steps"]) for case in plan["cases"]]
    groups = []
    for seed in sorted({row["seed"] for row in rows}):
        members = [row for row in rows if row["seed"] == seed]
        complete = [row for row in members if row["status"] == "completed"]
        reasons = []
        for key in ("data_identity_sha256", "batch_stream_sha256"):
            if any(row[key] is None for row in complete):
                reasons.append(f"completed cases lack valid {key} evidence")
            if len({row[key] for row in complete if row[key] is not None}) > 1:
                reasons.append(f"completed cases disagree on {key}")
        status = "failed" if reasons else "passed"
        if len(complete) != len(members):
            reasons.append("not all planned cases completed with valid output")
            if status != "failed":
                status = "insufficient"
        groups.append({"seed": seed, "status": status, "reasons": reasons,
                       "case_ids": [row["case_id"] for row in members]})
    if any(g["status"] == "failed" for g in groups):
        overall = "failed"
    elif any(g["status"] != "passed" for g in groups):
        overall = "insufficient"
    else:
        overall = "passed"
    return {
        "format_version": 1, "plan_sha256": plan["plan_sha256"],
        "status_counts": dict(Counter(row["status"] for row in rows)),
        "comparability": {"status": overall, "seed_groups": groups,
                          "reasons": [f"seed {g['seed']}: {r}" for g in groups for r in g["reasons"]]},
        "timing_scope": ("per-case complete optimizer-step durations after profiling warmup; "
                         "includes batch preparation and transfer, excludes evaluation/checkpoint time"),
        "throughput_scope": "measured valid tokens divided by summed measured step durations",
        "percentile_method": "linear interpolation at 0.9 * (sample_count - 1)",
        "interpretation": ("descriptive pilot measurements; CPU/synthetic cases are harness checks; "
                           "no speedup or quality-equivalence claim"),
        "cases": rows}


def execute_plan(output_dir: str | Path, *, allow_cpu: bool = False) -> dict:
    root = Path(output_dir).resolve()
    plan = common.read_json(root / "manifest.json")
    if plan.get("format_version") != 1 or not common.verify_seal(plan):
        raise ValueError("manifest version or identity is invalid")
    if source_identity()["python_source_sha256"] != plan["source"]["python_source_sha256"]:
        raise ValueError("source changed after planning; inspect and create a new plan")
    for case in plan["cases"]:
        if not re.fullmatch(r"[a-z0-9_-]+", case["case_id"]):
            raise ValueError("invalid case identifier")
        resolved = load_config(root / "configs" / f"{case['case_id']}.json")
        if common.json_sha256(resolved.to_dict()) != case["config_sha256"]:
            raise ValueError(f"resolved config changed for {case['case_id']}")
        if resolved.device == "cpu":
            if not allow_cpu:
                raise ValueError("CPU execution requires --allow-cpu and is a harness check only")
        elif resolved.device != "cuda":
            raise ValueError("pilot execution supports CUDA or explicitly allowed CPU only")
        elif not torch.cuda.is_available():
            raise RuntimeError("CUDA requested but unavailable; no pilot cases were started")
    for directory in ("runs", "logs", "execution"):
        (root / directory).mkdir(exist_ok=True)
    environment = common.child_environment()
    for case in plan["cases"]:
        case_id = case["case_id"]
        record_path = root / "execution" / f"{case_id}.json"
        # Re-entering an interrupted plan only runs untouched cases; evidence is never replaced.
        if record_path.exists() or (root / "runs" / case_id).exists():
            continue
        command = [sys.executable, "-m", "llmlab.train", "--config",
                   str(root / "configs" / f"{case_id}.json"), "--output-dir",
                   str(root / "runs" / case_id)]
        common.write_json(record_path, {"status": "running", "command": command,
                                        "returncode": None})
        result = run_training_case(command, root / "logs" / f"{case_id}.log",
                                   plan["timeout_seconds"], environment)
        common.write_json(record_path, result)
        common.write_json(root / "aggregate.json", aggregate_results(root, plan))
    aggregate = aggregate_results(root, plan)
    common.write_json(root / "aggregate.json", aggregate)
    return aggregate


def run_training_case(command, log_path, timeout, environment) -> dict:
    """Indirection point so tests can replace the subprocess."""
    return common.run_case(command, log_path=log_path, timeout=timeout, cwd=common.REPO_ROOT,
                           env=environment)


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    source = parser.add_mutually_exclusive_group(required=True)
    source.add_argument("--config", type=Path)
    source.add_argument("--run-plan", type=Path, help="execute a previously inspected plan")
    parser.add_argument("--output-dir", type=Path)
    parser.add_argument("--microbatches", nargs="+", type=int)
    parser.add_argument("--policies", nargs="+",
                        help="backend:checkpoint:microbatch combinations; default: full matrix")
    parser.add_argument("--effective-batch-size", type=int)
    parser.add_argument("--seeds", nargs="+", type=int)
    parser.add_argument("--warmup-steps", type=int,
                        help="timing exclusion only (default: 5); does not change LR warmup")
    parser.add_argument("--order-seed", type=int, help="case-order seed (default: 0)")
    parser.add_argument("--timeout-seconds", type=float,
                        help="per-case subprocess timeout (default: 600)")
    parser.add_argument("--device", choices=["cuda", "cpu"], help="pilot device (default: cuda)")
    parser.add_argument("--precision", choices=["fp32", "bf16"])
    parser.add_argument("--execute", action="store_true")
    parser.add_argument("--allow-cpu", action="store_true",
                        help="permit CPU execution for harness checks")
    args = parser.parse_args()
    if args.run_plan is not None:
        planning = (args.output_dir, args.microbatches, args.effective_batch_size, args.seeds,
                    args.precision, args.warmup_steps, args.order_seed, args.timeout_seconds,
                    args.device, args.policies)
        if any(value is not None for value in planning) or args.execute:
            parser.error("--run-plan uses the saved configuration; only --allow-cpu may accompany it")
        aggregate = execute_plan(args.run_plan, allow_cpu=args.allow_cpu)
        print(json.dumps(aggregate["status_counts"], sort_keys=True))
        return
    if args.output_dir is None or args.microbatches is None or args.effective_batch_size is None:
        parser.error("planning requires --output-dir, --microbatches, and --effective-batch-size")
    config = load_config(args.config)
    plan = make_plan(config, microbatches=args.microbatches,
                     effective_batch_size=args.effective_batch_size,
                     seeds=[config.seed] if args.seeds is None else args.seeds,
                     warmup_steps=5 if args.warmup_steps is None else args.warmup_steps,
                     device=args.device or "cuda", precision=args.precision,
                     order_seed=args.order_seed or 0,
                     timeout_seconds=600 if args.timeout_seconds is None else args.timeout_seconds,
                     policies=args.policies)
    root = write_plan(plan, args.output_dir)
    print(f"Planned {len(plan['cases'])} cases: {root / 'manifest.json'}")
    if args.execute:
        aggregate = execute_plan(root, allow_cpu=args.allow_cpu)
        print(json.dumps(aggregate["status_counts"], sort_keys=True))


if __name__ == "__main__":
    main()
