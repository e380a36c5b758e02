"""Bounded single-GPU study stages: several pilot jobs run one after another.

Equivalent of the reference's study runner (scripts/run_study.py:41-192): a stage
is a list of pilot jobs (config, microbatches, effective batch, seeds, optional
policy list, overrides, per-case and per-job limits); ``build_plan`` resolves a
stage - ``development`` (memory/throughput screens plus the quality development
run), ``timing-confirmation``, ``quality-confirmation`` or ``confirmation`` (both);
``run_stage`` snapshots the source hash, runs each job through ``pilot`` and
classifies it as ``completed``, ``completed_with_resource_limits`` (only OOM or
time-outs in jobs that allow them) or ``blocked``; a blocked job stops the stage.
Quality-confirmation stages refuse to start without a validated frozen target.
Default invocation prints the plan; ``--execute`` runs it.
"""

from __future__ import annotations

import argparse
import json
from dataclasses import replace
from pathlib import Path

from .. import pilot
from ..config import load_config
from ..train import source_identity
from . import common, quality_target

QUALITY_STAGES = ("quality-confirmation", "confirmation")
STAGES = ("development", "timing-confirmation", *QUALITY_STAGES)
QUALITY_PROTOCOL = {
    "workload": "100M/1K", "policies": ["sdpa:none:8", "sdpa:none:1", "sdpa:block:8"],
    "development_seed": 1337, "confirmation_seeds": [2027, 2028, 2029], "max_steps": 1200,
    "tokens_per_step": 8192, "train_warmup_steps": 50, "eval_interval": 50, "eval_batches": 64,
    "eval_batch_size": 1, "checkpoint_interval": 1200,
    "allocated_memory_budget_bytes": 3 * 2 ** 30,
    "memory_scope": "allocated memory only; does not establish fit on a physical 3 GiB GPU",
    "target_rule": "ceil(max(development validation losses at step 600) / 0.05) * 0.05",
    "target_step": 600, "target_rounding": "0.05",
    "confirmation_gate": "freeze numeric target and development evidence hashes before confirmation",
    "time_to_target_scope": ("first observed evaluation at or below the target; no interpolation; "
                             "training seconds up to that step"),
}
_QUALITY_OVERRIDES = {"max_steps": 1200, "warmup_steps": 50, "eval_interval": 50,
                      "eval_batches": 64, "checkpoint_interval": 1200}


def _job(name, config, microbatches, effective, *, seeds=None, case_timeout=120, job_timeout=1800,
         overrides=None, policies=None, allow_limits=False) -> dict:
    seeds = [1337] if seeds is None else seeds
    per_seed = len(policies) if policies else len(microbatches) * 4
    return {"name": name, "config": f"configs/{config}.json", "microbatches": microbatches,
            "effective_batch_size": effective, "seeds": seeds, "warmup_steps": 5,
            "case_timeout_seconds": case_timeout, "job_timeout_seconds": job_timeout,
            "overrides": overrides or {}, "policies": policies,
            "allow_resource_limits": allow_limits, "case_count": per_seed * len(seeds)}


def build_plan(stage: str, *, synthetic: bool = True) -> dict:
    """``synthetic`` selects the configs that need no dataset on disk."""
    if stage not in STAGES:
        raise ValueError(f"Unknown stage: {stage}")
    prefix = "synthetic" if synthetic else "scale"
    quality = dict(policies=QUALITY_PROTOCOL["policies"], overrides=dict(_QUALITY_OVERRIDES),
                   case_timeout=600, job_timeout=2400)
    if stage == "development":
        jobs = [
            _job("22m-4k-screen", f"{prefix}-22m-s4096", [1, 2], 2, allow_limits=True),
            _job("324m-1k-screen", f"{prefix}-324m-s1024", [1, 8], 8, case_timeout=180,
                 job_timeout=2400, allow_limits=True),
            _job("324m-4k-screen", f"{prefix}-324m-s4096", [1, 2], 2, case_timeout=300,
                 job_timeout=3600, allow_limits=True),
            _job("100m-1k-quality-dev", f"{prefix}-100m-s1024", [1, 8], 8, **quality),
        ]
    else:
        quality_jobs = [_job(f"100m-1k-quality-seed{seed}", f"{prefix}-100m-s1024", [1, 8], 8,
                             seeds=[seed], **quality)
                        for seed in QUALITY_PROTOCOL["confirmation_seeds"]]
        short = {"max_steps": 60, "checkpoint_interval": 60}
        timing_jobs = [
            _job("100m-1k-timing", f"{prefix}-100m-s1024", [1, 8], 8, seeds=[2027, 2028, 2029],
                 case_timeout=180, job_timeout=2400, overrides=short),
            _job("100m-4k-timing", f"{prefix}-100m-s4096", [1, 2], 2, seeds=[2027, 2028, 2029],
                 case_timeout=180, job_timeout=2400, overrides=short)]
        jobs = {"quality-confirmation": quality_jobs, "timing-confirmation": timing_jobs,
                "confirmation": quality_jobs + timing_jobs}[stage]
    seconds = sum(job["job_timeout_seconds"] for job in jobs)
    plan = {"format_version": 1, "stage": stage, "gpu": "B200", "concurrent_jobs": 1,
            "jobs": jobs, "quality_protocol": QUALITY_PROTOCOL,
            "case_count": sum(job["case_count"] for job in jobs),
            "max_job_seconds_sum": seconds, "gpu_minutes_at_time_limits": seconds / 60,
            "cost_scope": "job time limits only; one GPU"}
    return common.seal(plan)


def classify_job(aggregate: dict, allow_resource_limits: bool) -> str:
    counts = aggregate["status_counts"]
    if set(counts) <= {"completed"} and aggregate["comparability"]["status"] == "passed":
        return "completed"
    limited = {row.get("failure_kind") for row in aggregate["cases"] if row["status"] != "completed"}
    only_limits = limited <= {"oom", "timeout"} and all(
        row["status"] in ("completed", "failed", "timeout") for row in aggregate["cases"])
    if allow_resource_limits and only_limits and aggregate["comparability"]["status"] != "failed":
        return "completed_with_resource_limits"
    return "blocked"


def plan_job(job: dict, output: Path, *, device: str) -> Path:
    config = load_config(common.REPO_ROOT / job["config"])
    if job["overrides"]:
        config = replace(config, **job["overrides"])
    plan = pilot.make_plan(config, microbatches=job["microbatches"],
                           effective_batch_size=job["effective_batch_size"], seeds=job["seeds"],
                           warmup_steps=job["warmup_steps"], device=device,
                           timeout_seconds=job["case_timeout_seconds"], policies=job["policies"])
    return pilot.write_plan(plan, output)


def run_stage(plan: dict, output: Path, *, device: str = "cuda", target_file: Path | None = None,
              execute_job=None) -> dict:
    if not common.verify_seal(plan):
        raise ValueError("study plan was modified")
    if plan["stage"] in QUALITY_STAGES:
        if target_file is None:
            raise ValueError("quality confirmation needs a frozen target file")
        frozen = quality_target.validate_frozen(target_file)
        target = frozen["target"]["target_validation_loss"]
    else:
        target = None
    output = Path(output)
    output.mkdir(parents=True, exist_ok=False)
    snapshot = source_identity()["python_source_sha256"]
    execute_job = execute_job or (lambda root: pilot.execute_plan(root, allow_cpu=device == "cpu"))
    record = {"format_version": 1, "stage": plan["stage"], "plan_sha256": plan["plan_sha256"],
              "source_sha256": snapshot, "target_validation_loss": target, "jobs": [],
              "status": "running"}
    common.write_json(output / "study.json", record)
    for job in plan["jobs"]:
        entry = {"name": job["name"], "status": "running"}
        record["jobs"].append(entry)
        try:
            if source_identity()["python_source_sha256"] != snapshot:
                raise RuntimeError("source changed while the stage was running")
            root = plan_job(job, output / job["name"], device=device)
            aggregate = execute_job(root)
            entry["status_counts"] = aggregate["status_counts"]
            entry["status"] = classify_job(aggregate, job["allow_resource_limits"])
            if target is not None:
                entry["time_to_target"] = {
                    row["case_id"]: quality_target.time_to_target(root / "runs" / row["case_id"],
                                                                  float(target))
                    for row in aggregate["cases"] if row["status"] == "completed"}
        except Exception as error:
            entry.update(status="blocked", error=str(error))
        common.write_json(output / "study.json", record)
        if entry["status"] == "blocked":
            record["status"] = "blocked"
            break
    if record["status"] == "running":
        limited = any(j["status"] == "completed_with_resource_limits" for j in record["jobs"])
        record["status"] = "completed_with_resource_limits" if limited else "completed"
    common.write_json(output / "study.json", record)
    return record


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--stage", choices=STAGES, default="development")
    parser.add_argument("--output-dir", type=Path)
    parser.add_argument("--device", choices=["cuda", "cpu"], default="cuda")
    parser.add_argument("--target-file", type=Path)
    parser.add_argument("--real-data", action="store_true",
                        help="use the scale-* configs (token arrays on disk) instead of synthetic-*")
    parser.add_argument("--execute", action="store_true")
    args = parser.parse_args()
    plan = build_plan(args.stage, synthetic=not args.real_data)
    if not args.execute:
        print(json.dumps(plan, indent=2))
        return
    if args.output_dir is None:
        parser.error("--execute requires --output-dir")
    record = run_stage(plan, args.output_dir, device=args.device, target_file=args.target_file)
    print(json.dumps({"status": record["status"],
                      "jobs": [(j["name"], j["status"]) for j in record["jobs"]]}, indent=2))
    if record["status"] == "blocked":
        raise SystemExit(1)


if __name__ == "__main__":
    main()
