"""Bounded, recorded execution of the attention studies on a local GPU; dry run by default.

The reference launches each study stage as a cloud job with a pinned image, a
source snapshot, a hard job timeout and a cost estimate checked against a budget
(attention_lab/run_modal.py:29-150, run_extensions.py:75-283), and chains the
stages with gates (run_campaign.py:12-75).  Here the unit is a child process on
this machine's GPU and the currency is GPU-minutes, but the contract is the
same:

* ``manifest`` freezes the stage, its module and arguments, time limits, the
  sha256 of every source file and the worst-case cost before anything runs;
* ``execute`` refuses to reuse a directory, snapshots the hashed sources,
  re-checks that none changed, records the environment, runs the study in its
  own process group under a timeout (the whole group is killed on expiry, so a
  compiler child cannot outlive it) and always writes ``outcome.json``;
* ``campaign`` plans every stage first, refuses a plan whose cost at the time
  limits exceeds the budget, runs stages in order without retries and stops at
  the first stage whose study summary is not acceptable.

Layout of a run directory: ``launch.json``, ``source/``, ``environment.json``,
``command.json``, ``study.log``, ``study/`` (written by the stage) and
``outcome.json`` - what ``analyze_extensions`` reads.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import math
import os
import re
import signal
import subprocess
import sys
import time
import uuid
from datetime import datetime, timezone
from pathlib import Path

from .study import write_json

PACKAGE = Path(__file__).resolve().parents[1]
ROOT = PACKAGE.parent
_PKG = PACKAGE.name
# stage -> (module, module stage or None, default study seconds, maximum study seconds)
STAGES = {
    "smoke": (f"{_PKG}.attention.study", "smoke", 420, 480),
    "ablation": (f"{_PKG}.attention.study", "ablation", 840, 900),
    "flex_hints": (f"{_PKG}.attention.study", "flex_hints", 240, 300),
    "tuning": (f"{_PKG}.attention.study", "tuning", 840, 900),
    "confirmation": (f"{_PKG}.attention.study", "confirmation", 540, 600),
    "block": (f"{_PKG}.attention.block_benchmark", None, 360, 420),
    "decode-smoke": (f"{_PKG}.attention.decode_study", "smoke", 420, 480),
    "decode-study": (f"{_PKG}.attention.decode_study", "study", 540, 600),
    "backward-smoke": (f"{_PKG}.attention.backward_study", "smoke", 300, 480),
    "backward-study": (f"{_PKG}.attention.backward_study", "study", 540, 600),
}
CAMPAIGN_ORDER = ("smoke", "ablation", "flex_hints", "tuning", "confirmation", "block")
SOURCE_SUFFIXES = {".py", ".cu", ".cuh", ".h"}
TIMEOUT_HEADROOM = 60
RUN_ID = re.compile(r"[A-Za-z0-9_-]+")


def source_files() -> list[Path]:
    """Package sources, nested CUDA files included; build products and results are not."""
    skipped = {"__pycache__", "build", "runs", "results", "source"}
    files = []
    for directory, children, names in os.walk(PACKAGE, followlinks=False):
        children[:] = sorted(c for c in children if c not in skipped and not c.startswith("."))
        for name in sorted(names):
            path = Path(directory) / name
            if path.suffix in SOURCE_SUFFIXES:
                if path.is_symlink():
                    raise ValueError("Source file symlinks are not supported")
                files.append(path)
    return sorted(files)


def manifest(stage: str, seconds: int | None, run_id: str, *, gpus: int = 1) -> dict:
    if stage not in STAGES:
        raise ValueError(f"unknown stage {stage!r}")
    if not RUN_ID.fullmatch(run_id):
        raise ValueError("run ids may contain only letters, digits, underscores and hyphens")
    module, substage, default, maximum = STAGES[stage]
    seconds = default if seconds is None else seconds
    if not 60 <= seconds <= maximum:
        raise ValueError(f"{stage} time budget must be between 60 and {maximum} seconds")
    return {"schema_version": 1, "run_id": run_id, "stage": stage, "module": module,
            "module_stage": substage, "study_time_budget_seconds": seconds,
            "job_timeout_seconds": seconds + TIMEOUT_HEADROOM, "gpu": "B200",
            "python": "%d.%d" % sys.version_info[:2],
            "source_sha256": {str(p.relative_to(ROOT)): hashlib.sha256(p.read_bytes()).hexdigest()
                              for p in source_files()},
            "resources": {"gpus": gpus, "concurrent_jobs": 1, "retries": 0},
            "cost_estimate": {
                "gpu_minutes_at_timeout": round(gpus * (seconds + TIMEOUT_HEADROOM) / 60, 3),
                "scope": "upper bound at the job time limit; set-up before the job is not counted"}}


def study_command(settings: dict, root: Path) -> list[str]:
    command = [sys.executable, "-m", settings["module"], "--output-dir", str(root / "study")]
    if settings["module_stage"] is not None:
        command += ["--stage", settings["module_stage"]]
    command += ["--time-budget-seconds", str(settings["study_time_budget_seconds"])]
    if not settings["module"].endswith("backward_study"):
        command.append("--execute")
    if settings.get("tuning_dir"):
        command += ["--tuning-dir", settings["tuning_dir"]]
    return command


def stop_child(child) -> None:
    """End the child's whole process group, compiler subprocesses included."""
    if child.poll() is not None:
        return
    for sig in (signal.SIGTERM, signal.SIGKILL):
        try:
            os.killpg(child.pid, sig)
        except ProcessLookupError:
            return
        try:
            child.wait(timeout=3)
            return
        except subprocess.TimeoutExpired:
            continue


def environment() -> dict:
    record = {"python": sys.version}
    try:
        import torch
        record.update(torch=torch.__version__, cuda=torch.version.cuda,
                      device_count=torch.cuda.device_count(),
                      devices=[torch.cuda.get_device_name(i)
                               for i in range(torch.cuda.device_count())])
    except Exception as error:
        record["torch_error"] = str(error)
    for label, command in (("nvidia_smi", ["nvidia-smi"]), ("nvcc", ["nvcc", "--version"])):
        try:
            done = subprocess.run(command, capture_output=True, text=True, timeout=10)
            record[label] = {"stdout": done.stdout, "returncode": done.returncode}
        except (OSError, subprocess.TimeoutExpired) as error:
            record[label] = {"error": str(error)}
    return record


def run_child(command: list[str], log_path: Path, seconds: float) -> dict:
    with log_path.open("w") as log:
        child = subprocess.Popen(command, cwd=str(ROOT), stdout=log, stderr=subprocess.STDOUT,
                                 start_new_session=True)
        try:
            code = child.wait(timeout=seconds)
            return {"status": "completed" if code == 0 else "failed", "returncode": code}
        except subprocess.TimeoutExpired:
            stop_child(child)
            return {"status": "timed_out", "returncode": child.returncode}
        finally:
            stop_child(child)


def execute(settings: dict, output: Path, *, runner=run_child, require_gpu: bool = True) -> dict:
    """Run one frozen stage; ``runner`` is replaceable so tests need no GPU."""
    output = Path(output)
    if output.exists():
        raise FileExistsError(f"Refusing to replace existing run directory: {output}")
    required = settings["module"].replace(".", "/") + ".py"
    if required not in settings["source_sha256"]:
        raise FileNotFoundError(f"Study source is not part of the manifest: {required}")
    output.mkdir(parents=True)
    write_json(output / "launch.json", settings)
    started = time.monotonic()
    outcome = {"status": "failed", "run_id": settings["run_id"]}
    try:
        for name, expected in settings["source_sha256"].items():
            content = (ROOT / name).read_bytes()
            if hashlib.sha256(content).hexdigest() != expected:
                raise RuntimeError(f"Source changed after manifest creation: {name}")
            snapshot = output / "source" / name
            snapshot.parent.mkdir(parents=True, exist_ok=True)
            snapshot.write_bytes(content)
        record = environment()
        write_json(output / "environment.json", record)
        if require_gpu and not record.get("device_count"):
            raise RuntimeError("CUDA GPU is unavailable")
        command = study_command(settings, output)
        write_json(output / "command.json", {"argv": command})
        outcome.update(runner(command, output / "study.log", settings["job_timeout_seconds"]))
    except Exception as error:
        outcome.update(status="failed", error_type=type(error).__name__, error=str(error))
    outcome["wall_seconds"] = time.monotonic() - started
    write_json(output / "outcome.json", outcome)
    return outcome


def stage_acceptable(stage: str, study: dict) -> bool:
    """Tuning may contain infeasible candidates; every other stage must be complete and
    correct, with each requested baseline measured."""
    ok = study.get("status") == "passed" or (
        stage == "tuning" and study.get("status") == "completed_with_failures"
        and study.get("passed_cases", 0) > 0)
    return bool(ok and study.get("not_run_cases", 1) == 0
                and study.get("flex_failed_cases", 0) == 0)


def plan_campaign(prefix: str, *, budget_gpu_minutes: float, stages=CAMPAIGN_ORDER) -> dict:
    frozen = [manifest(stage, None, f"{prefix}-{stage}") for stage in stages]
    estimate = sum(s["cost_estimate"]["gpu_minutes_at_timeout"] for s in frozen)
    if (not math.isfinite(budget_gpu_minutes) or budget_gpu_minutes <= 0
            or estimate > budget_gpu_minutes):
        raise ValueError(f"planned {estimate:.1f} GPU-minutes exceeds the budget guard")
    return {"run_id": prefix, "gpu": "B200", "stages": frozen,
            "estimated_gpu_minutes_at_timeouts": round(estimate, 3),
            "scope": "Upper bound at the time limits; one GPU at a time, no automatic retries."}


def run_campaign(plan: dict, root: Path, *, execute_stage=execute) -> dict:
    root = Path(root)
    if root.exists():
        raise FileExistsError(f"Use a new run id: {root}")
    root.mkdir(parents=True)
    write_json(root / "campaign-plan.json", plan)
    outcomes = []
    for settings in plan["stages"]:
        stage = settings["stage"]
        if stage in ("confirmation", "block"):
            settings = {**settings, "tuning_dir": str(root / "tuning" / "study")}
        try:
            result = execute_stage(settings, root / stage)
        except Exception as error:
            outcomes.append({"stage": stage, "status": "launch_failed",
                             "error_type": type(error).__name__, "error": str(error)})
            write_json(root / "campaign-summary.json", {"status": "stopped", "outcomes": outcomes})
            return {"status": "stopped", "stage": stage, "outcomes": outcomes}
        summary_path = root / stage / "study" / "summary.json"
        study = json.loads(summary_path.read_text()) if summary_path.exists() else {}
        outcomes.append({"stage": stage, "job": result, "study": study})
        ok = result.get("status") == "completed" or stage == "tuning"
        ok = ok and stage_acceptable(stage, study)
        write_json(root / "campaign-summary.json",
                   {"status": "running" if ok else "stopped", "outcomes": outcomes})
        if not ok:
            return {"status": "stopped", "stage": stage, "outcomes": outcomes}
    write_json(root / "campaign-summary.json", {"status": "completed", "outcomes": outcomes})
    return {"status": "completed", "outcomes": outcomes}


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--stage", choices=[*STAGES, "campaign"], default="smoke")
    parser.add_argument("--time-budget-seconds", type=int)
    parser.add_argument("--budget-gpu-minutes", type=float, default=90.0)
    parser.add_argument("--run-id")
    parser.add_argument("--output-dir", type=Path)
    parser.add_argument("--tuning-dir", type=Path)
    parser.add_argument("--execute", action="store_true", help="actually start the bounded job")
    args = parser.parse_args(argv)
    stamp = datetime.now(timezone.utc).strftime("%Y%m%dT%H%M%SZ")
    run_id = args.run_id or f"attention-{args.stage}-{stamp}-{uuid.uuid4().hex[:6]}"
    output = args.output_dir or ROOT / "runs" / run_id
    try:
        if args.stage == "campaign":
            plan = plan_campaign(run_id, budget_gpu_minutes=args.budget_gpu_minutes)
        else:
            plan = manifest(args.stage, args.time_budget_seconds, run_id)
            if args.tuning_dir:
                plan["tuning_dir"] = str(args.tuning_dir)
    except ValueError as error:
        parser.error(str(error))
    if not args.execute:
        print(json.dumps(plan, indent=2))
        return 0
    result = run_campaign(plan, output) if args.stage == "campaign" else execute(plan, output)
    print(json.dumps({"status": result["status"], "output": str(output)}))
    return 0 if result["status"] == "completed" else 2


if __name__ == "__main__":
    raise SystemExit(main())
