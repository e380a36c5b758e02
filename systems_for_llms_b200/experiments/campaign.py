"""Two-stage campaign: correctness gate on two GPUs, then the eight-GPU study.

Same contract as the reference campaign (distributed/run_campaign.py:32-116):
``prepare_campaign`` freezes the payload manifest and both plans into one
definition with a hash and checks the worst-case cost against a budget (here
GPU-minutes rather than dollars) before anything runs; ``execute_campaign`` may
run a definition once, re-verifies definition and sources before each stage,
lets the smoke stage gate the scale stage, stops at the first failure without
retries and records every outcome in ``campaign.json``.
"""

from __future__ import annotations

import argparse
import json
import uuid
from datetime import datetime, timezone
from pathlib import Path

from . import common, launcher
from . import distributed_plan as planner

BUDGET_GPU_MINUTES = 600.0
STAGES = (("smoke", 2, 900), ("scale", 8, 2400))


def definition_hash(definition: dict) -> str:
    return common.json_sha256(definition)


def prepare_campaign(config_path, output_dir, *, stages=STAGES,
                     budget_gpu_minutes: float = BUDGET_GPU_MINUTES, device: str = "cuda") -> dict:
    output = Path(output_dir).resolve()
    if output.exists():
        raise FileExistsError(f"Output directory already exists: {output}")
    config = Path(config_path).resolve()
    if not config.is_file():
        raise FileNotFoundError(f"Config does not exist: {config}")
    payload = launcher.prepare_payload()
    stamp = datetime.now(timezone.utc).strftime("distributed-%Y%m%dT%H%M%SZ-")
    campaign_id = stamp + uuid.uuid4().hex[:8]
    frozen = []
    for stage, gpus, seconds in stages:
        options = {"stage": stage, "gpus": gpus, "timeout_seconds": seconds, "device": device}
        checked = launcher.validate_options(options)
        planner.validate_plan(checked["plan"])
        frozen.append({"name": stage, "options": options, "plan": checked["plan"],
                       "output_dir": str(output / stage), "estimate": checked["estimate"],
                       "job_gpu_minutes_at_timeout": seconds * gpus / 60})
    worst = sum(stage["job_gpu_minutes_at_timeout"] for stage in frozen)
    if worst > budget_gpu_minutes:
        raise ValueError(f"Worst-case {worst:.0f} GPU-minutes exceeds the working budget of "
                         f"{budget_gpu_minutes:.0f}")
    definition = {
        "campaign_id": campaign_id, "output_dir": str(output), "config_path": str(config),
        "config_sha256": common.file_sha256(config), "working_budget_gpu_minutes": budget_gpu_minutes,
        "gpu_minutes_at_timeouts": worst, "payload": payload, "stages": frozen,
        "cost_scope": ("All allocated GPUs count during every case; set-up and test time are "
                       "inside the per-stage job limit."),
        "failure_policy": ("Stop at the first failed gate or stage; no retries and no automatic "
                           "confirmation stage.")}
    return {"format_version": 1, "status": "planned", "definition": definition,
            "definition_sha256": definition_hash(definition),
            "stages": [{"name": stage["name"], "status": "not_run"} for stage in frozen]}


def _verify(campaign: dict) -> None:
    definition = campaign["definition"]
    if campaign["definition_sha256"] != definition_hash(definition):
        raise ValueError("Frozen campaign definition changed; prepare a new campaign")
    launcher.verify_payload(definition["payload"])
    if common.file_sha256(definition["config_path"]) != definition["config_sha256"]:
        raise RuntimeError("Config changed after the campaign was frozen; prepare a new campaign")
    for stage in definition["stages"]:
        planner.validate_plan(stage["plan"])


def run_stage(stage: dict, base_config: dict) -> dict:
    """One launcher pipeline; separated so tests can substitute it."""
    return launcher.run_pipeline(stage["options"], base_config, Path(stage["output_dir"]))


def execute_campaign(campaign: dict) -> dict:
    _verify(campaign)
    if campaign["status"] != "planned":
        raise ValueError("A campaign can only execute once")
    definition = campaign["definition"]
    output = Path(definition["output_dir"])
    output.mkdir(parents=True, exist_ok=False)
    base_config = common.read_json(definition["config_path"])

    def save():
        common.write_json(output / "campaign.json", campaign)

    campaign["status"] = "running"
    save()
    for index, stage in enumerate(definition["stages"]):
        record = campaign["stages"][index]
        try:
            _verify(campaign)
            record["status"] = "running"
            save()
            print(f"Starting {stage['name']}: {stage['options']['gpus']} GPUs, "
                  f"{len(stage['plan']['cases'])} cases", flush=True)
            summary = run_stage(stage, base_config)
            record["summary"] = {k: v for k, v in summary.items() if k != "preflight"}
            record["status"] = summary["status"]
            if isinstance(summary.get("wall_seconds"), (int, float)):
                record["gpu_minutes_used"] = summary["wall_seconds"] * stage["options"]["gpus"] / 60
            if summary["status"] != "completed":
                raise RuntimeError(f"{stage['name']} did not pass; later stages are blocked")
        except Exception as error:
            record.update(status="failed", error=str(error))
            campaign["status"] = "failed"
            for later in campaign["stages"][index + 1:]:
                later["blocked_by"] = stage["name"]
            save()
            return campaign
        save()
    campaign["status"] = "completed"
    save()
    return campaign


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--config", type=Path,
                        default=common.REPO_ROOT / "configs" / "synthetic-324m-s1024.json")
    parser.add_argument("--output-dir", type=Path, required=True)
    parser.add_argument("--execute", action="store_true")
    args = parser.parse_args()
    try:
        campaign = prepare_campaign(args.config, args.output_dir)
    except (FileNotFoundError, FileExistsError, ValueError) as error:
        parser.error(str(error))
    brief = {"mode": "execute" if args.execute else "dry_run", "status": campaign["status"],
             "definition_sha256": campaign["definition_sha256"],
             "gpu_minutes_at_timeouts": campaign["definition"]["gpu_minutes_at_timeouts"],
             "stages": [(s["name"], len(s["plan"]["cases"])) for s in campaign["definition"]["stages"]]}
    print(json.dumps(brief, indent=2), flush=True)
    if args.execute:
        result = execute_campaign(campaign)
        print(json.dumps({"status": result["status"], "stages": result["stages"]}, indent=2))
        if result["status"] != "completed":
            raise SystemExit(1)


if __name__ == "__main__":
    main()
