"""Freeze a development-derived validation-loss target, and verify it later.

The reference's quality study (scripts/quality_target.py:57-183) derives a
target from paired development runs - ``ceil(max(validation loss at the target
step) / 0.05) * 0.05``, computed in decimal arithmetic - writes it exactly once
next to the evidence it came from, and re-validates evidence, source and data
hashes before any confirmation run uses it.  This module provides the same three
operations for pilot aggregates produced by this package:

    derive_target(aggregate, runs_dir)     -> target record (no side effects)
    freeze_target(aggregate_path, output)  -> writes frozen-target.json once ("x" mode)
    validate_frozen(path)                  -> re-hashes inputs and current sources
"""

from __future__ import annotations

import argparse
import json
from decimal import ROUND_CEILING, Decimal
from pathlib import Path

from . import common

DEFAULT_ROUNDING = "0.05"


def ceiling_to_step(value: float, step: str = DEFAULT_ROUNDING) -> str:
    """``ceil(value / step) * step`` in exact decimal arithmetic, as a string."""
    quantum = Decimal(step)
    if quantum <= 0:
        raise ValueError("rounding step must be positive")
    scaled = (Decimal(repr(value)) / quantum).to_integral_value(rounding=ROUND_CEILING)
    return str((scaled * quantum).quantize(quantum))


def _loss_at(run_dir: Path, step: int) -> float:
    events = common.read_jsonl(run_dir / "metrics.jsonl")
    matches = [e["valid_loss"] for e in events if e.get("event") == "eval" and e.get("step") == step]
    if len(matches) != 1:
        raise ValueError(f"{run_dir.name}: expected exactly one evaluation at step {step}")
    if not common.is_finite(matches[0]):
        raise ValueError(f"{run_dir.name}: non-finite validation loss at step {step}")
    return matches[0]


def derive_target(aggregate: dict, runs_dir: Path, *, target_step: int,
                  rounding: str = DEFAULT_ROUNDING) -> dict:
    """Target from a pilot aggregate whose cases all completed comparably."""
    if aggregate.get("comparability", {}).get("status") != "passed":
        raise ValueError("development comparability did not pass")
    rows = aggregate["cases"]
    if not rows or any(row["status"] != "completed" for row in rows):
        raise ValueError("every development case must complete")
    if len({row["batch_stream_sha256"] for row in rows}) != 1:
        raise ValueError("development cases did not see the same batches")
    losses = {row["case_id"]: _loss_at(Path(runs_dir) / row["case_id"], target_step) for row in rows}
    worst = max(losses.values())
    return {"target_step": target_step, "target_rounding": rounding,
            "target_rule": f"ceil(max(development validation losses at step {target_step}) / "
                           f"{rounding}) * {rounding}",
            "development_losses": losses, "max_development_loss": worst,
            "target_validation_loss": ceiling_to_step(worst, rounding),
            "data_identity_sha256": rows[0]["data_identity_sha256"],
            "batch_stream_sha256": rows[0]["batch_stream_sha256"],
            "plan_sha256": aggregate["plan_sha256"]}


def freeze_target(aggregate_path: Path, output_path: Path, *, target_step: int,
                  rounding: str = DEFAULT_ROUNDING) -> dict:
    aggregate_path = Path(aggregate_path).resolve()
    aggregate = common.read_json(aggregate_path)
    root = aggregate_path.parent
    target = derive_target(aggregate, root / "runs", target_step=target_step, rounding=rounding)
    manifest = common.read_json(root / "manifest.json")
    inputs = {"aggregate.json": common.file_sha256(aggregate_path),
              "manifest.json": common.file_sha256(root / "manifest.json")}
    for case_id in target["development_losses"]:
        inputs[f"runs/{case_id}/metrics.jsonl"] = common.file_sha256(
            root / "runs" / case_id / "metrics.jsonl")
    record = {"format_version": 1, "target": target, "evidence_root": str(root),
              "input_sha256": inputs,
              "source_sha256": manifest["source"]["python_source_sha256"]}
    record["frozen_sha256"] = common.json_sha256({k: v for k, v in record.items()})
    with open(output_path, "x") as handle:      # a target is frozen exactly once
        handle.write(json.dumps(record, indent=2, allow_nan=False) + "\n")
    return record


def validate_frozen(path: Path, *, check_source: bool = True) -> dict:
    record = common.read_json(path)
    body = {k: v for k, v in record.items() if k != "frozen_sha256"}
    if record.get("format_version") != 1 or common.json_sha256(body) != record.get("frozen_sha256"):
        raise ValueError("frozen target was modified")
    root = Path(record["evidence_root"])
    for relative, digest in record["input_sha256"].items():
        if common.file_sha256(root / relative) != digest:
            raise ValueError(f"evidence changed after the target was frozen: {relative}")
    aggregate = common.read_json(root / "aggregate.json")
    again = derive_target(aggregate, root / "runs", target_step=record["target"]["target_step"],
                          rounding=record["target"]["target_rounding"])
    if again != record["target"]:
        raise ValueError("re-derived target differs from the frozen one")
    if check_source:
        from ..train import source_identity
        if source_identity()["python_source_sha256"] != record["source_sha256"]:
            raise ValueError("training source changed since the target was frozen")
    return record


def time_to_target(run_dir: Path, target: float) -> dict | None:
    """First evaluation at or below the target: step, tokens and training seconds."""
    seconds_by_step = {}
    for event in common.read_jsonl(Path(run_dir) / "metrics.jsonl"):
        if event.get("event") == "train":
            seconds_by_step[event["step"]] = event["train_seconds"]
        elif event.get("event") == "eval" and event["valid_loss"] <= target:
            return {"step": event["step"], "valid_loss": event["valid_loss"],
                    "train_seconds": seconds_by_step.get(event["step"])}
    return None


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = parser.add_subparsers(dest="command", required=True)
    freeze = sub.add_parser("freeze")
    freeze.add_argument("--aggregate", type=Path, required=True)
    freeze.add_argument("--output", type=Path, required=True)
    freeze.add_argument("--target-step", type=int, required=True)
    freeze.add_argument("--rounding", default=DEFAULT_ROUNDING)
    check = sub.add_parser("validate")
    check.add_argument("--target", type=Path, required=True)
    args = parser.parse_args()
    if args.command == "freeze":
        record = freeze_target(args.aggregate, args.output, target_step=args.target_step,
                               rounding=args.rounding)
    else:
        record = validate_frozen(args.target)
    print(json.dumps(record["target"], indent=2))


if __name__ == "__main__":
    main()
