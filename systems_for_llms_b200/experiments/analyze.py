"""Analysis of distributed experiment runs: re-verification, statistics, report.

Counterpart of the reference's analysis (distributed/analyze.py:18-621).  Given
the output directory of ``distributed_plan.run_plan`` it

* re-opens every completed case, re-runs ``inspect_case`` on the rank files and
  recomputes throughput from the raw per-step times instead of trusting the
  aggregate;
* matches every case to its single-GPU baseline on ``MATCH_KEYS`` plus a
  provenance hash (source, initial parameters, data, batch and learning-rate
  streams);
* summarises each policy across seeds (``policy_statistics``) and forms paired
  within-seed ratios for the canonical questions - DDP and TP against one GPU,
  sharded AdamW and FSDP against DDP, block checkpointing against none
  (``paired_comparisons``);
* accounts for what the launch cost: one row per stage with the wall time of its launcher
  pipeline, the GPUs it held and the GPU-minutes that makes (the reference bills dollars
  per function second, distributed/analyze.py:152-169; GPU-minutes are the unit here),
  next to the estimate recorded before the launch and the GPU-seconds the measured
  updates actually used;
* writes ``summary.json`` and a Markdown report with the hashes of its inputs, and
  optional PNG/SVG plots when matplotlib is installed (Agg backend).

Seeds are the replicates; the steps of one run are not.
"""

from __future__ import annotations

import argparse
import json
import statistics
from pathlib import Path

from . import common
from . import distributed_plan as planner

MATCH_KEYS = ("model", "context_length", "seed", "precision", "checkpointing",
              "global_batch_size", "steps", "warmup_steps")
POLICY_KEYS = tuple(k for k in MATCH_KEYS if k != "seed") + (
    "mode", "world_size", "microbatch_size", "sync_policy", "bucket_cap_mb")
METHODS = {"ddp": "DDP", "zero1": "DDP + sharded AdamW", "fsdp": "FSDP", "tp": "Tensor parallel",
           "naive": "Per-parameter all-reduce", "single": "Single GPU"}
TIMING_NOTE = ("Each optimizer step follows an inter-rank barrier and device synchronization. "
               "Reported time is the maximum rank time, including data, backward synchronization, "
               "clipping, update and loss reduction; it excludes the timing-max reduction, "
               "evaluation, setup and checkpoint writes.")
COST_NOTE = ("Active GPU-seconds per update = participating GPUs x measured training seconds / "
             "measured updates; lower-world-size baselines leave the other allocated GPUs idle.")
METRIC_FIELDS = ("tokens_per_second", "peak_cuda_allocated_bytes", "optimizer_state_bytes_max_rank",
                 "active_gpu_seconds_per_update", "valid_loss", "throughput_speedup",
                 "strong_scaling_efficiency")
RATIOS = (("tokens_per_second", "throughput_ratio"),
          ("peak_cuda_allocated_bytes", "allocated_memory_ratio"),
          ("optimizer_state_bytes_max_rank", "optimizer_state_ratio"),
          ("active_gpu_seconds_per_update", "active_gpu_seconds_ratio"))


def describe(values) -> dict:
    values = list(values)
    return {"count": len(values), "mean": statistics.mean(values),
            "median": statistics.median(values),
            "sample_sd": statistics.stdev(values) if len(values) > 1 else None,
            "min": min(values), "max": max(values)}


def verify_case(run_dir: Path, row: dict) -> dict:
    """Re-derive a completed case from its rank files; returns the enriched row."""
    case_dir = run_dir / "cases" / row["case_id"]
    case = {k: row[k] for k in ("case_id", "mode", "world_size", "model", "context_length",
                                "global_batch_size", "microbatch_size", "checkpointing",
                                "sync_policy", "bucket_cap_mb", "seed", "steps", "precision",
                                "warmup_steps", "timeout_seconds")}
    summary, signature = planner.inspect_case(case_dir, case)
    rows = common.read_jsonl(case_dir / "rank-0-metrics.jsonl")
    measured = [r["step_seconds"] for r in rows
                if r["event"] == "train" and r["step"] > case["warmup_steps"]]
    tokens = case["global_batch_size"] * case["context_length"]
    enriched = dict(row)
    enriched.update(
        tokens_per_second=len(measured) * tokens / sum(measured),
        step_seconds_median=statistics.median(measured),
        step_seconds_p90=common.percentile_linear(measured, 0.9),
        active_gpu_seconds_per_update=case["world_size"] * sum(measured) / len(measured),
        valid_loss=summary["valid_loss"],
        peak_cuda_allocated_bytes=summary.get("peak_cuda_allocated_bytes"),
        optimizer_state_bytes_max_rank=summary.get("optimizer_state_bytes_max_rank"),
        provenance_sha256=common.json_sha256(signature),
        checkpoint_comparison_provenance_sha256=common.json_sha256(
            {k: v for k, v in signature.items() if k != "source"} | {"source": signature["source"]}))
    return enriched


def policy_statistics(rows: list[dict]) -> list[dict]:
    """One entry per policy, summarised across seeds."""
    groups: dict = {}
    for row in rows:
        if row["status"] == "completed":
            groups.setdefault(tuple(row[k] for k in POLICY_KEYS), []).append(row)
    result = []
    for key, cases in sorted(groups.items(), key=lambda item: str(item[0])):
        seeds = [row["seed"] for row in cases]
        if len(set(seeds)) != len(seeds):
            raise ValueError("Repeated policy has more than one case for a seed")
        metrics = {f: describe(row[f] for row in cases) for f in METRIC_FIELDS
                   if all(row.get(f) is not None for row in cases)}
        ordered = sorted(cases, key=lambda row: row["seed"])
        result.append({"policy": dict(zip(POLICY_KEYS, key)), "seeds": sorted(seeds),
                       "case_ids": [row["case_id"] for row in ordered], "metrics": metrics})
    return result


def _references(row: dict) -> list[tuple]:
    mode, world, ckpt = row["mode"], row["world_size"], row["checkpointing"]
    found = []
    if mode in ("ddp", "tp"):
        found.append((f"{mode}_vs_single", "single", 1, ckpt))
    if mode in ("zero1", "fsdp"):
        found.append((f"{mode}_vs_ddp", "ddp", world, ckpt))
    if mode in ("ddp", "fsdp") and ckpt == "block":
        found.append((f"{mode}_block_vs_none", mode, world, "none"))
    return found


def paired_comparisons(rows: list[dict]) -> list[dict]:
    """Within-seed ratios between canonical policies with matching provenance."""
    base_keys = tuple(k for k in MATCH_KEYS if k not in ("seed", "checkpointing")) + (
        "microbatch_size", "sync_policy", "bucket_cap_mb")
    canonical = [r for r in rows if r["status"] == "completed"
                 and r["microbatch_size"] == (1 if r["context_length"] == 4096 else 4)
                 and r["sync_policy"] == "last" and r["bucket_cap_mb"] == 25]
    lookup = {}
    for row in canonical:
        key = tuple(row[k] for k in base_keys) + (row["seed"], row["mode"], row["world_size"],
                                                  row["checkpointing"])
        if key in lookup:
            raise ValueError("Ambiguous canonical policy for paired comparisons")
        lookup[key] = row
    groups: dict = {}
    for row in canonical:
        base = tuple(row[k] for k in base_keys)
        for name, mode, world, ckpt in _references(row):
            other = lookup.get(base + (row["seed"], mode, world, ckpt))
            if other is None:
                continue
            field = ("provenance_sha256" if ckpt == row["checkpointing"]
                     else "checkpoint_comparison_provenance_sha256")
            if row.get(field) != other.get(field):
                continue
            key = base + (name, row["world_size"], row["checkpointing"], world, ckpt)
            group = groups.setdefault(key, {
                "comparison": name, "settings": dict(zip(base_keys, base)),
                "numerator": {"mode": row["mode"], "world_size": row["world_size"],
                              "checkpointing": row["checkpointing"]},
                "denominator": {"mode": mode, "world_size": world, "checkpointing": ckpt},
                "pairs": []})
            values = {metric: row[f] / other[f] for f, metric in RATIOS
                      if row.get(f) is not None and other.get(f) is not None and other[f] > 0}
            values["validation_loss_difference"] = row["valid_loss"] - other["valid_loss"]
            if mode == "single":
                values["strong_scaling_efficiency"] = values["throughput_ratio"] / row["world_size"]
            group["pairs"].append({"seed": row["seed"], "numerator_case_id": row["case_id"],
                                   "denominator_case_id": other["case_id"], **values})
    result = []
    for _, group in sorted(groups.items(), key=lambda item: str(item[0])):
        group["pairs"].sort(key=lambda pair: pair["seed"])
        group["seeds"] = [pair["seed"] for pair in group["pairs"]]
        group["paired_count"] = len(group["pairs"])
        shared = set.intersection(*(set(pair) for pair in group["pairs"])) - {
            "seed", "numerator_case_id", "denominator_case_id"}
        group["metrics"] = {f: describe(pair[f] for pair in group["pairs"]) for f in sorted(shared)}
        result.append(group)
    return result


def _positive(value, what: str) -> float:
    if not common.is_finite(value, positive=True):
        raise ValueError(f"{what} must be finite and positive")
    return float(value)


def cost_rows(run_dir: str | Path, cases: list[dict] | None = None) -> list[dict]:
    """GPU-minutes per stage from the launcher's and the campaign's own records.

    ``run_dir`` is the study directory a launcher pipeline wrote (``<stage>/study``); its
    parent holds ``launch-summary.json`` and, for a campaign, the grandparent holds
    ``campaign.json`` with one record per stage.  A stage that never reported is listed
    with ``None`` figures rather than dropped.
    """
    run_dir = Path(run_dir)
    stage_root = run_dir.parent
    campaign_path = stage_root.parent / "campaign.json"
    stages = []
    if campaign_path.is_file():
        campaign = common.read_json(campaign_path)
        for definition, record in zip(campaign["definition"]["stages"], campaign["stages"]):
            stages.append((definition["name"], Path(definition["output_dir"]), definition, record))
    elif (stage_root / "launch-summary.json").is_file():
        stages.append((None, stage_root, {}, {}))
    rows = []
    for name, root, definition, record in stages:
        report_path = root / "launch-summary.json"
        report = common.read_json(report_path) if report_path.is_file() else {}
        estimate = report.get("estimate", definition.get("estimate", {}))
        gpus = report.get("gpus", definition.get("options", {}).get("gpus"))
        seconds = report.get("wall_seconds")
        used = None
        if seconds is not None and gpus is not None:
            used = (_positive(seconds, "launcher wall time") * _positive(gpus, "GPU count") / 60)
        rows.append({"stage": name or report.get("stage"),
                     "status": report.get("status", record.get("status", "not_reported")),
                     "wall_seconds": seconds, "allocated_gpus": gpus, "gpu_minutes_used": used,
                     "gpu_minutes_at_timeouts": estimate.get("worst_case_gpu_minutes"),
                     "recorded_estimate": estimate})
    if cases is not None:
        # the measured updates belong to the stage whose study directory was analysed
        active = sum(row["active_gpu_seconds_measured"] for row in cases
                     if row.get("active_gpu_seconds_measured") is not None)
        for row, (_, root, _, _) in zip(rows, stages):
            if root.resolve() == stage_root.resolve():
                row["active_gpu_minutes_measured"] = active / 60
    return rows


def build_summary(run_dir: str | Path) -> dict:
    run_dir = Path(run_dir)
    aggregate = common.read_json(run_dir / "aggregate.json")
    plan = common.read_json(run_dir / "plan.json")
    planner.validate_plan(plan)
    if aggregate["plan_sha256"] != plan["plan_sha256"]:
        raise ValueError("aggregate.json belongs to a different plan")
    rows = []
    for row in aggregate["cases"]:
        rows.append(verify_case(run_dir, row) if row["status"] == "completed" else dict(row))
    planner.add_scaling_metrics(rows, aggregate["allocated_gpus"])
    baselines = {tuple(r[k] for k in MATCH_KEYS): r for r in rows
                 if r["status"] == "completed" and r["mode"] == "single"}
    for row in rows:
        if row["status"] != "completed":
            continue
        base = baselines.get(tuple(row[k] for k in MATCH_KEYS))
        row["matched_baseline_case_id"] = base["case_id"] if base else None
    inputs = {name: common.file_sha256(run_dir / name) for name in ("aggregate.json", "plan.json")}
    return {"format_version": 1, "stage": plan["stage"], "plan_sha256": plan["plan_sha256"],
            "status": aggregate["status"], "input_sha256": inputs,
            "baseline_match_fields": list(MATCH_KEYS), "timing_note": TIMING_NOTE,
            "cost_note": COST_NOTE, "cases": rows, "policies": policy_statistics(rows),
            "paired": paired_comparisons(rows), "cost": cost_rows(run_dir, rows)}


def _fmt(value, digits=2) -> str:
    if value is None:
        return "-"
    if isinstance(value, float):
        return f"{value:,.{digits}f}"
    return str(value)


def render_report(summary: dict) -> str:
    lines = [f"# Distributed study - stage `{summary['stage']}`", "",
             f"Plan `{summary['plan_sha256'][:16]}`, status **{summary['status']}**.", "",
             summary["timing_note"], "", summary["cost_note"], "", "## Policies", "",
             "| method | GPUs | ctx | ckpt | mb | seeds | tokens/s (mean) | sd | peak GiB | opt state GiB | speed-up | efficiency |",
             "|---|---|---|---|---|---|---|---|---|---|---|---|"]
    for entry in summary["policies"]:
        policy, metrics = entry["policy"], entry["metrics"]
        def mean(field, scale=1.0):
            return metrics[field]["mean"] / scale if field in metrics else None
        lines.append("| " + " | ".join([
            METHODS.get(policy["mode"], policy["mode"]), str(policy["world_size"]),
            str(policy["context_length"]), policy["checkpointing"], str(policy["microbatch_size"]),
            str(len(entry["seeds"])), _fmt(mean("tokens_per_second"), 0),
            _fmt(metrics.get("tokens_per_second", {}).get("sample_sd"), 0),
            _fmt(mean("peak_cuda_allocated_bytes", 2 ** 30), 3),
            _fmt(mean("optimizer_state_bytes_max_rank", 2 ** 30), 3),
            _fmt(mean("throughput_speedup"), 2), _fmt(mean("strong_scaling_efficiency"), 3)]) + " |")
    lines += ["", "## Paired comparisons (within seed)", "",
              "| comparison | GPUs | pairs | throughput x | memory x | optimizer state x | val-loss diff |",
              "|---|---|---|---|---|---|---|"]
    for group in summary["paired"]:
        metrics = group["metrics"]
        def median(field):
            return metrics[field]["median"] if field in metrics else None
        lines.append("| " + " | ".join([
            group["comparison"], str(group["numerator"]["world_size"]), str(group["paired_count"]),
            _fmt(median("throughput_ratio"), 3), _fmt(median("allocated_memory_ratio"), 3),
            _fmt(median("optimizer_state_ratio"), 3),
            _fmt(median("validation_loss_difference"), 4)]) + " |")
    if summary.get("cost"):
        lines += ["", "## Cost (GPU-minutes)", "",
                  "| stage | status | GPUs | wall s | GPU-min used | GPU-min at time limits | "
                  "GPU-min in measured updates |", "|---|---|---|---|---|---|---|"]
        for row in summary["cost"]:
            lines.append("| " + " | ".join([
                str(row["stage"]), str(row["status"]), _fmt(row["allocated_gpus"]),
                _fmt(row["wall_seconds"], 1), _fmt(row["gpu_minutes_used"], 2),
                _fmt(row["gpu_minutes_at_timeouts"], 1),
                _fmt(row.get("active_gpu_minutes_measured"), 2)]) + " |")
    failed = [row for row in summary["cases"] if row["status"] != "completed"]
    if failed:
        lines += ["", "## Cases without a result", ""]
        lines += [f"- `{row['case_id']}`: {row['status']} {row.get('error', '')}" for row in failed]
    lines += ["", "Inputs: " + ", ".join(f"`{name}` {digest[:16]}"
                                         for name, digest in summary["input_sha256"].items()), ""]
    return "\n".join(lines)


def plot_series(summary: dict) -> dict:
    """Throughput against GPU count per (method, checkpointing), averaged over seeds."""
    series: dict = {}
    for entry in summary["policies"]:
        policy = entry["policy"]
        if "tokens_per_second" not in entry["metrics"] or policy["context_length"] != 1024:
            continue
        key = (policy["mode"], policy["checkpointing"])
        series.setdefault(key, []).append((policy["world_size"],
                                           entry["metrics"]["tokens_per_second"]["mean"]))
    return {key: sorted(points) for key, points in series.items()}


def write_plots(summary: dict, output: Path) -> list[str]:
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        return []
    figure, axis = plt.subplots(figsize=(7, 4.5))
    for (mode, ckpt), points in sorted(plot_series(summary).items()):
        axis.plot([p[0] for p in points], [p[1] for p in points], marker="o",
                  label=f"{METHODS.get(mode, mode)} ({ckpt})")
    axis.set_xlabel("GPUs")
    axis.set_ylabel("tokens / s")
    axis.set_xscale("log", base=2)
    axis.legend(fontsize=7)
    files = []
    for suffix in ("png", "svg"):
        path = output / f"throughput.{suffix}"
        figure.savefig(path, dpi=150, bbox_inches="tight")
        files.append(path.name)
    plt.close(figure)
    return files


def write_report(run_dir, output_dir, *, plots: bool = True) -> dict:
    output = Path(output_dir)
    output.mkdir(parents=True, exist_ok=False)
    summary = build_summary(run_dir)
    common.write_json(output / "summary.json", summary)
    files = write_plots(summary, output) if plots else []
    (output / "README.md").write_text(render_report(summary))
    return {"summary": "summary.json", "report": "README.md", "plots": files}


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--run-dir", type=Path, required=True)
    parser.add_argument("--output-dir", type=Path, required=True)
    parser.add_argument("--no-plots", action="store_true")
    args = parser.parse_args()
    print(json.dumps(write_report(args.run_dir, args.output_dir, plots=not args.no_plots), indent=2))


if __name__ == "__main__":
    main()
