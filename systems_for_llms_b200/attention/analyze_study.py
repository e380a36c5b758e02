"""Summaries of recorded attention experiments; never runs GPU work.

What the reference's analysis reports (attention_lab/analyze_study.py:62-357),
for run directories written by ``study.run_study`` and
``block_benchmark.run_block_study``:

* ablation ratios between lowering variants, paired only when workload, input
  seed, configuration, and recorded environment all match; every group that
  could not be paired is counted under the reason (missing, failed, ambiguous,
  incompatible, not applicable) instead of being dropped silently;
* confirmation ratios (fixed default over transferred winner);
* baseline ratios against SDPA and FlexAttention, tuning configurations kept
  separate rather than reporting only the best;
* block-level and isolated-attention ratios;
* first-call observations, a per-workload tuning table with Spearman rank
  associations, and regret statistics of the offline search replay.

A ratio above one favours the denominator.  A missing measurement is never
counted as a success.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import math
import statistics
from collections import defaultdict
from pathlib import Path

ABLATION_PAIRS = (("csr_masked", "csr_full"), ("csr_full", "interval_split"),
                  ("interval_masked", "interval_split"))
_IDENTITY = ("workload_id", "length", "dim", "batch", "heads", "dtype", "spec", "document_ids",
             "seed")
_ENVIRONMENT = ("hardware", "software", "timing_scope", "warmup", "repeats", "inner_repeats")


def read(path):
    return json.loads(Path(path).read_text())


def positive(value) -> bool:
    return (isinstance(value, (int, float)) and not isinstance(value, bool)
            and math.isfinite(value) and value > 0)


def eligible(measurement: dict) -> bool:
    return (measurement.get("status") == "passed" and measurement.get("correct") is True
            and positive(measurement.get("latency_ms")))


def group_key(record: dict, *, configuration: bool = True, environment: bool = True) -> str:
    case, measured = record["case"], record["measurement"]
    key = {name: case.get(name) for name in _IDENTITY}
    if environment:
        key.update({name: measured.get(name) for name in _ENVIRONMENT})
    if configuration:
        config = dict(case.get("config") or {})
        # the lowering variant is what an ablation compares; tile sizes must still match
        config.pop("implementation", None)
        config.pop("use_full_blocks", None)
        key["config"] = config
    return json.dumps(key, sort_keys=True)


def ratio_stats(pairs: list[dict]) -> dict:
    values = [pair["ratio"] for pair in pairs]
    return {"paired_cases": len(values),
            "geomean_speedup": math.exp(statistics.mean(map(math.log, values))) if values else None,
            "median_speedup": statistics.median(values) if values else None,
            "min_speedup": min(values, default=None), "max_speedup": max(values, default=None),
            "regressions": sum(v < 1 for v in values),
            "regressions_over_5_percent": sum(v < 1 / 1.05 for v in values),
            "improvements": sum(v > 1 for v in values), "ties": sum(v == 1 for v in values)}


def _label(case: dict, confirmation: bool):
    if not confirmation:
        return case.get("variant")
    selection = case.get("selection")
    if selection == "fixed_default":
        return "fixed_default"
    if isinstance(selection, dict) and (selection.get("policy")
                                        == "fastest_correct_training_configuration"):
        return "transferred"
    return None


def comparisons(records: list[dict], *, confirmation: bool = False) -> list[dict]:
    groups = defaultdict(lambda: defaultdict(list))
    for record in records:
        label = _label(record["case"], confirmation)
        if label is not None:
            key = group_key(record, configuration=not confirmation, environment=False)
            groups[key][label].append(record)
    wanted = (("fixed_default", "transferred"),) if confirmation else ABLATION_PAIRS
    reports = []
    for left_label, right_label in wanted:
        pairs = []
        counts = dict.fromkeys(("missing_counterpart_groups", "failed_groups", "ambiguous_groups",
                                "incompatible_environment_groups", "not_applicable_groups"), 0)
        for group in groups.values():
            if left_label not in group and right_label not in group:
                continue
            sample = next(iter(group.values()))[0]["case"]
            if right_label.startswith("interval") and (sample.get("spec") or {}).get("same_document"):
                counts["not_applicable_groups"] += 1
                continue
            left, right = group.get(left_label, []), group.get(right_label, [])
            if not left or not right:
                counts["missing_counterpart_groups"] += 1
            elif len(left) != 1 or len(right) != 1:
                counts["ambiguous_groups"] += 1
            elif not (eligible(left[0]["measurement"]) and eligible(right[0]["measurement"])):
                counts["failed_groups"] += 1
            elif (group_key(left[0], configuration=not confirmation)
                  != group_key(right[0], configuration=not confirmation)):
                counts["incompatible_environment_groups"] += 1
            else:
                a, b = left[0], right[0]
                pairs.append({"comparison": f"{left_label}/{right_label}",
                              "workload_id": b["case"]["workload_id"], "seed": b["case"]["seed"],
                              "left_case_id": a["case"]["case_id"],
                              "right_case_id": b["case"]["case_id"],
                              "left_latency_ms": a["measurement"]["latency_ms"],
                              "right_latency_ms": b["measurement"]["latency_ms"],
                              "ratio": (a["measurement"]["latency_ms"]
                                        / b["measurement"]["latency_ms"])})
        by_workload = defaultdict(list)
        for pair in pairs:
            by_workload[pair["workload_id"]].append(pair)
        reports.append({"comparison": f"{left_label}/{right_label}", **ratio_stats(pairs), **counts,
                        "pairs": pairs, "by_workload": {k: ratio_stats(v)
                                                        for k, v in sorted(by_workload.items())}})
    return reports


def candidate_label(case: dict) -> str:
    config = case["config"]
    label = f"{case['variant']}:{config['block_q']}x{config['block_k']}"
    selection = case.get("selection")
    selection = "transferred" if isinstance(selection, dict) else selection
    return label + (f":{selection}" if selection else "")


def baselines(records: list[dict], directory: Path) -> list[dict]:
    by_id = {record["case"]["case_id"]: record for record in records}
    pairs_path = Path(directory) / "baseline_pairs.json"
    sources = ({item["case_id"]: item.get("baseline_source_case_id") for item in read(pairs_path)}
               if pairs_path.exists() else {})
    groups = defaultdict(lambda: {"pairs": [], "unavailable": 0, "candidate_failed": 0})
    for record in records:
        case, measured = record["case"], record["measurement"]
        for baseline in ("sdpa", "flex"):
            if baseline == "sdpa":
                source, latency = record, measured.get("baseline_latency_ms")
                profile = measured.get("baseline", "unspecified")
                available = positive(latency)
            else:
                source = (record if eligible(measured.get("flex", {}))
                          else by_id.get(sources.get(case["case_id"])))
                flex = source["measurement"].get("flex", {}) if source else {}
                latency = flex.get("latency_ms")
                profile = "contiguous_blocks" if flex.get("contiguous_hint") else "default"
                available = (source is not None and eligible(flex)
                             and group_key(source, configuration=False)
                             == group_key(record, configuration=False))
            group = groups[(candidate_label(case), baseline, profile)]
            if not eligible(measured):
                group["candidate_failed"] += 1
            elif not available:
                group["unavailable"] += 1
            else:
                group["pairs"].append({"workload_id": case["workload_id"], "seed": case["seed"],
                                       "case_id": case["case_id"],
                                       "baseline_source_case_id": source["case"]["case_id"],
                                       "baseline_latency_ms": latency,
                                       "candidate_latency_ms": measured["latency_ms"],
                                       "ratio": latency / measured["latency_ms"]})
    return [{"candidate": key[0], "baseline": key[1], "baseline_variant": key[2],
             **ratio_stats(value["pairs"]), "baseline_unavailable": value["unavailable"],
             "candidate_failed": value["candidate_failed"], "pairs": value["pairs"]}
            for key, value in sorted(groups.items())]


def block_variant_ok(value: dict, field: str = "block_latency_ms") -> bool:
    return (value.get("status") == "passed" and value.get("correct") is True
            and positive(value.get(field)))


def block_eligible(measured: dict) -> bool:
    variants = measured.get("variants", {})
    return (measured.get("status") == "passed" and measured.get("correct") is True
            and measured.get("reference_finite") is True
            and measured.get("inputs_weights_unchanged") is True
            and all(block_variant_ok(variants.get(name, {}))
                    for name in ("custom_interval_split", "sdpa")))


def block_comparisons(records: list[dict]) -> list[dict]:
    groups = defaultdict(lambda: {"pairs": [], "failed_or_unavailable": 0})
    for record in records:
        case, measured = record["case"], record["measurement"]
        variants = measured.get("variants", {})
        candidate = variants.get("custom_interval_split", {})
        for name, baseline in variants.items():
            if name == "custom_interval_split":
                continue
            for scope, field in (("single_block_forward", "block_latency_ms"),
                                 ("isolated_attention_forward", "attention_latency_ms")):
                group = groups[(name, scope)]
                valid = (measured.get("inputs_weights_unchanged") is True
                         and measured.get("reference_finite") is True
                         and block_variant_ok(candidate, field) and block_variant_ok(baseline, field))
                if not valid:
                    group["failed_or_unavailable"] += 1
                    continue
                group["pairs"].append({
                    "case_id": case["case_id"], "seed": case["seed"], "length": case["length"],
                    "dim": case["dim"], "pattern": case["pattern"], "config": case["config"],
                    "selection": case.get("selection"), "candidate_latency_ms": candidate[field],
                    "baseline_latency_ms": baseline[field],
                    "ratio": baseline[field] / candidate[field],
                    "isolated_attention_fraction": measured.get(
                        f"isolated_attention_fraction_{name}"),
                    "amdahl_estimate": measured.get(f"amdahl_estimate_vs_{name}")})
    return [{"baseline": key[0], "scope": key[1], **ratio_stats(value["pairs"]),
             "failed_or_unavailable": value["failed_or_unavailable"], "pairs": value["pairs"],
             "interpretation": ("Same weights, operators and input seed within a case; one bf16 "
                                "inference block, not a whole model. Attention and block times are "
                                "separate measurements; Amdahl figures are illustrative.")}
            for key, value in sorted(groups.items())]


def ranks(values: list[float]) -> list[float]:
    """Average ranks, ties sharing the mean of the positions they span."""
    order = sorted(range(len(values)), key=values.__getitem__)
    result, start = [0.0] * len(values), 0
    while start < len(order):
        end = start + 1
        while end < len(order) and values[order[end]] == values[order[start]]:
            end += 1
        for index in order[start:end]:
            result[index] = (start + end - 1) / 2
        start = end
    return result


def spearman(rows: list[dict], field: str) -> dict:
    points = [(row[field], row["latency_ms"]) for row in rows
              if isinstance(row.get(field), (int, float)) and not isinstance(row[field], bool)
              and math.isfinite(row[field])]
    if len(points) < 3:
        return {"samples": len(points), "spearman_rho": None}
    x, y = ranks([p[0] for p in points]), ranks([p[1] for p in points])
    constant = len(set(x)) == 1 or len(set(y)) == 1
    return {"samples": len(points),
            "spearman_rho": None if constant else statistics.correlation(x, y)}


TUNING_FIELDS = ("block_q", "block_k", "mask_density", "first_call_ms")


def tuning(records: list[dict]) -> list[dict]:
    rows, failures = defaultdict(list), defaultdict(list)
    for record in records:
        case, measured = record["case"], record["measurement"]
        if not eligible(measured):
            failures[case["workload_id"]].append({"case_id": case["case_id"],
                                                  "config": case["config"],
                                                  "status": measured.get("status"),
                                                  "error": measured.get("error")})
            continue
        rows[case["workload_id"]].append({
            "case_id": case["case_id"], "config": case["config"],
            "latency_ms": measured["latency_ms"], "block_q": case["config"]["block_q"],
            "block_k": case["config"]["block_k"], "mask_density": measured.get("mask_density"),
            "first_call_ms": measured.get("first_call_ms")})
    return [{"workload_id": workload, "valid_configurations": len(rows[workload]),
             "failed_configurations": failures[workload],
             "rows_by_latency": sorted(rows[workload], key=lambda row: row["latency_ms"]),
             "associations": {field: spearman(rows[workload], field) for field in TUNING_FIELDS},
             "scope": "Rank associations across configurations of one workload; not causal."}
            for workload in sorted(set(rows) | set(failures))]


def regret_stats(key, values: list) -> dict:
    valid = [v for v in values if v is not None]
    return {"method": key[0], "budget": key[1], "trials": len(values),
            "failed_trials": len(values) - len(valid),
            "mean_relative_regret": statistics.mean(valid) if valid else None,
            "median_relative_regret": statistics.median(valid) if valid else None,
            "max_relative_regret": max(valid, default=None)}


def replay_summary(directory: Path):
    path = Path(directory) / "search_replay.json"
    if not path.exists():
        return None
    replay, overall, per_workload = read(path), defaultdict(list), []
    for workload in replay.get("workloads", []):
        local = defaultdict(list)
        for trial in workload.get("trials", []):
            value = trial.get("relative_regret")
            ok = (isinstance(value, (int, float)) and not isinstance(value, bool)
                  and math.isfinite(value) and value >= 0)
            for table in (local, overall):
                table[(trial["method"], trial["budget"])].append(value if ok else None)
        per_workload.append({"workload_id": workload["workload_id"], "status": workload["status"],
                             "groups": [regret_stats(k, v) for k, v in sorted(local.items())]})
    return {"methodology": replay.get("methodology"), "workloads": per_workload,
            "groups": [regret_stats(k, v) for k, v in sorted(overall.items())]}


def setup_observations(records: list[dict]) -> list[dict]:
    groups = defaultdict(list)
    for record in records:
        measured = record["measurement"]
        if eligible(measured):
            groups[record["case"]["variant"]].append(
                {"case_id": record["case"]["case_id"],
                 "first_call_ms": measured.get("first_call_ms"),
                 "flex_first_call_ms": measured.get("flex", {}).get("first_call_ms")})
    result = []
    for variant, rows in sorted(groups.items()):
        fields = {}
        for field in ("first_call_ms", "flex_first_call_ms"):
            values = [row[field] for row in rows if positive(row[field]) or row[field] == 0]
            fields[field] = {"samples": len(values),
                             "median": statistics.median(values) if values else None,
                             "min": min(values, default=None), "max": max(values, default=None)}
        result.append({"variant": variant, "statistics_ms": fields, "cases": rows,
                       "scope": ("Successful candidates only; a first call includes mask upload, "
                                 "library load or cache lookup, launch and synchronisation.")})
    return result


def analyze_directory(directory) -> dict:
    directory = Path(directory)
    paths = sorted((directory / "cases").glob("*.json"))
    records = [read(path) for path in paths]
    identifiers = [record["case"]["case_id"] for record in records]
    if len(identifiers) != len(set(identifiers)):
        raise ValueError(f"Duplicate case IDs in {directory}")
    plan = read(directory / "plan.json") if (directory / "plan.json").exists() else {}
    status = read(directory / "summary.json") if (directory / "summary.json").exists() else {}
    stage = plan.get("stage", status.get("stage", directory.parent.name))
    is_block = stage == "block" or any("variants" in r["measurement"] and "variant" not in r["case"]
                                       for r in records)
    ok = block_eligible if is_block else eligible
    failures = [{"case_id": r["case"]["case_id"], "status": r["measurement"].get("status"),
                 "error": r["measurement"].get("error")}
                for r in records if not ok(r["measurement"])]
    requested = [r for r in records if r["case"].get("include_flex")]
    planned = len(plan["cases"]) if "cases" in plan else status.get("planned_cases")
    environments = {json.dumps({n: r["measurement"].get(n)
                                for n in ("hardware", "software", "timing_scope")}, sort_keys=True)
                    for r in records}
    return {"directory": str(directory), "stage": stage,
            "status": status.get("status", "not_recorded"), "planned_cases": planned,
            "recorded_cases": len(records),
            "not_recorded_cases": max(0, planned - len(records)) if isinstance(planned, int) else None,
            "passed_cases": len(records) - len(failures), "failed_cases": len(failures),
            "failures": failures, "flex_requested": len(requested),
            "flex_failed_or_unavailable": sum(not eligible(r["measurement"].get("flex", {}))
                                              for r in requested),
            "environments": [json.loads(value) for value in sorted(environments)],
            "source_sha256": status.get("source_sha256"),
            "evidence_files_sha256": {p.name: hashlib.sha256(p.read_bytes()).hexdigest()
                                      for p in paths},
            "ablations": comparisons(records) if stage == "ablation" else [],
            "confirmation": comparisons(records, confirmation=True)
            if stage == "confirmation" else [],
            "baselines": [] if is_block else baselines(records, directory),
            "block_comparisons": block_comparisons(records) if is_block else [],
            "setup_observations": [] if is_block else setup_observations(records),
            "tuning": tuning(records) if stage == "tuning" else [],
            "search_replay": replay_summary(directory)}


def analyze(root) -> dict:
    root = Path(root).resolve()
    directories = {path.parent for path in root.rglob("cases") if path.is_dir()}
    if root.name == "cases":
        directories.add(root.parent)
    if not directories:
        raise ValueError(f"No cases directories found in {root}")
    return {"schema_version": 1, "input": str(root),
            "scope": ("Forward CUDA-graph replay timings unless a recorded environment says "
                      "otherwise; attention microbenchmarks and single-block studies are reported "
                      "separately. Ratios above one favour the denominator; geometric means weight "
                      "each paired workload and input seed equally. No best-only filtering and no "
                      "pooling across runs or across default and hinted baselines."),
            "studies": [analyze_directory(path) for path in sorted(directories)]}


def fmt(value) -> str:
    return "-" if value is None else f"{value:.4g}"


def _ratio_row(name: str, item: dict, tail: str) -> str:
    return (f"| {name} | {item['paired_cases']} | {fmt(item['geomean_speedup'])}x | "
            f"{fmt(item['min_speedup'])}-{fmt(item['max_speedup'])}x | {item['regressions']} | "
            f"{tail} |")


def markdown(summary: dict) -> str:
    lines = ["# Attention experiment report", "", summary["scope"], ""]
    for study in summary["studies"]:
        lines += [f"## {study['stage']}: {study['directory']}", "",
                  f"Status: {study['status']}. Recorded {study['recorded_cases']} of "
                  f"{study['planned_cases']} planned cases; passed {study['passed_cases']}, failed "
                  f"{study['failed_cases']}. Flex baseline failed or unavailable in "
                  f"{study['flex_failed_or_unavailable']} of {study['flex_requested']} requests.", ""]
        for label in ("ablations", "confirmation"):
            if study[label]:
                lines += [f"### {label.capitalize()}", "",
                          "| Ratio | Pairs | Geomean | Range | Regressions | Missing / failed / "
                          "ambiguous / incompatible |", "|---|---:|---:|---:|---:|---:|"]
                for item in study[label]:
                    lines.append(_ratio_row(item["comparison"], item, " / ".join(
                        str(item[k]) for k in ("missing_counterpart_groups", "failed_groups",
                                               "ambiguous_groups",
                                               "incompatible_environment_groups"))))
                lines.append("")
        if study["block_comparisons"]:
            lines += ["### One block and isolated attention", "",
                      "| Baseline / scope | Pairs | Geomean | Range | Regressions | Failed or "
                      "unavailable |", "|---|---:|---:|---:|---:|---:|"]
            for item in study["block_comparisons"]:
                lines.append(_ratio_row(f"{item['baseline']} / {item['scope']}", item,
                                        str(item["failed_or_unavailable"])))
            lines.append("")
        if study["baselines"]:
            lines += ["### External baselines", "",
                      "| Candidate vs baseline | Pairs | Geomean | Range | Regressions | "
                      "Unavailable / candidate failed |", "|---|---:|---:|---:|---:|---:|"]
            for item in study["baselines"]:
                name = f"{item['candidate']} vs {item['baseline']} ({item['baseline_variant']})"
                lines.append(_ratio_row(name, item,
                                        f"{item['baseline_unavailable']} / {item['candidate_failed']}"))
            lines.append("")
        if study["setup_observations"]:
            lines += ["### First-call observations", "",
                      "| Variant | First call median (ms) | Range (ms) |", "|---|---:|---:|"]
            for item in study["setup_observations"]:
                first = item["statistics_ms"]["first_call_ms"]
                lines.append(f"| {item['variant']} | {fmt(first['median'])} | "
                             f"{fmt(first['min'])}-{fmt(first['max'])} |")
            lines.append("")
        for workload in study["tuning"]:
            rows = workload["rows_by_latency"]
            span = (f"latency {fmt(rows[0]['latency_ms'])}-{fmt(rows[-1]['latency_ms'])} ms; "
                    if rows else "")
            lines.append(f"- {workload['workload_id']}: {len(rows)} valid, "
                         f"{len(workload['failed_configurations'])} failed; {span}" + "; ".join(
                             f"{name} rho={fmt(v['spearman_rho'])} (n={v['samples']})"
                             for name, v in workload["associations"].items()))
        if study["tuning"]:
            lines.append("")
        replay = study.get("search_replay")
        if replay:
            lines += ["### Offline search replay", "", replay.get("methodology") or "", "",
                      "| Method | Budget | Trials | Failed | Mean regret | Median regret |",
                      "|---|---:|---:|---:|---:|---:|"]
            for item in replay["groups"]:
                lines.append(f"| {item['method']} | {item['budget']} | {item['trials']} | "
                             f"{item['failed_trials']} | {fmt(item['mean_relative_regret'])} | "
                             f"{fmt(item['median_relative_regret'])} |")
            lines.append("")
        if study["failures"]:
            lines += ["### Failures", ""]
            lines += [f"- {item['case_id']}: "
                      + str(item.get("error") or item["status"]).replace("\n", " ")
                      for item in study["failures"]]
            lines.append("")
    return "\n".join(lines) + "\n"


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--input", type=Path, required=True)
    parser.add_argument("--output-dir", type=Path, required=True)
    args = parser.parse_args(argv)
    summary = analyze(args.input)
    args.output_dir.mkdir(parents=True, exist_ok=True)
    (args.output_dir / "SUMMARY.json").write_text(json.dumps(summary, indent=2, allow_nan=False)
                                                  + "\n")
    (args.output_dir / "REPORT.md").write_text(markdown(summary))
    print(json.dumps({"studies": len(summary["studies"]), "output_dir": str(args.output_dir)}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
