"""Four-panel figure of recorded attention experiments; reads evidence files only.

Panels, after the reference's figure (attention_lab/plot_results.py:115-282):
lowering ablations per workload, tuning spread (every configuration's latency
relative to the workload's best), block-level and isolated-attention ratios, and
the default against the contiguity-hinted FlexAttention baseline.  The series
behind each panel come from ``analyze_study.analyze_directory`` and are
available without matplotlib (``ablation_series`` and friends); only
``make_figure`` needs it.  Whiskers are observed ranges over input seeds, not
confidence intervals, and failed or missing cases are counted in the caption,
never drawn as if measured.
"""

from __future__ import annotations

import argparse
import json
import math
import re
import statistics
from collections import defaultdict
from pathlib import Path

from .analyze_study import analyze_directory, positive

COLORS = ("#2369A8", "#D77A26", "#24977F", "#9467A8", "#C45763")
_WORKLOAD = re.compile(r"n(\d+)-d(\d+)-(\w+)")


def grouped_ratios(pairs: list[dict], key: str = "workload_id") -> dict:
    """Geometric mean and observed range of the valid ratios per group."""
    grouped = defaultdict(list)
    for pair in pairs:
        if positive(pair.get("ratio")):
            grouped[pair[key]].append(pair["ratio"])
    return {name: {"mean": math.exp(statistics.mean(math.log(v) for v in values)),
                   "low": min(values), "high": max(values), "count": len(values)}
            for name, values in grouped.items()}


def workload_order(name: str):
    match = _WORKLOAD.search(name)
    return (int(match[1]), int(match[2]), match[3]) if match else (0, 0, name)


def workload_label(name: str) -> str:
    match = _WORKLOAD.search(name)
    if not match:
        return name.replace("tune-", "").replace("window", "window ")
    length = int(match[1])
    size = f"{length // 1024}K" if length % 1024 == 0 else str(length)
    return f"{size} / D{match[2]} / {'window 128' if match[3] == 'window' else match[3]}"


def load_studies(root) -> list[dict]:
    root = Path(root).resolve()
    directories = {path.parent for path in root.rglob("cases") if path.is_dir()}
    studies = []
    for directory in sorted(directories):
        paths = sorted((directory / "cases").glob("*.json"))
        if not paths:
            continue
        relative = directory.relative_to(root) if directory != root else Path(directory.name)
        run = relative.parent if relative.name == "study" else relative
        studies.append({"run": str(run), "directory": directory,
                        "records": [json.loads(p.read_text()) for p in paths],
                        "report": analyze_directory(directory)})
    return studies


def ablation_series(studies) -> dict:
    """comparison -> {workload -> mean/low/high/count} over all ablation runs."""
    series = {}
    for item in (i for s in studies for i in s["report"]["ablations"]):
        series.setdefault(item["comparison"], {}).update(grouped_ratios(item["pairs"]))
    return series


def tuning_series(studies) -> dict:
    """workload -> sorted latencies relative to that workload's fastest configuration."""
    series = {}
    for workload in (w for s in studies for w in s["report"]["tuning"]):
        rows = workload["rows_by_latency"]
        if rows:
            best = rows[0]["latency_ms"]
            series[workload["workload_id"]] = [row["latency_ms"] / best for row in rows]
    return series


def block_series(studies) -> dict:
    """(baseline, scope) -> {case label -> ratio}."""
    series = {}
    for item in (i for s in studies for i in s["report"]["block_comparisons"]):
        target = series.setdefault((item["baseline"], item["scope"]), {})
        for pair in item["pairs"]:
            if positive(pair.get("ratio")):
                target[f"n{pair['length']}-d{pair['dim']}-{pair['pattern']}"] = pair["ratio"]
    return series


def hint_series(studies) -> dict:
    """Flex baseline variant (default / contiguous_blocks) -> {workload -> stats}."""
    series = {}
    for item in (i for s in studies for i in s["report"]["baselines"]):
        if item["baseline"] == "flex" and item["candidate"].startswith("interval_split"):
            series.setdefault(item["baseline_variant"], {}).update(grouped_ratios(item["pairs"]))
    return series


def _bars(axis, title, groups: dict, xlabel: str) -> None:
    """Horizontal grouped bars with range whiskers; one colour per series."""
    names = sorted({w for g in groups.values() for w in g}, key=workload_order)
    if not names:
        axis.set_title(title, loc="left")
        axis.text(0.5, 0.5, "No valid measurements available", ha="center", va="center",
                  transform=axis.transAxes, color="#657180")
        axis.set_xticks([])
        axis.set_yticks([])
        return
    height = 0.8 / max(1, len(groups))
    for index, (label, stats) in enumerate(groups.items()):
        rows = [(i, stats[name]) for i, name in enumerate(names) if name in stats]
        positions = [i + index * height for i, _ in rows]
        means = [s["mean"] if isinstance(s, dict) else s for _, s in rows]
        axis.barh(positions, means, height=height * 0.9, color=COLORS[index % len(COLORS)],
                  label=str(label))
        for position, (_, s) in zip(positions, rows):
            if isinstance(s, dict):
                axis.plot([s["low"], s["high"]], [position, position], color="#243246", lw=1)
    axis.axvline(1.0, color="#657180", lw=1, ls="--")
    axis.set_yticks([i + 0.4 - height / 2 for i in range(len(names))])
    axis.set_yticklabels([workload_label(n) for n in names])
    axis.invert_yaxis()
    axis.set_xlabel(xlabel)
    axis.set_title(title, loc="left")
    axis.legend(fontsize=7, frameon=False)


def make_figure(root, output) -> dict:
    import matplotlib
    matplotlib.use("Agg")
    import matplotlib.pyplot as plt

    studies = load_studies(root)
    figure, axes = plt.subplots(2, 2, figsize=(16, 11))
    _bars(axes[0, 0], "Lowering ablations", ablation_series(studies),
          "left variant latency / right variant latency")
    tuning = tuning_series(studies)
    axis = axes[0, 1]
    for index, (workload, ratios) in enumerate(sorted(tuning.items())):
        axis.plot(range(len(ratios)), ratios, marker="o", ms=3, color=COLORS[index % len(COLORS)],
                  label=workload_label(workload))
    axis.set_title("Tuning: latency relative to the best configuration", loc="left")
    axis.set_xlabel("configuration rank")
    if tuning:
        axis.legend(fontsize=7, frameon=False)
    _bars(axes[1, 0], "One block and isolated attention",
          {f"{b} / {s}": v for (b, s), v in block_series(studies).items()},
          "baseline latency / this kernel's latency")
    _bars(axes[1, 1], "FlexAttention with and without the contiguity hint", hint_series(studies),
          "Flex latency / interval kernel latency")
    total = sum(s["report"]["recorded_cases"] for s in studies)
    failed = sum(s["report"]["failed_cases"] for s in studies)
    figure.suptitle("Attention specialisation: measured trade-offs", x=0.055, ha="left",
                    fontsize=18, fontweight="bold")
    figure.text(0.055, 0.02, f"Ratios above 1 favour this package's kernel. {total} recorded "
                f"cases, {failed} failed. Whiskers are observed seed ranges.", fontsize=9,
                color="#657180")
    figure.subplots_adjust(left=0.14, right=0.98, bottom=0.09, top=0.9, wspace=0.43, hspace=0.4)
    output = Path(output)
    output.parent.mkdir(parents=True, exist_ok=True)
    figure.savefig(output, dpi=180, facecolor="white")
    plt.close(figure)
    return {"output": str(output.resolve()), "study_runs": len(studies), "recorded_cases": total,
            "failed_cases": failed}


def main(argv=None) -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--input", type=Path, required=True)
    parser.add_argument("--output", type=Path, required=True)
    args = parser.parse_args(argv)
    if args.output.suffix.lower() != ".png":
        parser.error("--output must name a .png file")
    print(json.dumps(make_figure(args.input, args.output)))


if __name__ == "__main__":
    main()
