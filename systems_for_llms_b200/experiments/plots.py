"""Bar and curve plots from pilot aggregates and run evidence (matplotlib, Agg).

Counterpart of the reference's plot scripts (scripts/plot_pilot.py,
scripts/plot_quality.py): ``plot_pilot`` draws throughput and peak allocated
memory per policy from ``aggregate.json``; ``plot_quality`` draws validation loss
against training seconds for every run of a quality job and marks the frozen
target.  matplotlib is optional; without it the functions raise ``ImportError``
when called, importing this module never fails.
"""

from __future__ import annotations

import argparse
from pathlib import Path

from . import common


def _pyplot():
    import matplotlib
    matplotlib.use("Agg")
    import matplotlib.pyplot as plt
    return plt


def pilot_series(aggregate: dict) -> list[dict]:
    """Rows for plotting: label, throughput, peak GiB (completed cases only)."""
    rows = []
    for row in aggregate["cases"]:
        if row["status"] != "completed":
            continue
        label = (f"{row['attention_backend']}/{row['activation_checkpointing']}/"
                 f"mb{row['batch_size']}/s{row['seed']}")
        peak = row.get("peak_cuda_allocated_bytes")
        rows.append({"label": label, "tokens_per_second": row["tokens_per_second"],
                     "peak_gib": None if peak is None else peak / 2 ** 30})
    return sorted(rows, key=lambda r: r["label"])


def plot_pilot(aggregate_path: Path, output: Path) -> Path:
    plt = _pyplot()
    rows = pilot_series(common.read_json(aggregate_path))
    figure, (left, right) = plt.subplots(1, 2, figsize=(11, 4))
    labels = [r["label"] for r in rows]
    left.barh(labels, [r["tokens_per_second"] for r in rows])
    left.set_xlabel("tokens / s")
    right.barh(labels, [r["peak_gib"] or 0 for r in rows])
    right.set_xlabel("peak allocated GiB")
    right.set_yticklabels([])
    figure.tight_layout()
    figure.savefig(output, dpi=150)
    plt.close(figure)
    return output


def quality_curves(job_root: Path) -> dict[str, list[tuple[float, float]]]:
    """case id -> [(training seconds, validation loss)] from each run's metrics."""
    curves = {}
    for run in sorted((Path(job_root) / "runs").iterdir()):
        seconds, points = {}, []
        for event in common.read_jsonl(run / "metrics.jsonl"):
            if event["event"] == "train":
                seconds[event["step"]] = event["train_seconds"]
            elif event["event"] == "eval":
                points.append((seconds.get(event["step"], 0.0), event["valid_loss"]))
        curves[run.name] = points
    return curves


def plot_quality(job_root: Path, output: Path, target: float | None = None) -> Path:
    plt = _pyplot()
    figure, axis = plt.subplots(figsize=(7, 4.5))
    for name, points in quality_curves(job_root).items():
        axis.plot([p[0] for p in points], [p[1] for p in points], label=name, linewidth=1)
    if target is not None:
        axis.axhline(target, color="black", linestyle="--", linewidth=0.8, label=f"target {target}")
    axis.set_xlabel("training seconds")
    axis.set_ylabel("validation loss")
    axis.legend(fontsize=6)
    figure.tight_layout()
    figure.savefig(output, dpi=150)
    plt.close(figure)
    return output


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    sub = parser.add_subparsers(dest="command", required=True)
    a = sub.add_parser("pilot")
    a.add_argument("--aggregate", type=Path, required=True)
    a.add_argument("--output", type=Path, required=True)
    b = sub.add_parser("quality")
    b.add_argument("--job-root", type=Path, required=True)
    b.add_argument("--output", type=Path, required=True)
    b.add_argument("--target", type=float)
    args = parser.parse_args()
    if args.command == "pilot":
        print(plot_pilot(args.aggregate, args.output))
    else:
        print(plot_quality(args.job_root, args.output, args.target))


if __name__ == "__main__":
    main()
