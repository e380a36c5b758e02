"""Plan and execute matched-batch distributed comparisons on one GPU host.

Equivalent of the reference's planner (distributed/run_experiments.py:19-351):
the same model table and the same four stages - ``smoke`` (10 cases), ``screen``
(20), ``scale`` (38) and ``confirmation`` (21) - in a recorded shuffled order
(seed 336) with a plan hash; ``validate_plan`` checks every layout;
``case_config`` / ``command_for`` turn a case into a config file and a
``torch.distributed.run`` command line for ``llmdist.train``; ``run_plan`` runs
cases sequentially as process groups with per-case timeouts, classifies OOM from
the log tail, verifies each finished case against the plan (``inspect_case``),
checks that policies of one (model, context, seed, precision) group saw the same
source, initialisation, data and batch stream, stops at the first failure
(later cases are recorded ``not_run``; there is no retry) and keeps
``aggregate.json`` current; ``add_scaling_metrics`` attaches speed-up and
strong-scaling efficiency against the matched single-GPU case.

Launch differs in one detail: rendezvous uses an explicit ``--master-addr
127.0.0.1`` and a per-case port instead of ``--standalone``, because the container
host name need not resolve.
"""

from __future__ import annotations

import argparse
import hashlib
import json
import math
import random
import re
import signal
import subprocess
import sys
import time
from copy import deepcopy
from pathlib import Path

from . import common

MODELS = {
    "tiny": {"vocab_size": 128, "d_model": 64, "num_layers": 2, "num_heads": 4, "d_ff": 128},
    "100m": {"vocab_size": 10000, "d_model": 768, "num_layers": 12, "num_heads": 12, "d_ff": 2048},
    "324m": {"vocab_size": 10000, "d_model": 1024, "num_layers": 24, "num_heads": 16, "d_ff": 2752},
}
MODES = ("single", "naive", "ddp", "zero1", "fsdp", "tp")
ORDER_SEED = 336
STAGES = ("smoke", "screen", "scale", "confirmation")


def plan_hash(plan: dict) -> str:
    body = {k: v for k, v in plan.items() if k != "plan_sha256"}
    return hashlib.sha256(json.dumps(body, sort_keys=True).encode()).hexdigest()


def _case(mode, world, *, model="324m", context=1024, global_batch=32, microbatch=4,
          checkpointing="none", sync="last", bucket=25, seed=1337, steps=60,
          precision="bf16") -> dict:
    case_id = (f"{model}-s{context}-{mode}-w{world}-mb{microbatch}-{checkpointing}-{sync}"
               f"-b{bucket}-{precision}-seed{seed}")
    tiny = model == "tiny"
    return {"case_id": case_id, "mode": mode, "world_size": world, "model": model,
            "context_length": context, "global_batch_size": global_batch,
            "microbatch_size": microbatch, "checkpointing": checkpointing, "sync_policy": sync,
            "bucket_cap_mb": bucket, "seed": seed, "steps": steps, "precision": precision,
            "warmup_steps": 1 if tiny else 5, "timeout_seconds": 120 if tiny else 240}


def _world_for(mode: str, many: int) -> int:
    return 1 if mode == "single" else many


def _stage_cases(stage: str) -> list[dict]:
    cases = []
    if stage == "smoke":
        tiny = dict(model="tiny", context=32, global_batch=8, microbatch=2, steps=5)
        cases += [_case(m, _world_for(m, 2), precision="fp32", **tiny) for m in MODES]
        cases += [_case(m, _world_for(m, 2), checkpointing="block", precision="bf16", **tiny)
                  for m in ("single", "ddp", "zero1", "tp")]
    elif stage == "screen":
        for model in ("100m", "324m"):
            for ckpt in ("none", "block"):
                cases += [_case(m, _world_for(m, 2), model=model, global_batch=8,
                                checkpointing=ckpt, steps=30)
                          for m in ("single", "ddp", "zero1", "fsdp", "tp")]
    elif stage == "scale":
        for ckpt in ("none", "block"):
            cases.append(_case("single", 1, checkpointing=ckpt))
            cases += [_case(m, w, checkpointing=ckpt) for m in ("ddp", "zero1", "fsdp", "tp")
                      for w in (2, 4, 8)]
        cases.append(_case("naive", 8))
        cases.append(_case("ddp", 8, microbatch=1))
        cases.append(_case("ddp", 8, microbatch=1, sync="every"))
        cases += [_case("ddp", 8, microbatch=1, bucket=b) for b in (1, 100)]
        long = dict(context=4096, global_batch=8, microbatch=1)
        for ckpt in ("none", "block"):
            cases += [_case(m, _world_for(m, 8), checkpointing=ckpt, **long)
                      for m in ("single", "ddp")]
        cases += [_case(m, 8, checkpointing="block", **long) for m in ("zero1", "fsdp", "tp")]
    elif stage == "confirmation":
        for seed in (2027, 2028, 2029):
            cases += [_case(m, _world_for(m, 8), seed=seed)
                      for m in ("single", "ddp", "zero1", "fsdp", "tp")]
            cases += [_case(m, 8, checkpointing="block", seed=seed) for m in ("ddp", "fsdp")]
    else:
        raise ValueError(f"Unknown stage: {stage}")
    return cases


def build_plan(stage: str) -> dict:
    cases = _stage_cases(stage)
    random.Random(ORDER_SEED).shuffle(cases)     # order is fixed before anything runs
    plan = {
        "format_version": 1, "stage": stage, "cases": cases, "case_count": len(cases),
        "required_gpus": max(case["world_size"] for case in cases), "order_seed": ORDER_SEED,
        "comparability": ("Same model/context/seed has identical global batch, optimizer schedule, "
                          "validation windows and ordered examples; rank-local microbatch and "
                          "parallelism differ"),
        "cost_scope": ("Active GPU-seconds describe algorithmic resource use; all allocated GPUs "
                       "remain occupied during lower-world-size baselines"),
        "interpretation": ("Fixed-global-batch strong scaling; short screens do not establish time "
                           "to convergence or a quality-equivalence claim"),
        "failure_policy": ("Preserve the first failure and stop; subsequent cases remain not_run. "
                           "No automatic retry."),
    }
    validate_plan(plan)
    plan["plan_sha256"] = plan_hash(plan)
    return plan


def validate_plan(plan: dict) -> None:
    if plan.get("plan_sha256") and plan["plan_sha256"] != plan_hash(plan):
        raise ValueError("Distributed plan hash mismatch")
    cases = plan["cases"]
    if not cases or len({case["case_id"] for case in cases}) != len(cases):
        raise ValueError("Plan must have distinct nonempty cases")
    layouts = {}
    for case in cases:
        if not re.fullmatch(r"[A-Za-z0-9_-]+", case["case_id"]):
            raise ValueError("Case identifier must be safe and nonempty")
        world, batch, micro = case["world_size"], case["global_batch_size"], case["microbatch_size"]
        if any(type(n) is not int for n in (world, batch, micro)) or world not in (1, 2, 4, 8) \
                or batch <= 0 or micro <= 0:
            raise ValueError("Invalid rank or batch layout")
        mode = case["mode"]
        if mode not in MODES:
            raise ValueError("Unknown parallelism mode")
        if (mode == "single") != (world == 1):
            raise ValueError("Single mode and one-rank layout must coincide")
        if batch % (micro * (1 if mode == "tp" else world)):
            raise ValueError("Global batch must divide across ranks and microbatches")
        model = MODELS[case["model"]]
        if mode == "tp" and (model["num_heads"] % world or model["d_ff"] % world):
            raise ValueError("TP requires divisible attention heads and feed-forward width")
        if case["sync_policy"] not in ("last", "every") or (
                case["sync_policy"] == "every" and mode not in ("ddp", "zero1")):
            raise ValueError("Invalid synchronization policy")
        if case["checkpointing"] not in ("none", "block") or case["precision"] not in ("fp32", "bf16"):
            raise ValueError("Invalid checkpointing or precision policy")
        if not math.isfinite(case["bucket_cap_mb"]) or case["bucket_cap_mb"] <= 0:
            raise ValueError("Bucket capacity must be positive and finite")
        if type(case["context_length"]) is not int or case["context_length"] <= 0 \
                or case["timeout_seconds"] <= 0:
            raise ValueError("Invalid context or timeout")
        if not 0 <= case["warmup_steps"] < case["steps"]:
            raise ValueError("Invalid timing warmup")
        group = (case["model"], case["context_length"], case["seed"], case["precision"])
        layout = (batch, case["steps"], case["warmup_steps"])
        if layouts.setdefault(group, layout) != layout:
            raise ValueError("Comparable policies must share global batch, steps and timing warmup")
    if plan["case_count"] != len(cases) \
            or plan["required_gpus"] != max(case["world_size"] for case in cases):
        raise ValueError("Plan case or GPU count mismatch")


def case_config(base: dict, case: dict, device: str = "cuda") -> dict:
    config = deepcopy(base)
    config["model"].update(MODELS[case["model"]])
    config["model"].update(context_length=case["context_length"], attention_backend="sdpa",
                           activation_checkpointing=case["checkpointing"])
    steps = case["steps"]
    config.update(seed=case["seed"], device=device, precision=case["precision"], num_threads=2,
                  batch_size=case["global_batch_size"], grad_accum_steps=1, max_steps=steps,
                  warmup_steps=min(5, steps - 1), eval_interval=steps, eval_batches=8,
                  eval_batch_size=1, checkpoint_interval=steps)
    if case["model"] == "tiny":
        config["data"] = {"kind": "synthetic", "synthetic_tokens": 4096}
    return config


def command_for(case: dict, config_path, destination, device: str = "cuda",
                port: int = 29700) -> list[str]:
    command = [sys.executable]
    if case["world_size"] > 1:
        command += ["-m", "torch.distributed.run", "--nnodes=1",
                    f"--nproc-per-node={case['world_size']}", "--master-addr", "127.0.0.1",
                    "--master-port", str(port), "--max-restarts=0", "--module", "llmdist.train"]
    else:
        command += ["-m", "llmdist.train"]
    command += ["--config", str(config_path), "--output-dir", str(destination), "--mode",
                case["mode"], "--global-batch-size", str(case["global_batch_size"]),
                "--microbatch-size", str(case["microbatch_size"]), "--warmup-steps",
                str(case["warmup_steps"]), "--sync-policy", case["sync_policy"],
                "--bucket-cap-mb", str(case["bucket_cap_mb"]), "--device", device]
    return command


def _expect(condition: bool, message: str) -> None:
    if not condition:
        raise ValueError(message)


def inspect_case(path: Path, case: dict) -> tuple[dict, dict]:
    """Re-derives every claim of a finished case from its rank files."""
    path = Path(path)
    summary = common.read_json(path / "summary.json")
    _expect(summary["status"] == "completed" and summary["step"] == case["steps"],
            "Case did not complete all planned updates")
    tokens = case["global_batch_size"] * case["context_length"]
    expected_model = dict(MODELS[case["model"]], context_length=case["context_length"],
                          activation_checkpointing=case["checkpointing"], attention_backend="sdpa")
    shared = ("status", "mode", "world_size", "global_batch_size", "microbatch_size", "step",
              "tokens_seen", "tokens_per_step", "measured_steps", "batch_stream_sha256")
    metadata, streams, train = [], [], []
    for rank in range(case["world_size"]):
        meta = common.read_json(path / f"rank-{rank}-metadata.json")
        rows = common.read_jsonl(path / f"rank-{rank}-metrics.jsonl")
        rank_summary = common.read_json(path / f"rank-{rank}-summary.json")
        train = [row for row in rows if row["event"] == "train"]
        _expect([row["step"] for row in train] == list(range(1, case["steps"] + 1))
                and rank_summary["status"] == "completed",
                "Missing rank training updates or summary")
        for key in ("mode", "world_size", "global_batch_size", "microbatch_size", "sync_policy",
                    "bucket_cap_mb"):
            _expect(meta[key] == case[key], f"Executed layout differs from the plan: {key}")
        _expect(meta["rank"] == rank and meta["timing_warmup_steps"] == case["warmup_steps"]
                and meta["profile_steps"] == 0,
                "Executed rank, warmup or profiling differs from the plan")
        config = meta["config"]
        _expect(all(config["model"][k] == v for k, v in expected_model.items()),
                "Executed model or checkpointing differs from the plan")
        _expect(all(config[k] == case[k] for k in ("seed", "precision"))
                and config["max_steps"] == case["steps"],
                "Executed seed, precision or step horizon differs from the plan")
        _expect(all(row["tokens_seen"] == row["step"] * tokens for row in train),
                "Training token accounting differs from the plan")
        for row in train:
            finite = all(math.isfinite(row[k]) for k in ("loss", "gradient_norm", "step_seconds",
                                                         "learning_rate"))
            _expect(finite and row["step_seconds"] > 0,
                    "Nonfinite training metric or invalid step time")
        digest = hashlib.sha256("".join(row["batch_start_sha256"] for row in train).encode()).hexdigest()
        _expect(all(rank_summary[k] == summary[k] for k in shared)
                and digest == summary["batch_stream_sha256"],
                "Rank summary or batch-stream digest differs from actual metrics")
        streams.append([(row["batch_start_sha256"], row["learning_rate"], row["tokens_seen"])
                        for row in train])
        metadata.append(meta)
    for key in ("mode", "world_size", "global_batch_size", "microbatch_size", "sync_policy"):
        _expect(summary[key] == case[key], f"Summary differs from the plan: {key}")
    measured = [row["step_seconds"] for row in train if row["step"] > case["warmup_steps"]]
    _expect(summary["tokens_seen"] == case["steps"] * tokens and summary["tokens_per_step"] == tokens
            and summary["measured_steps"] == len(measured)
            and math.isclose(summary["measured_train_seconds"], sum(measured), rel_tol=1e-10)
            and math.isclose(summary["tokens_per_second"], len(measured) * tokens / sum(measured),
                             rel_tol=1e-10)
            and math.isfinite(summary["valid_loss"]),
            "Summary timing, token accounting or validation loss is invalid")
    _expect(all(stream == streams[0] for stream in streams),
            "Global batch or learning-rate stream differs across ranks")
    for key in ("data_identity", "source", "initial_parameter_sha256"):
        _expect(all(meta[key] == metadata[0][key] for meta in metadata),
                f"Rank provenance mismatch: {key}")
    signature = {key: metadata[0][key] for key in ("data_identity", "source",
                                                   "initial_parameter_sha256")}
    signature["batch_stream_sha256"] = summary["batch_stream_sha256"]
    signature["learning_rate_stream_sha256"] = hashlib.sha256(
        json.dumps(streams[0]).encode()).hexdigest()
    return summary, signature


def add_scaling_metrics(rows: list[dict], allocated_gpus: int) -> None:
    def key_of(row):
        return (row["model"], row["context_length"], row["seed"], row["precision"],
                row["checkpointing"])
    baselines = {key_of(r): r for r in rows if r["status"] == "completed" and r["mode"] == "single"}
    for row in rows:
        if "subprocess_seconds" in row:
            row["allocated_gpu_seconds_subprocess"] = allocated_gpus * row["subprocess_seconds"]
        if row["status"] != "completed":
            continue
        row["active_gpu_seconds_measured"] = row["world_size"] * row["measured_train_seconds"]
        baseline = baselines.get(key_of(row))
        if baseline:
            speedup = row["tokens_per_second"] / baseline["tokens_per_second"]
            row["throughput_speedup"] = speedup
            row["strong_scaling_efficiency"] = speedup / row["world_size"]
            row["baseline_case_id"] = baseline["case_id"]


def launch_case(command, log_path, timeout, env):
    """Runs one case; separated so tests can substitute it."""
    return common.run_case(command, log_path=log_path, timeout=timeout, cwd=common.REPO_ROOT,
                           env=env)


def run_plan(plan: dict, base: dict, output: Path, *, device: str = "cuda",
             allocated_gpus: int | None = None) -> dict:
    validate_plan(plan)
    allocated_gpus = plan["required_gpus"] if allocated_gpus is None else allocated_gpus
    if type(allocated_gpus) is not int or allocated_gpus < plan["required_gpus"]:
        raise ValueError("Allocated GPU count must cover all planned ranks")
    output = Path(output)
    output.mkdir(parents=True, exist_ok=False)
    for folder in ("configs", "cases", "logs"):
        (output / folder).mkdir()
    common.write_json(output / "plan.json", plan)
    rows: list[dict] = []
    signatures: dict = {}
    aggregate = {"status": "running", "planned_count": len(plan["cases"]), "cases": rows,
                 "plan_sha256": plan["plan_sha256"], "allocated_gpus": allocated_gpus}
    env = common.child_environment({"OMP_NUM_THREADS": "2", "TORCH_NCCL_ASYNC_ERROR_HANDLING": "1"})

    def on_terminate(signum, frame):
        raise TimeoutError("Outer job terminated; the active case was stopped")

    previous = signal.signal(signal.SIGTERM, on_terminate)
    try:
        for index, case in enumerate(plan["cases"]):
            row = dict(case, status="running")
            rows.append(row)
            common.write_json(output / "aggregate.json", aggregate)
            config_path = output / "configs" / f"{case['case_id']}.json"
            destination = output / "cases" / case["case_id"]
            common.write_json(config_path, case_config(base, case, device))
            log_path = output / "logs" / f"{case['case_id']}.log"
            print(f"[{index + 1}/{len(plan['cases'])}] {case['case_id']}", flush=True)
            started = time.monotonic()
            try:
                command = command_for(case, config_path, destination, device, port=29700 + index % 200)
                result = launch_case(command, log_path, case["timeout_seconds"], env)
                if result["status"] == "timeout":
                    row["status"] = "timeout"
                    raise TimeoutError("Distributed case exceeded its limit")
                if result["status"] != "completed":
                    row["status"] = "oom" if result.get("failure_kind") == "oom" else "failed"
                    raise RuntimeError(result.get("error", "worker failed"))
                summary, signature = inspect_case(destination, case)
                group = (case["model"], case["context_length"], case["seed"], case["precision"])
                if signatures.setdefault(group, signature) != signature:
                    raise ValueError(
                        "Cross-policy source, initialization, dataset or batch stream mismatch")
                row.update(summary, comparability="passed")
            except Exception as error:
                if row["status"] == "running":
                    row["status"] = "invalid"
                row["error"] = str(error)
                rows.extend(dict(later, status="not_run") for later in plan["cases"][index + 1:])
            finally:
                row["subprocess_seconds"] = time.monotonic() - started
                add_scaling_metrics(rows, allocated_gpus)
                done = len(rows) == len(plan["cases"]) and all(r["status"] == "completed"
                                                               for r in rows)
                aggregate["status"] = "completed" if done else "running"
                if row["status"] != "completed":
                    aggregate["status"] = "failed"
                common.write_json(output / "aggregate.json", aggregate)
            if row["status"] != "completed":
                break
    finally:
        signal.signal(signal.SIGTERM, previous)
    return aggregate


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--stage", choices=STAGES, default="smoke")
    parser.add_argument("--plan", type=Path)
    parser.add_argument("--config", type=Path, required=True)
    parser.add_argument("--output-dir", type=Path, required=True)
    parser.add_argument("--device", choices=["cuda", "cpu"], default="cuda")
    parser.add_argument("--allocated-gpus", type=int)
    parser.add_argument("--execute", action="store_true")
    args = parser.parse_args()
    plan = common.read_json(args.plan) if args.plan else build_plan(args.stage)
    validate_plan(plan)
    if not args.execute:
        print(json.dumps(plan, indent=2))
        return
    result = run_plan(plan, common.read_json(args.config), args.output_dir, device=args.device,
                      allocated_gpus=args.allocated_gpus)
    print(json.dumps({"status": result["status"], "cases": len(result["cases"])}, indent=2))
    if result["status"] != "completed":
        raise SystemExit(1)


if __name__ == "__main__":
    main()
