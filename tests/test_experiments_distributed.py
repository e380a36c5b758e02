"""Distributed experiment planner: plans, commands, case inspection, the plan runner.

One real single-rank CPU run (module fixture) gives genuine rank files for
``inspect_case``; everything that concerns failure handling replaces the subprocess
launcher, including the time-out, which is injected with a tiny limit.
"""

import copy
import json
import sys
from pathlib import Path

import pytest

from systems_for_llms_b200.experiments import common
from systems_for_llms_b200.experiments import distributed_plan as planner

BASE_CONFIG = json.loads((Path(__file__).resolve().parents[1] / "configs" / "smoke.json").read_text())


def tiny_case(mode="single", world=1, **changes):
    options = dict(model="tiny", context=32, global_batch=8, microbatch=2, steps=4,
                   precision="fp32")
    options.update(changes)
    return planner._case(mode, world, **options)


def sealed(cases):
    plan = {"format_version": 1, "stage": "custom", "cases": cases, "case_count": len(cases),
            "required_gpus": max(case["world_size"] for case in cases),
            "order_seed": planner.ORDER_SEED}
    plan["plan_sha256"] = planner.plan_hash(plan)
    return plan


# --------------------------------------------------------------------- plans --
@pytest.mark.parametrize("stage, count, gpus", [("smoke", 10, 2), ("screen", 20, 2),
                                                ("scale", 38, 8), ("confirmation", 21, 8)])
def test_stage_sizes_and_determinism(stage, count, gpus):
    plan = planner.build_plan(stage)
    assert plan["case_count"] == count == len(plan["cases"])
    assert plan["required_gpus"] == gpus
    assert plan == planner.build_plan(stage)
    assert plan["plan_sha256"] == planner.plan_hash(plan)
    planner.validate_plan(plan)
    ordered = sorted(plan["cases"], key=lambda case: case["case_id"])
    assert ordered != plan["cases"]          # shuffled, and the order is part of the hash


def test_scale_stage_has_the_long_context_and_bucket_cases():
    cases = {case["case_id"]: case for case in planner.build_plan("scale")["cases"]}
    assert "324m-s4096-tp-w8-mb1-block-last-b25-bf16-seed1337" in cases
    assert "324m-s1024-ddp-w8-mb1-none-every-b25-bf16-seed1337" in cases
    assert {cases[c]["bucket_cap_mb"] for c in cases if "-mb1-none-last-" in c
            and "-s1024-ddp-w8" in c} == {1, 25, 100}
    long = [case for case in cases.values() if case["context_length"] == 4096]
    assert all(case["global_batch_size"] == 8 and case["microbatch_size"] == 1 for case in long)


def test_unknown_stage():
    with pytest.raises(ValueError, match="Unknown stage"):
        planner.build_plan("production")


@pytest.mark.parametrize("edit, message", [
    (lambda c: c.update(world_size=3), "rank or batch layout"),
    (lambda c: c.update(mode="pipeline"), "Unknown parallelism"),
    (lambda c: c.update(mode="ddp"), "must coincide"),
    (lambda c: c.update(microbatch_size=3), "divide across ranks"),
    (lambda c: c.update(sync_policy="every"), "synchronization policy"),
    (lambda c: c.update(checkpointing="full"), "checkpointing or precision"),
    (lambda c: c.update(bucket_cap_mb=0), "Bucket capacity"),
    (lambda c: c.update(warmup_steps=4), "timing warmup"),
    (lambda c: c.update(case_id="../escape"), "safe and nonempty"),
    (lambda c: c.update(timeout_seconds=0), "context or timeout"),
])
def test_validate_plan_rejects(edit, message):
    case = tiny_case()
    edit(case)
    plan = sealed([case])
    with pytest.raises(ValueError, match=message):
        planner.validate_plan(plan)


def test_validate_plan_checks_hash_counts_and_group_layouts():
    plan = sealed([tiny_case()])
    plan["cases"][0]["steps"] = 5
    with pytest.raises(ValueError, match="hash mismatch"):
        planner.validate_plan(plan)
    plan = sealed([tiny_case(), tiny_case("ddp", 2, steps=6)])
    with pytest.raises(ValueError, match="share global batch"):
        planner.validate_plan(plan)
    plan = sealed([tiny_case("tp", 8)])
    with pytest.raises(ValueError, match="TP requires divisible"):
        planner.validate_plan(plan)
    plan = sealed([tiny_case()])
    plan["case_count"] = 2
    plan["plan_sha256"] = planner.plan_hash(plan)
    with pytest.raises(ValueError, match="count mismatch"):
        planner.validate_plan(plan)


def test_case_config_and_command():
    case = tiny_case("zero1", 2, checkpointing="block")
    config = planner.case_config(BASE_CONFIG, case, "cpu")
    assert config["model"]["d_model"] == 64 and config["model"]["context_length"] == 32
    assert config["model"]["attention_backend"] == "sdpa"
    assert config["model"]["activation_checkpointing"] == "block"
    assert (config["batch_size"], config["grad_accum_steps"], config["max_steps"]) == (8, 1, 4)
    assert config["eval_interval"] == config["checkpoint_interval"] == 4
    assert config["num_threads"] == 2 and config["eval_batches"] == 8
    assert config["data"] == {"kind": "synthetic", "synthetic_tokens": 4096}
    assert BASE_CONFIG["model"]["d_model"] != 64            # the base was not modified
    command = planner.command_for(case, "c.json", "out", "cpu", port=29777)
    assert command[:3] == [sys.executable, "-m", "torch.distributed.run"]
    assert "--nproc-per-node=2" in command and "--max-restarts=0" in command
    assert command[command.index("--master-addr") + 1] == "127.0.0.1"
    assert command[command.index("--master-port") + 1] == "29777"
    assert command[command.index("--module") + 1] == "llmdist.train"
    assert command[command.index("--mode") + 1] == "zero1"
    single = planner.command_for(tiny_case(), "c.json", "out", "cpu")
    assert single[:3] == [sys.executable, "-m", "llmdist.train"]
    assert "torch.distributed.run" not in single


# --------------------------------------------------- one real run, inspected --
@pytest.fixture(scope="module")
def real_run(tmp_path_factory):
    plan = sealed([tiny_case()])
    output = tmp_path_factory.mktemp("dist") / "run"
    aggregate = planner.run_plan(plan, copy.deepcopy(BASE_CONFIG), output, device="cpu")
    return plan, output, aggregate


def test_real_single_rank_run_passes_inspection(real_run):
    plan, output, aggregate = real_run
    assert aggregate["status"] == "completed", aggregate["cases"][0].get("error")
    row = aggregate["cases"][0]
    assert row["comparability"] == "passed" and row["tokens_per_step"] == 8 * 32
    assert row["active_gpu_seconds_measured"] == pytest.approx(row["measured_train_seconds"])
    assert row["throughput_speedup"] == pytest.approx(1.0)
    assert row["strong_scaling_efficiency"] == pytest.approx(1.0)
    assert json.loads((output / "plan.json").read_text()) == plan
    summary, signature = planner.inspect_case(output / "cases" / plan["cases"][0]["case_id"],
                                              plan["cases"][0])
    assert set(signature) == {"data_identity", "source", "initial_parameter_sha256",
                              "batch_stream_sha256", "learning_rate_stream_sha256"}
    with pytest.raises(FileExistsError):
        planner.run_plan(plan, copy.deepcopy(BASE_CONFIG), output, device="cpu")


@pytest.mark.parametrize("tamper, message", [
    ("drop_row", "Missing rank training updates"),
    ("tokens", "token accounting"),
    ("throughput", "Summary timing"),
    ("layout", "Executed layout differs"),
    ("nan", "Nonfinite training metric"),
])
def test_inspection_rejects_tampered_evidence(real_run, tmp_path, tamper, message):
    import shutil
    plan, output, _ = real_run
    case = plan["cases"][0]
    copy_dir = tmp_path / "case"
    shutil.copytree(output / "cases" / case["case_id"], copy_dir)
    metrics = copy_dir / "rank-0-metrics.jsonl"
    rows = [json.loads(line) for line in metrics.read_text().splitlines()]
    if tamper == "drop_row":
        rows = [row for row in rows if not (row["event"] == "train" and row["step"] == 2)]
    elif tamper == "tokens":
        next(row for row in rows if row["event"] == "train")["tokens_seen"] += 1
    elif tamper == "nan":
        next(row for row in rows if row["event"] == "train")["loss"] = float("nan")
    metrics.write_text("".join(json.dumps(row) + "\n" for row in rows))
    if tamper == "throughput":
        for name in ("summary.json", "rank-0-summary.json"):
            document = json.loads((copy_dir / name).read_text())
            document["tokens_per_second"] *= 1.5
            (copy_dir / name).write_text(json.dumps(document))
    if tamper == "layout":
        document = json.loads((copy_dir / "rank-0-metadata.json").read_text())
        document["microbatch_size"] = 4
        (copy_dir / "rank-0-metadata.json").write_text(json.dumps(document))
    with pytest.raises(ValueError, match=message):
        planner.inspect_case(copy_dir, case)


# ------------------------------------------------------------ plan execution --
def test_timeout_stops_the_plan_and_later_cases_are_not_run(tmp_path):
    slow = tiny_case()
    slow["timeout_seconds"] = 0.001                        # the real launcher, a tiny limit
    plan = sealed([slow, tiny_case("ddp", 2), tiny_case("zero1", 2)])
    aggregate = planner.run_plan(plan, copy.deepcopy(BASE_CONFIG), tmp_path / "run", device="cpu")
    assert aggregate["status"] == "failed"
    assert [row["status"] for row in aggregate["cases"]] == ["timeout", "not_run", "not_run"]
    assert "exceeded" in aggregate["cases"][0]["error"]
    assert aggregate["cases"][0]["allocated_gpu_seconds_subprocess"] == pytest.approx(
        2 * aggregate["cases"][0]["subprocess_seconds"])
    assert json.loads((tmp_path / "run" / "aggregate.json").read_text())["status"] == "failed"


def test_oom_and_failures_are_classified_without_retry(tmp_path, monkeypatch):
    calls = []

    def launcher(command, log_path, timeout, env):
        calls.append(command)
        return {"status": "failed", "returncode": 1, "failure_kind": "oom",
                "error": "CUDA out of memory"}

    monkeypatch.setattr(planner, "launch_case", launcher)
    plan = sealed([tiny_case(), tiny_case("ddp", 2)])
    aggregate = planner.run_plan(plan, copy.deepcopy(BASE_CONFIG), tmp_path / "run", device="cpu")
    assert len(calls) == 1
    assert [row["status"] for row in aggregate["cases"]] == ["oom", "not_run"]
    assert calls[0][-1] == "cpu" and aggregate["allocated_gpus"] == 2


def test_cross_policy_signature_mismatch_is_invalid(tmp_path, monkeypatch):
    monkeypatch.setattr(planner, "launch_case", lambda *a, **k: {"status": "completed"})
    signatures = iter([{"source": "a"}, {"source": "b"}])
    summary = {"status": "completed", "tokens_per_second": 10.0, "measured_train_seconds": 1.0}
    monkeypatch.setattr(planner, "inspect_case",
                        lambda path, case: (dict(summary), next(signatures)))
    plan = sealed([tiny_case(), tiny_case("ddp", 2)])
    aggregate = planner.run_plan(plan, copy.deepcopy(BASE_CONFIG), tmp_path / "run", device="cpu")
    assert [row["status"] for row in aggregate["cases"]] == ["completed", "invalid"]
    assert "mismatch" in aggregate["cases"][1]["error"]


def test_run_plan_needs_enough_gpus(tmp_path):
    plan = sealed([tiny_case("ddp", 2)])
    with pytest.raises(ValueError, match="cover all planned ranks"):
        planner.run_plan(plan, copy.deepcopy(BASE_CONFIG), tmp_path / "run", allocated_gpus=1)


def test_scaling_metrics_use_the_matched_single_baseline():
    def row(mode, world, rate, ckpt="none", status="completed"):
        return {"case_id": f"{mode}{world}{ckpt}", "model": "324m", "context_length": 1024,
                "seed": 1, "precision": "bf16", "checkpointing": ckpt, "mode": mode,
                "world_size": world, "status": status, "tokens_per_second": rate,
                "measured_train_seconds": 2.0, "subprocess_seconds": 5.0}
    rows = [row("single", 1, 100.0), row("ddp", 8, 600.0), row("ddp", 8, 300.0, ckpt="block"),
            row("tp", 8, 50.0, status="failed")]
    planner.add_scaling_metrics(rows, 8)
    assert rows[1]["throughput_speedup"] == 6.0
    assert rows[1]["strong_scaling_efficiency"] == 0.75
    assert rows[1]["baseline_case_id"] == "single1none"
    assert rows[1]["active_gpu_seconds_measured"] == 16.0
    assert "throughput_speedup" not in rows[2]               # no single baseline with block
    assert "active_gpu_seconds_measured" not in rows[3]
    assert all(r["allocated_gpu_seconds_subprocess"] == 40.0 for r in rows)
