"""Pilot planner, evidence aggregation and executor (CPU, no training run).

Run artefacts are written by hand so that each aggregation rule is exercised on its
own: warm-up exclusion, truncated or malformed metrics, time-outs, identity
mismatches, comparability within a seed.  The executor is driven with a stand-in for
the training subprocess.
"""

import json
from dataclasses import replace
from pathlib import Path

import pytest

from systems_for_llms_b200 import pilot
from systems_for_llms_b200.config import load_config
from systems_for_llms_b200.experiments import common

SMOKE = Path(__file__).resolve().parents[1] / "configs" / "smoke.json"
SOURCE = {"python_source_sha256": "ab" * 32, "git_commit": None}


@pytest.fixture(autouse=True)
def fixed_source(monkeypatch):
    monkeypatch.setattr(pilot, "source_identity", lambda: dict(SOURCE))


def config(**changes):
    return replace(load_config(SMOKE), **changes)


def plan_for(**overrides):
    arguments = dict(microbatches=[1, 2], effective_batch_size=4, seeds=[7, 3], warmup_steps=2,
                     device="cpu", order_seed=5, timeout_seconds=30)
    arguments.update(overrides)
    return pilot.make_plan(config(max_steps=6), **arguments)


# ------------------------------------------------------------------ planning --
def test_plan_is_the_full_matrix_sealed_and_deterministic():
    plan = plan_for()
    assert len(plan["cases"]) == 2 * 2 * 2 * 2
    assert common.verify_seal(plan)
    assert plan == plan_for()
    ids = [case["case_id"] for case in plan["cases"]]
    assert len(set(ids)) == len(ids)
    for case in plan["cases"]:
        labels = case["labels"]
        assert labels["batch_size"] * labels["grad_accum_steps"] == 4
        assert case["config"]["batch_size"] == labels["batch_size"]
        assert case["config"]["model"]["attention_backend"] == labels["attention_backend"]
        assert case["config_sha256"] == common.json_sha256(case["config"])
        assert case["tokens_per_step"] == 4 * case["config"]["model"]["context_length"]
        assert case["source_sha256"] == SOURCE["python_source_sha256"]


def test_order_seed_shuffles_without_changing_the_cases():
    one, two = plan_for(order_seed=1), plan_for(order_seed=2)
    first = [case["case_id"] for case in one["cases"]]
    second = [case["case_id"] for case in two["cases"]]
    assert first != second and sorted(first) == sorted(second)
    assert one["plan_sha256"] != two["plan_sha256"]


def test_policies_select_cases():
    plan = plan_for(policies=["sdpa:block:2", "eager:none:1"], seeds=[1])
    assert sorted(case["case_id"] for case in plan["cases"]) == [
        "eager-none-mb1-acc4-seed1", "sdpa-block-mb2-acc2-seed1"]


@pytest.mark.parametrize("overrides, message", [
    (dict(policies=[]), "must not be empty"),
    (dict(policies=["flash:none:1"]), "backend:checkpoint:microbatch"),
    (dict(policies=["sdpa:none:4"]), "belong to microbatches"),
    (dict(policies=["sdpa:none:1", "sdpa:none:1"]), "duplicate"),
    (dict(microbatches=[3]), "divide"),
    (dict(microbatches=[1, 1]), "duplicate"),
    (dict(seeds=[]), "must not be empty"),
    (dict(seeds=[-1]), "seeds must be integers"),
    (dict(warmup_steps=6), "less than max_steps"),
    (dict(warmup_steps=0), "positive integer"),
    (dict(device="mps"), "cuda, or cpu"),
    (dict(timeout_seconds=float("inf")), "finite and positive"),
    (dict(effective_batch_size=True), "positive integer"),
    (dict(order_seed=1.5), "order_seed"),
])
def test_plan_rejects_bad_arguments(overrides, message):
    with pytest.raises(ValueError, match=message):
        plan_for(**overrides)


def test_write_plan_never_reuses_a_directory(tmp_path):
    plan = plan_for(seeds=[1], microbatches=[2])
    root = pilot.write_plan(plan, tmp_path / "pilot")
    assert json.loads((root / "manifest.json").read_text()) == plan
    for case in plan["cases"]:
        assert json.loads((root / case["config_path"]).read_text()) == case["config"]
    with pytest.raises(FileExistsError):
        pilot.write_plan(plan, tmp_path / "pilot")


# --------------------------------------------------------------- aggregation --
def write_run(root: Path, case: dict, *, steps=None, status="completed", step_seconds=None,
              identity=None, metadata=None, summary=None, execution="completed", hashes=None):
    """Hand-written evidence of one case; every argument overrides one aspect."""
    steps = case["max_steps"] if steps is None else steps
    run = root / "runs" / case["case_id"]
    run.mkdir(parents=True)
    durations = step_seconds or [0.5] * steps
    rows = [{"event": "start", "step": 0}]
    for index in range(1, steps + 1):
        digest = (hashes[index - 1] if hashes else f"{index:064x}")
        rows.append({"event": "train", "step": index, "loss": 3.0 - 0.1 * index,
                     "step_seconds": durations[index - 1],
                     "tokens_seen": index * case["tokens_per_step"],
                     "batch_start_sha256": digest})
    (run / "metrics.jsonl").write_text("".join(json.dumps(r) + "\n" for r in rows))
    document = {"config_sha256": case["config_sha256"],
                "source": {"python_source_sha256": case["source_sha256"]},
                "data_identity": identity or {"kind": "synthetic", "sha256": "cd" * 32},
                "gpu_name": None, "gpu_count": 0}
    document.update(metadata or {})
    (run / "metadata.json").write_text(json.dumps(document))
    body = {"status": status, "step": steps, "tokens_seen": steps * case["tokens_per_step"],
            "valid_loss": 2.5, "setup_seconds": 0.1, "train_seconds": 1.0, "eval_seconds": 0.1,
            "checkpoint_seconds": 0.0, "wall_seconds": 1.3, "peak_cuda_allocated_bytes": None,
            "peak_cuda_reserved_bytes": None}
    body.update(summary or {})
    (run / "summary.json").write_text(json.dumps(body))
    if execution is not None:
        (root / "execution").mkdir(exist_ok=True)
        record = ({"status": execution, "returncode": 0, "wall_seconds": 2.0}
                  if isinstance(execution, str) else execution)
        (root / "execution" / f"{case['case_id']}.json").write_text(json.dumps(record))


@pytest.fixture
def one_seed(tmp_path):
    plan = plan_for(seeds=[1], microbatches=[2], policies=["sdpa:none:2", "sdpa:block:2"])
    return tmp_path, plan


def test_warmup_rows_are_excluded_and_p90_is_interpolated(one_seed):
    root, plan = one_seed
    case = plan["cases"][0]
    write_run(root, case, step_seconds=[9.0, 9.0, 1.0, 2.0, 3.0, 4.0])
    row = pilot.summarize_case(root, case, plan["warmup_steps"])
    assert row["status"] == "completed" and row["measured_steps"] == 4
    assert row["step_seconds_median"] == 2.5
    assert row["step_seconds_p90"] == pytest.approx(3.7)     # 0.9 * (4 - 1) = index 2.7
    assert row["tokens_per_second"] == pytest.approx(case["tokens_per_step"] * 4 / 10.0)
    assert row["last_train_loss"] == pytest.approx(2.4)
    assert len(row["batch_stream_sha256"]) == 64


def test_truncated_metrics_are_insufficient_not_completed(one_seed):
    root, plan = one_seed
    case = plan["cases"][0]
    write_run(root, case, steps=4, status="paused")
    row = pilot.summarize_case(root, case, plan["warmup_steps"])
    assert row["status"] == "insufficient_samples"
    assert row["measured_steps"] == 2 and row["batch_stream_sha256"] is None


def test_malformed_metrics_are_invalid(one_seed):
    root, plan = one_seed
    case = plan["cases"][0]
    write_run(root, case)
    path = root / "runs" / case["case_id"] / "metrics.jsonl"
    rows = [json.loads(line) for line in path.read_text().splitlines()]
    rows[3]["step"] = 7                                     # not consecutive
    path.write_text("".join(json.dumps(r) + "\n" for r in rows))
    row = pilot.summarize_case(root, case, plan["warmup_steps"])
    assert row["status"] == "invalid_output" and "consecutive" in row["error"]


def test_missing_files_and_identity_mismatch(one_seed):
    root, plan = one_seed
    first, second = plan["cases"]
    row = pilot.summarize_case(root, first, plan["warmup_steps"])
    assert row["status"] == "missing_output" and "summary.json is missing" in row["error"]
    write_run(root, second, metadata={"config_sha256": "00" * 32})
    row = pilot.summarize_case(root, second, plan["warmup_steps"])
    assert row["status"] == "invalid_output" and "config identity" in row["error"]


def test_timeout_and_oom_are_classified(one_seed):
    root, plan = one_seed
    first, second = plan["cases"]
    (root / "execution").mkdir()
    (root / "execution" / f"{first['case_id']}.json").write_text(json.dumps(
        {"status": "timeout", "returncode": -9, "wall_seconds": 30.0, "error": "timed out"}))
    row = pilot.summarize_case(root, first, plan["warmup_steps"])
    assert row["status"] == "timeout" and row["failure_kind"] == "timeout"
    (root / "execution" / f"{second['case_id']}.json").write_text(json.dumps(
        {"status": "failed", "returncode": 1, "wall_seconds": 3.0}))
    (root / "logs").mkdir()
    (root / "logs" / f"{second['case_id']}.log").write_text(
        "torch.OutOfMemoryError: CUDA out of memory. Tried to allocate 2 GiB")
    row = pilot.summarize_case(root, second, plan["warmup_steps"])
    assert row["status"] == "failed" and row["failure_kind"] == "oom"


def test_non_finite_summary_numbers_are_invalid(one_seed):
    root, plan = one_seed
    case = plan["cases"][0]
    write_run(root, case, summary={"wall_seconds": -1.0})
    row = pilot.summarize_case(root, case, plan["warmup_steps"])
    assert row["status"] == "invalid_output" and "nonnegative" in row["error"]


def test_comparability_needs_the_same_data_and_batch_stream(one_seed):
    root, plan = one_seed
    first, second = plan["cases"]
    write_run(root, first)
    write_run(root, second)
    aggregate = pilot.aggregate_results(root, plan)
    assert aggregate["comparability"]["status"] == "passed"
    assert aggregate["status_counts"] == {"completed": 2}
    assert aggregate["plan_sha256"] == plan["plan_sha256"]


def test_comparability_fails_on_a_different_batch_stream(one_seed):
    root, plan = one_seed
    first, second = plan["cases"]
    write_run(root, first)
    write_run(root, second, hashes=[f"{index + 100:064x}" for index in range(6)])
    aggregate = pilot.aggregate_results(root, plan)
    assert aggregate["comparability"]["status"] == "failed"
    assert any("batch_stream_sha256" in reason for reason in aggregate["comparability"]["reasons"])


def test_comparability_is_insufficient_when_a_case_is_missing(one_seed):
    root, plan = one_seed
    write_run(root, plan["cases"][0])
    aggregate = pilot.aggregate_results(root, plan)
    assert aggregate["comparability"]["status"] == "insufficient"


# ------------------------------------------------------------------ executor --
def test_executor_runs_untouched_cases_continues_after_failure_never_overwrites(
        tmp_path, monkeypatch):
    plan = plan_for(seeds=[1], microbatches=[2])
    root = pilot.write_plan(plan, tmp_path / "pilot")
    by_id = {case["case_id"]: case for case in plan["cases"]}
    failing = plan["cases"][1]["case_id"]
    touched = plan["cases"][2]["case_id"]
    (root / "runs").mkdir()
    (root / "runs" / touched).mkdir()                       # evidence from an earlier attempt
    (root / "runs" / touched / "keep.txt").write_text("old")
    calls = []

    def fake_run(command, log_path, timeout, environment):
        case_id = Path(command[command.index("--output-dir") + 1]).name
        calls.append(case_id)
        assert timeout == plan["timeout_seconds"] and "-m" in command
        if case_id == failing:
            return {"status": "failed", "returncode": 1, "wall_seconds": 0.1, "error": "boom"}
        write_run(root, by_id[case_id], execution=None)
        return {"status": "completed", "returncode": 0, "wall_seconds": 0.2}

    monkeypatch.setattr(pilot, "run_training_case", fake_run)
    with pytest.raises(ValueError, match="allow-cpu"):
        pilot.execute_plan(root)
    aggregate = pilot.execute_plan(root, allow_cpu=True)
    assert touched not in calls and failing in calls and len(calls) == 3
    assert (root / "runs" / touched / "keep.txt").read_text() == "old"
    assert aggregate["status_counts"]["failed"] == 1
    assert json.loads((root / "aggregate.json").read_text()) == aggregate
    calls.clear()
    pilot.execute_plan(root, allow_cpu=True)                 # second entry: nothing left to run
    assert calls == []


def test_executor_refuses_changed_source_or_config(tmp_path, monkeypatch):
    plan = plan_for(seeds=[1], microbatches=[2], policies=["sdpa:none:2"])
    root = pilot.write_plan(plan, tmp_path / "pilot")
    monkeypatch.setattr(pilot, "run_training_case",
                        lambda *a, **k: pytest.fail("a case was started"))
    monkeypatch.setattr(pilot, "source_identity", lambda: {"python_source_sha256": "ff" * 32})
    with pytest.raises(ValueError, match="source changed"):
        pilot.execute_plan(root, allow_cpu=True)
    monkeypatch.setattr(pilot, "source_identity", lambda: dict(SOURCE))
    path = root / plan["cases"][0]["config_path"]
    edited = json.loads(path.read_text())
    edited["learning_rate"] *= 2
    path.write_text(json.dumps(edited))
    with pytest.raises(ValueError, match="resolved config changed"):
        pilot.execute_plan(root, allow_cpu=True)
    manifest = json.loads((root / "manifest.json").read_text())
    manifest["warmup_steps"] = 1                            # tampered after sealing
    (root / "manifest.json").write_text(json.dumps(manifest))
    with pytest.raises(ValueError, match="identity is invalid"):
        pilot.execute_plan(root, allow_cpu=True)
