"""Orchestration logic of the attention studies, driven by injected evaluators (no GPU).

Mirrors the reference's harness tests (attention_lab/test_study.py, test_search.py,
test_gpu_search.py, test_block_benchmark.py, test_analyze_study.py): fake timings go
in through ``evaluate=`` parameters or a patched ``run_case``.
"""

import json
import math
from dataclasses import asdict
from pathlib import Path
from unittest import mock

import pytest
import torch

from systems_for_llms_b200.attention import (analyze_extensions, analyze_study, backward_study,
                                             block_benchmark, decode_study, gpu_search, launcher,
                                             study)
from systems_for_llms_b200.attention.masks import MaskSpec
from systems_for_llms_b200.attention.search import (FIELD_ORDER, CandidateResult, KernelConfig,
                                                    default_configs, differing_fields, replay,
                                                    sanitize, search)


# ------------------------------------------------------------------ search ------
def latency_of(config: KernelConfig) -> float:
    """A separable cost with one clear optimum: two streams, interval, wide key blocks."""
    return (1.0 + 0.01 * config.block_q / 64 + 0.02 * (128 // config.block_k)
            + (0.3 if config.implementation == "csr" else 0.0)
            + (0.1 if not config.use_full_blocks else 0.0)
            + {"two_stream": 0.0, "two_stream_smem_p": 0.05, "one_stream": 0.4}[config.pipeline])


def fake_evaluate(config):
    return CandidateResult(True, latency_of(config))


def test_space_sizes_per_head_dimension():
    wide = default_configs(64)
    assert len(wide) == 42 and len(set(wide)) == 42
    assert {c.pipeline for c in wide} == {"two_stream", "two_stream_smem_p", "one_stream"}
    narrow = default_configs(128)
    assert len(narrow) == 14 and {c.pipeline for c in narrow} == {"one_stream"}
    # the interval form has no schedule granularity: it appears once per remaining setting
    assert sum(c.implementation == "interval" for c in wide) == 6
    assert all((c.block_q, c.block_k) == (128, 128) for c in wide if c.implementation == "interval")


@pytest.mark.parametrize("method", ["random", "descent"])
def test_search_respects_budget_and_never_repeats(method):
    result = search(fake_evaluate, budget=9, method=method, seed=3)
    configs = [o.config for o in result.history]
    assert len(configs) == 9 == len(set(configs))
    assert result.best.result.latency_ms == min(o.result.latency_ms for o in result.history)
    assert json.loads(result.to_json())["evaluations"] == 9


def test_search_is_deterministic_per_seed():
    a = search(fake_evaluate, budget=12, method="descent", seed=5)
    b = search(fake_evaluate, budget=12, method="descent", seed=5)
    assert [o.config for o in a.history] == [o.config for o in b.history]
    c = search(fake_evaluate, budget=12, method="descent", seed=6)
    assert [o.config for o in a.history] != [o.config for o in c.history]


def test_descent_sweeps_one_field_at_a_time_from_the_incumbent():
    start = KernelConfig(64, 32, "csr", False, "one_stream")
    result = search(fake_evaluate, budget=20, method="descent", seed=1, start=start)
    first, *rest = result.history
    assert first.origin == "start" and first.config == start and first.parent is None
    incumbent, incumbent_ms = first.config, first.result.latency_ms
    swept = []
    for observation in rest:
        if not observation.origin.startswith("sweep:"):
            break
        name = observation.origin.split(":")[1]
        assert name in FIELD_ORDER and observation.parent is not None
        assert differing_fields(observation.parent, observation.config) == 1
        assert getattr(observation.parent, name) != getattr(observation.config, name)
        # a sweep step is always taken from a configuration at least as fast as all before it
        assert latency_of(observation.parent) <= incumbent_ms + 1e-12
        incumbent_ms = min(incumbent_ms, latency_of(observation.parent))
        swept.append(name)
    assert swept[0] == "pipeline" and len(set(swept)) >= 3
    # on a separable cost the descent reaches the global optimum well inside the budget
    assert result.best.result.latency_ms == pytest.approx(min(map(latency_of, default_configs())))


def test_descent_restarts_far_from_what_it_measured():
    flat = search(lambda c: CandidateResult(True, 1.0), budget=42, method="descent", seed=0)
    restarts = [o for o in flat.history if o.origin == "restart"]
    assert restarts and len(flat.history) == 42
    for observation in restarts:
        before = [o.config for o in flat.history[:observation.evaluation - 1]]
        reach = min(differing_fields(observation.config, c) for c in before)
        others = [c for c in default_configs() if c not in before]
        assert reach == max(min(differing_fields(c, m) for m in before) for c in others)


def test_failures_spend_budget_and_are_recorded():
    def flaky(config):
        if config.block_k == 32:
            raise RuntimeError("out of resources")
        return fake_evaluate(config)

    for method in ("random", "descent"):
        result = search(flaky, budget=42, method=method, seed=0)
        failed = [o for o in result.history if not o.result.eligible]
        assert len(result.history) == 42 and len(failed) == 12
        assert all("out of resources" in o.result.error for o in failed)
        assert result.best.config.block_k != 32


def test_sanitize_rejects_malformed_results():
    assert sanitize("fast").error.startswith("invalid_result")
    assert not sanitize(CandidateResult(True, float("nan"))).eligible
    assert not sanitize(CandidateResult(True, -1.0)).eligible
    assert not sanitize(CandidateResult(1, 1.0)).eligible
    assert sanitize(CandidateResult(True, 2)).eligible
    assert not CandidateResult(True, 1.0, error="late failure").eligible


def test_bad_arguments_raise():
    with pytest.raises(ValueError):
        search(fake_evaluate, budget=-1)
    with pytest.raises(ValueError):
        search(fake_evaluate, budget=2, method="grid")
    with pytest.raises(TypeError):
        search(fake_evaluate, [("not", "a config")], budget=1)
    with pytest.raises(TypeError):
        search(fake_evaluate, budget=1, start="fastest")
    with pytest.raises(ValueError):
        KernelConfig(0, 64)
    with pytest.raises(ValueError):
        KernelConfig(64, 64, pipeline="three_stream")


def test_offline_replay_matches_a_live_search():
    live = search(fake_evaluate, budget=42, method="random", seed=0)
    again = replay(live.to_dict()["history"], budget=8, method="descent", seed=2)
    direct = search(fake_evaluate, [o.config for o in live.history], budget=8, method="descent",
                    seed=2)
    assert again.best.config == direct.best.config
    partial = replay(live.to_dict()["history"][:5], budget=10, method="random", seed=0,
                     configs=default_configs())
    assert sum(o.result.eligible for o in partial.history) <= 5


# --------------------------------------------------------------- gpu_search ------
def test_gpu_search_confirms_winner_on_a_fresh_seed():
    seeds = []

    def fake_run_case(**kwargs):
        seeds.append(kwargs["seed"])
        config = KernelConfig(kwargs["block_q"], kwargs["block_k"], kwargs["implementation"],
                              kwargs["use_full_blocks"])
        return {"correct": True, "status": "passed", "latency_ms": latency_of(config)}

    with mock.patch.object(gpu_search.benchmark, "run_case", fake_run_case):
        report = gpu_search.run_experiment(budget=6, method="random", search_seed=1, length=256,
                                           seed=40, spec=MaskSpec(causal=True))
    assert report["status"] == "passed"
    assert seeds == [40] * 6 + [41]
    assert report["confirmation"]["counts_toward_search_budget"] is False
    assert len(report["measurements"]) == 6


def test_gpu_search_fails_when_confirmation_is_wrong():
    calls = {"n": 0}

    def fake_run_case(**kwargs):
        calls["n"] += 1
        return {"correct": calls["n"] <= 4, "latency_ms": 1.0}

    with mock.patch.object(gpu_search.benchmark, "run_case", fake_run_case):
        report = gpu_search.run_experiment(budget=4, method="random", length=128)
    assert report["status"] == "failed"
    with pytest.raises(ValueError):
        gpu_search.run_experiment(budget=0)
    with pytest.raises(ValueError):
        gpu_search.run_experiment(budget=4, block_q=64)


def test_spec_for_mask_names():
    assert gpu_search.spec_for("combined", 7, 1) == MaskSpec(True, 7, 1, True)
    assert gpu_search.spec_for("dense", 7, 1) == MaskSpec()


# -------------------------------------------------------------------- study ------
def test_plans_are_deterministic_with_expected_sizes():
    sizes = {stage: len(study.build_plan(stage)["cases"]) for stage in study.STAGES}
    assert sizes == {"smoke": 20, "ablation": 120, "flex_hints": 24, "tuning": 134,
                     "confirmation": 12}
    assert study.build_plan("ablation") == study.build_plan("ablation")
    with pytest.raises(ValueError):
        study.build_plan("everything")


def test_document_cases_never_use_the_interval_lowering():
    for stage in study.STAGES:
        for case in study.build_plan(stage)["cases"]:
            if case["spec"]["same_document"]:
                assert case["config"]["implementation"] == "csr"
                assert len(case["document_ids"]) == case["length"]


def test_ablation_order_is_shuffled_per_seed():
    cases = study.build_plan("ablation")["cases"]
    first = [c["variant"] for c in cases if c["workload_id"] == "n1024-d64-causal"]
    orders = {tuple(first[i:i + 4]) for i in range(0, 12, 4)}
    assert len(orders) > 1 and all(sorted(o) == sorted(study.VARIANTS) for o in orders)


def plausible(**kwargs):
    config = KernelConfig(kwargs["block_q"], kwargs["block_k"], kwargs["implementation"],
                          kwargs["use_full_blocks"])
    measured = {"status": "passed", "correct": True, "latency_ms": latency_of(config),
                "baseline_latency_ms": 2.0, "baseline": "sdpa_native", "first_call_ms": 3.0,
                "baseline_over_custom": 2.0 / latency_of(config), "mask_density": 0.5}
    if kwargs["include_flex"]:
        measured["flex"] = {"status": "passed", "correct": True, "latency_ms": 1.5,
                            "contiguous_hint": kwargs["flex_contiguous"]}
    return measured


def test_run_study_records_every_case(tmp_path):
    plan = study.build_plan("ablation")
    summary = study.run_study(plan, tmp_path / "run", evaluate=plausible)
    assert summary["status"] == "passed" and summary["passed_cases"] == 120
    assert summary["flex_requested_cases"] == 36 == summary["flex_passed_cases"]
    assert len(list((tmp_path / "run" / "cases").glob("*.json"))) == 120
    pairs = json.loads((tmp_path / "run" / "baseline_pairs.json").read_text())
    assert all(p["flex_speedup"] is not None for p in pairs)
    with pytest.raises(FileExistsError):
        study.run_study(plan, tmp_path / "run", evaluate=plausible)


def test_smoke_stops_at_first_failure(tmp_path):
    calls = []

    def evaluate(**kwargs):
        calls.append(1)
        if len(calls) == 3:
            raise RuntimeError("mismatch")
        return plausible(**kwargs)

    summary = study.run_study(study.build_plan("smoke"), tmp_path / "s", evaluate=evaluate)
    assert summary["status"] == "stopped_after_failure"
    assert summary["completed_cases"] == 3 and summary["not_run_cases"] == 17


def test_fatal_device_errors_stop_any_stage(tmp_path):
    def evaluate(**kwargs):
        return {"status": "failed", "correct": False, "error": "CUDA error: an illegal memory access"}

    summary = study.run_study(study.build_plan("ablation"), tmp_path / "f", evaluate=evaluate)
    assert summary["status"] == "stopped_after_failure" and summary["completed_cases"] == 1


def test_time_budget_is_checked_between_cases(tmp_path):
    ticks = iter(range(0, 10_000, 400))
    with mock.patch.object(study.time, "monotonic", lambda: next(ticks)):
        summary = study.run_study(study.build_plan("smoke"), tmp_path / "t", evaluate=plausible,
                                  time_budget_seconds=900)
    assert summary["status"] == "time_budget_exhausted" and summary["completed_cases"] < 20
    with pytest.raises(ValueError):
        study.run_study(study.build_plan("smoke"), tmp_path / "u", evaluate=plausible,
                        time_budget_seconds=math.inf)


def test_tuning_writes_winners_and_replay_then_confirmation_transfers(tmp_path):
    summary = study.run_study(study.build_plan("tuning"), tmp_path / "tuning", evaluate=plausible)
    assert summary["status"] == "passed"
    winners = json.loads((tmp_path / "tuning" / "winners.json").read_text())
    assert set(winners) == {"tune-causal", "tune-window128", "tune-window512", "tune-document"}
    assert winners["tune-causal"]["config"]["implementation"] == "interval"
    assert winners["tune-document"]["config"]["implementation"] == "csr"
    replayed = json.loads((tmp_path / "tuning" / "search_replay.json").read_text())
    assert all(w["status"] == "completed" for w in replayed["workloads"])
    full = [t for t in replayed["workloads"][0]["trials"] if t["budget"] == 12]
    assert all(t["relative_regret"] >= 0 for t in full)
    plan = study.build_plan("confirmation", winners=study.load_winners(tmp_path / "tuning"))
    assert len(plan["cases"]) == 24
    transferred = [c for c in plan["cases"] if c["case_id"].endswith("-transferred")]
    assert len(transferred) == 12
    assert all(c["selection"]["source_case_id"] for c in transferred)


def test_replay_reports_incomplete_tables():
    records = [{"case": c, "measurement": plausible(**study.case_arguments(c, plan))}
               for plan in [study.build_plan("tuning")] for c in plan["cases"][:5]]
    report = study.replay_search(records)
    assert report["workloads"][0]["status"] == "incomplete_table"


# ---------------------------------------------------------- block benchmark ------
def block_measurement(case, **kwargs):
    variants = {"custom_interval_split": {"status": "passed", "correct": True,
                                          "block_latency_ms": 1.0, "attention_latency_ms": 0.2},
                "sdpa": {"status": "passed", "correct": True, "block_latency_ms": 1.3,
                         "attention_latency_ms": 0.5}}
    result = {"status": "passed", "correct": True, "reference_finite": True,
              "inputs_weights_unchanged": True, "variants": variants}
    block_benchmark.add_speedups(result)
    return result


def test_block_plan_freezes_configurations():
    plan = block_benchmark.build_block_plan()
    assert len(plan["cases"]) == 8
    assert all(c["selection"]["policy"] == "fixed_default" for c in plan["cases"])
    winner = {"tune-causal": {"case_id": "x", "config": asdict(KernelConfig(64, 32, "csr", False))}}
    plan = block_benchmark.build_block_plan(winner)
    causal = [c for c in plan["cases"] if c["pattern"] == "causal"]
    assert all(c["config"]["block_k"] == 32 and c["selection"]["source_case_id"] == "x"
               for c in causal)
    with pytest.raises(ValueError):
        block_benchmark.build_block_plan({"tune-causal": {"config": asdict(KernelConfig(16, 16))}})


def test_block_study_bookkeeping(tmp_path):
    summary = block_benchmark.run_block_study(tmp_path / "b", evaluate=block_measurement)
    assert summary["status"] == "passed" and summary["passed_cases"] == 8
    record = json.loads(next((tmp_path / "b" / "cases").glob("*.json")).read_text())
    measured = record["measurement"]
    assert measured["speedup_vs_sdpa"] == pytest.approx(1.3)
    assert measured["attention_speedup_vs_sdpa"] == pytest.approx(2.5)
    fraction = 0.5 / 1.3
    assert measured["amdahl_estimate_vs_sdpa"] == pytest.approx(1 / (1 - fraction + fraction / 2.5))
    with pytest.raises(ValueError):
        block_benchmark.run_block_study(tmp_path / "c", tuning_dir=tmp_path, winners={},
                                        evaluate=block_measurement)


def test_block_study_counts_failures_and_rejects_non_tuning_dirs(tmp_path):
    def broken(case, **kwargs):
        result = block_measurement(case)
        result["variants"]["sdpa"]["block_latency_ms"] = -1.0
        return result

    summary = block_benchmark.run_block_study(tmp_path / "b", evaluate=broken)
    assert summary["status"] == "completed_with_failures" and summary["failed_cases"] == 8
    study.write_json(tmp_path / "held" / "plan.json", {"stage": "confirmation"})
    with pytest.raises(ValueError):
        block_benchmark.training_winners(tmp_path / "held")


# ------------------------------------------------------------------ analysis ------
def test_analysis_pairs_ablations_and_counts_the_unpairable(tmp_path):
    study.run_study(study.build_plan("ablation"), tmp_path / "ablation", evaluate=plausible)
    report = analyze_study.analyze(tmp_path)["studies"][0]
    by_name = {item["comparison"]: item for item in report["ablations"]}
    assert by_name["csr_masked/csr_full"]["paired_cases"] == 36
    assert by_name["csr_full/interval_split"]["paired_cases"] == 24
    assert by_name["csr_full/interval_split"]["not_applicable_groups"] == 12
    assert by_name["csr_full/interval_split"]["geomean_speedup"] == pytest.approx(
        latency_of(KernelConfig(128, 128, "csr", True))
        / latency_of(KernelConfig(128, 128, "interval", True)))
    assert by_name["interval_masked/interval_split"]["regressions"] == 0
    flex = [b for b in report["baselines"] if b["baseline"] == "flex"]
    assert sum(b["paired_cases"] for b in flex) == 120
    text = analyze_study.markdown(analyze_study.analyze(tmp_path))
    assert "csr_full/interval_split" in text and "External baselines" in text


def test_analysis_treats_missing_and_failed_as_such(tmp_path):
    def evaluate(**kwargs):
        if kwargs["implementation"] == "interval" and not kwargs["use_full_blocks"]:
            return {"status": "failed", "correct": False, "error": "boom"}
        return plausible(**kwargs)

    study.run_study(study.build_plan("ablation"), tmp_path / "ablation", evaluate=evaluate)
    report = analyze_study.analyze_directory(tmp_path / "ablation")
    item = {i["comparison"]: i for i in report["ablations"]}["interval_masked/interval_split"]
    assert item["paired_cases"] == 0 and item["failed_groups"] == 24
    assert report["failed_cases"] == 24 and len(report["failures"]) == 24


def test_analysis_of_tuning_confirmation_and_block_runs(tmp_path):
    study.run_study(study.build_plan("tuning"), tmp_path / "tuning", evaluate=plausible)
    winners = study.load_winners(tmp_path / "tuning")
    study.run_study(study.build_plan("confirmation", winners=winners), tmp_path / "confirmation",
                    evaluate=plausible)
    block_benchmark.run_block_study(tmp_path / "block", winners=winners,
                                    evaluate=block_measurement)
    summary = analyze_study.analyze(tmp_path)
    stages = {s["stage"]: s for s in summary["studies"]}
    assert set(stages) == {"tuning", "confirmation", "block"}
    tuning = stages["tuning"]["tuning"]
    assert tuning[0]["valid_configurations"] in (14, 36, 42)
    assert stages["tuning"]["search_replay"]["groups"]
    confirmation = stages["confirmation"]["confirmation"][0]
    assert confirmation["paired_cases"] == 12 and confirmation["geomean_speedup"] >= 1.0
    scopes = {(b["baseline"], b["scope"]) for b in stages["block"]["block_comparisons"]}
    assert ("sdpa", "single_block_forward") in scopes
    assert "Offline search replay" in analyze_study.markdown(summary)


def test_rank_ties_and_spearman():
    assert analyze_study.ranks([3.0, 1.0, 3.0, 2.0]) == [2.5, 0.0, 2.5, 1.0]
    rows = [{"x": i, "latency_ms": float(i * i)} for i in range(1, 6)]
    assert analyze_study.spearman(rows, "x")["spearman_rho"] == pytest.approx(1.0)
    assert analyze_study.spearman(rows[:2], "x")["spearman_rho"] is None


# ------------------------------------------------------------------ launcher ------
def test_manifest_bounds_and_contents():
    settings = launcher.manifest("tuning", None, "run-1")
    assert settings["job_timeout_seconds"] == settings["study_time_budget_seconds"] + 60
    assert any(name.endswith("attention/study.py") for name in settings["source_sha256"])
    assert any(name.endswith(".cu") for name in settings["source_sha256"])
    with pytest.raises(ValueError):
        launcher.manifest("tuning", 10, "run-1")
    with pytest.raises(ValueError):
        launcher.manifest("tuning", None, "bad id")
    with pytest.raises(ValueError):
        launcher.manifest("nonsense", None, "x")


def test_execute_snapshots_sources_and_records_outcome(tmp_path):
    settings = launcher.manifest("decode-smoke", 60, "unit")
    seen = {}

    def runner(command, log_path, seconds):
        seen.update(command=command, seconds=seconds)
        log_path.write_text("ran\n")
        return {"status": "completed", "returncode": 0}

    outcome = launcher.execute(settings, tmp_path / "run", runner=runner, require_gpu=False)
    assert outcome["status"] == "completed" and seen["seconds"] == 120
    assert seen["command"][1:3] == ["-m", settings["module"]] and "--execute" in seen["command"]
    for name in ("launch.json", "environment.json", "command.json", "outcome.json"):
        assert (tmp_path / "run" / name).is_file()
    assert (tmp_path / "run" / "source" / next(iter(settings["source_sha256"]))).is_file()
    with pytest.raises(FileExistsError):
        launcher.execute(settings, tmp_path / "run", runner=runner, require_gpu=False)


def test_execute_detects_changed_sources_and_timeouts(tmp_path):
    settings = launcher.manifest("smoke", None, "unit")
    first = next(iter(settings["source_sha256"]))
    tampered = {**settings, "source_sha256": {**settings["source_sha256"], first: "0" * 64}}
    outcome = launcher.execute(tampered, tmp_path / "a", runner=lambda *a: {}, require_gpu=False)
    assert outcome["status"] == "failed" and "Source changed" in outcome["error"]
    outcome = launcher.execute(settings, tmp_path / "b", require_gpu=False,
                               runner=lambda *a: {"status": "timed_out", "returncode": -15})
    assert outcome["status"] == "timed_out"


def test_run_child_kills_the_process_group_on_timeout(tmp_path):
    import sys
    result = launcher.run_child([sys.executable, "-c", "import time; time.sleep(30)"],
                                tmp_path / "log.txt", 0.5)
    assert result["status"] == "timed_out"
    result = launcher.run_child([sys.executable, "-c", "print('ok')"], tmp_path / "log2.txt", 20)
    assert result == {"status": "completed", "returncode": 0}
    assert (tmp_path / "log2.txt").read_text().strip() == "ok"


def test_campaign_budget_guard_and_gating(tmp_path):
    with pytest.raises(ValueError):
        launcher.plan_campaign("c", budget_gpu_minutes=5)
    plan = launcher.plan_campaign("c", budget_gpu_minutes=90)
    assert [s["stage"] for s in plan["stages"]] == list(launcher.CAMPAIGN_ORDER)
    ran = []

    def execute_stage(settings, output):
        ran.append(settings["stage"])
        status = "completed_with_failures" if settings["stage"] == "ablation" else "passed"
        study.write_json(output / "study" / "summary.json",
                         {"status": status, "not_run_cases": 0, "flex_failed_cases": 0})
        if settings["stage"] in ("confirmation", "block"):
            assert settings["tuning_dir"].endswith("tuning/study")
        return {"status": "completed"}

    result = launcher.run_campaign(plan, tmp_path / "c", execute_stage=execute_stage)
    assert result["status"] == "stopped" and result["stage"] == "ablation"
    assert ran == ["smoke", "ablation"]
    assert launcher.stage_acceptable("tuning", {"status": "completed_with_failures",
                                                "passed_cases": 3, "not_run_cases": 0})
    assert not launcher.stage_acceptable("smoke", {"status": "passed", "not_run_cases": 2})


# ----------------------------------------------------- backward / decode study ------
def test_dense_oracle_agrees_with_the_mask_compiler_semantics():
    from systems_for_llms_b200.attention.benchmark import dense_mask
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 2, 37, 16) for _ in range(3))
    docs = [i // 9 for i in range(37)]
    spec = MaskSpec(causal=True, window_left=5, same_document=True)
    got = backward_study.dense_attention(q, k, v, spec, docs)
    mask = dense_mask(37, spec, docs)
    scores = (q @ k.transpose(-1, -2)) * 16 ** -0.5
    want = scores.masked_fill(~mask, float("-inf")).softmax(-1) @ v
    torch.testing.assert_close(got, want)


def test_scale_aware_comparison_rejects_zero_gradients():
    reference = torch.full((8, 8), 1e-4)
    assert backward_study.scale_aware_comparison(reference * 1.01, reference)["correct"]
    assert not backward_study.scale_aware_comparison(torch.zeros(8, 8), reference)["correct"]
    assert not backward_study.scale_aware_comparison(torch.full((8, 8), float("nan")),
                                                     reference)["correct"]


def test_backward_run_jobs_budget_failures_and_fatal_stop(tmp_path):
    jobs = [("correctness", lambda: {"kind": "correctness", "status": "passed"}),
            ("performance", lambda: (_ for _ in ()).throw(ValueError("bad shape"))),
            ("performance", lambda: (_ for _ in ()).throw(
                backward_study.TrainingCaptureError("capture failed"))),
            ("transformer", lambda: {"kind": "transformer", "status": "passed"})]
    report = backward_study.run_jobs(jobs, tmp_path, {}, 100.0)
    assert report["status"] == "failed" and report["completed_cases"] == 3
    assert report["stopped_after_cuda_failure"] and report["cases"][2]["fatal_cuda_state"]
    assert (tmp_path / "case_002.json").is_file()
    (tmp_path / "b").mkdir()
    partial = backward_study.run_jobs(jobs[:1] * 3, tmp_path / "b", {}, 0.0)
    assert partial["status"] == "partial_budget" and partial["completed_cases"] == 0


def test_backward_plan_sizes():
    assert len(backward_study.planned_jobs("smoke")) == 8
    assert len(backward_study.planned_jobs("study")) == 14


def test_decode_smoke_plan_is_582_checks_and_reference_handles_empty_rows():
    assert len(decode_study.REFERENCE_VARIANTS) * decode_study.smoke_case_count() == 582
    assert len(decode_study.VARIANTS) * decode_study.smoke_case_count() == 873
    torch.manual_seed(0)
    q = torch.randn(2, 4, 8)
    k, v = torch.randn(2, 2, 5, 8), torch.randn(2, 2, 5, 8)
    out = decode_study.reference(q, k, v, torch.tensor([0, 3]))
    assert torch.equal(out[0], torch.zeros(4, 8))
    scores = torch.einsum("hd,hnd->hn", q[1], k[1].repeat_interleave(2, 0)[:, :3]) * 8 ** -0.5
    want = torch.einsum("hn,hnd->hd", scores.softmax(-1), v[1].repeat_interleave(2, 0)[:, :3])
    torch.testing.assert_close(out[1], want)


def decode_record(seed):
    timings = {}
    for variant, base in (("token", 2.0), ("tile", 1.0)):
        for splits in decode_study.STUDY_SPLITS:
            ms = base / min(splits, 8) + 0.01 * splits
            timings[f"cuda_{variant}_split_{splits}"] = {"median_ms": ms, "samples_ms": [ms] * 3}
    timings["sdpa_flash"] = {"median_ms": 0.5, "samples_ms": [0.5, 0.5, 0.5]}
    record = {"batch": 1, "query_heads": 32, "kv_heads": 4, "groups": 8, "length": 4096,
              "dim": 128, "dtype": "torch.bfloat16", "seed": seed, "timings": timings,
              "checks": {"sdpa_flash": {"max_abs_error": 1e-3}}, "setup": {},
              "cache_bytes": 2 * 4 * 4096 * 128 * 2}
    decode_study.summarise_case(record)
    return record


def test_decode_case_summary_and_study_summary():
    record = decode_record(211)
    assert record["best_observed"] == "cuda_tile_split_8"
    assert record["best_tile_over_best_token"] == pytest.approx((2 / 8 + 0.08) / (1 / 8 + 0.08))
    assert record["speedups"]["sdpa_flash"] == pytest.approx(0.5 / (1 / 8 + 0.08))
    assert record["effective_kv_bandwidth_gbs"] == pytest.approx(
        record["cache_bytes"] / ((1 / 8 + 0.08) * 1e6))
    summary = decode_study.study_summary([record, decode_record(212)])
    assert summary["paired_baselines_best_observed"]["sdpa_flash"]["paired_cases"] == 2
    assert summary["planned_cases"] == 30


def extension_run(root: Path, study_files: dict, outcome="completed"):
    study.write_json(root / "outcome.json", {"status": outcome})
    study.write_json(root / "environment.json", {"devices": ["B200"], "torch": "2.11", "cuda": "12.8"})
    for name, value in study_files.items():
        study.write_json(root / "study" / name, value)


def test_extension_report_pools_only_finished_runs(tmp_path):
    records = [decode_record(211), decode_record(212)]
    extension_run(tmp_path / "decode", {
        "summary.json": {"status": "completed", "planned_cases": 30, "preflight": {"cases": 582}},
        "benchmark.json": records,
        "preflight/correctness.json": [{"finite": True, "max_abs_error": 0.004}] * 5})
    timing = {"timing": {"samples_ms": [1.0, 1.2, 1.1], "mode": "cuda_graph"}}
    slow = {"timing": {"samples_ms": [2.2, 2.2, 2.2], "mode": "cuda_graph"}}
    case = {"kind": "attention_training", "status": "passed", "n": 1024, "d": 64,
            "spec": {"causal": True, "window_left": 127, "window_right": None,
                     "same_document": False},
            "variants": {analyze_extensions.CUSTOM: {"status": "passed", "backward_only": timing,
                                                     "forward_backward": timing},
                         "pytorch_sdpa_bool_mask": {"status": "passed", "backward_only": slow,
                                                    "forward_backward": slow,
                                                    "errors": {"dq": {"max_abs_error": 0.01}}}}}
    extension_run(tmp_path / "backward", {
        "summary.json": {"status": "passed", "planned_cases": 1, "cases": [case],
                         "limitations": ["no dropout"]}})
    decode = analyze_extensions.decode_analysis(tmp_path / "decode")
    assert decode["aggregate_eligible"] and decode["distinct_shapes"] == 1
    assert decode["fixed_split"]["1"]["geomean_speedup"] == pytest.approx(2.01 / 1.01)
    assert decode["best_observed_baselines"]["sdpa_flash"]["wins"] == 2
    assert decode["correctness"]["record_count"] == 5
    backward = analyze_extensions.backward_analysis(tmp_path / "backward")
    assert backward["aggregates"][0]["geomean_speedup"] == pytest.approx(2.0)
    assert any(row.get("max_abs_error") == 0.01 for row in backward["raw_errors"])
    unfinished = tmp_path / "timed-out"
    extension_run(unfinished, {"summary.json": {"status": "completed"},
                               "benchmark.json": records}, outcome="timed_out")
    assert analyze_extensions.decode_analysis(unfinished)["fixed_split"] == {}
    code = analyze_extensions.main(["--decode-dir", str(tmp_path / "decode"), "--backward-dir",
                                    str(tmp_path / "backward"), "--diagnostic-dir",
                                    str(unfinished), "--output-dir", str(tmp_path / "out")])
    assert code == 0
    text = (tmp_path / "out" / "report.md").read_text()
    assert "causal+window(127,None)" in text and "Diagnostic runs" in text
    with pytest.raises(ValueError):
        analyze_extensions.median({"samples_ms": [1.0, -2.0]})


# --------------------------------------------------------------------- plots ------
def test_plot_series_come_from_recorded_evidence(tmp_path):
    from systems_for_llms_b200.attention import plot_results
    study.run_study(study.build_plan("ablation"), tmp_path / "ablation", evaluate=plausible)
    study.run_study(study.build_plan("tuning"), tmp_path / "tuning", evaluate=plausible)
    study.run_study(study.build_plan("flex_hints"), tmp_path / "hints", evaluate=plausible)
    block_benchmark.run_block_study(tmp_path / "block", evaluate=block_measurement)
    studies = plot_results.load_studies(tmp_path)
    assert {s["run"] for s in studies} == {"ablation", "tuning", "hints", "block"}
    ablation = plot_results.ablation_series(studies)
    assert len(ablation["csr_masked/csr_full"]) == 12
    assert ablation["csr_full/interval_split"]["n1024-d64-causal"]["count"] == 3
    tuning = plot_results.tuning_series(studies)
    assert all(ratios[0] == 1.0 and ratios == sorted(ratios) for ratios in tuning.values())
    blocks = plot_results.block_series(studies)
    assert blocks[("sdpa", "single_block_forward")]["n1024-d64-causal"] == pytest.approx(1.3)
    hints = plot_results.hint_series(studies)
    assert set(hints) == {"default", "contiguous_blocks"}
    assert plot_results.workload_label("n4096-d128-window") == "4K / D128 / window 128"


def test_reference_module_paths_resolve():
    import attention_lab.analyze_study
    import attention_lab.cuda_decode.study
    import attention_lab.gpu_search
    import attention_lab.run_extensions
    import attention_lab.study
    assert attention_lab.study.build_plan is study.build_plan
    assert attention_lab.run_extensions.manifest is launcher.manifest
