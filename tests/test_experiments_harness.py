"""Launcher, campaign, study runner, frozen quality target, analysis and plots (CPU only).

Nothing here starts a training run: subprocess launchers are replaced, the preflight
script is executed against a stand-in ``torch`` module and a stand-in ``subprocess.run``,
and the analysis reads hand-written rank files.
"""

import copy
import hashlib
import json
import subprocess
import sys
import types
from pathlib import Path

import pytest

from systems_for_llms_b200 import pilot
from systems_for_llms_b200.experiments import (analyze, campaign, common, launcher, plots,
                                                quality_target, study)
from systems_for_llms_b200.experiments import distributed_plan as planner

ROOT = Path(__file__).resolve().parents[1]
SMOKE_CONFIG = ROOT / "configs" / "smoke.json"


# ------------------------------------------------------------------ launcher --
def fake_tree(tmp_path: Path) -> Path:
    root = tmp_path / "tree"
    (root / "pkg" / "sub").mkdir(parents=True)
    (root / "pkg" / "a.py").write_text("A = 1\n")
    (root / "pkg" / "sub" / "b.py").write_text("B = 2\n")
    (root / "pkg" / "__pycache__").mkdir()
    (root / "pkg" / "__pycache__" / "a.cpython-312.pyc").write_bytes(b"\0")
    (root / "pkg" / "kernel.so").write_bytes(b"\0")
    (root / "configs").mkdir()
    (root / "configs" / "c.json").write_text("{}")
    (root / "notes.txt").write_text("not shipped")
    return root


def test_payload_lists_only_matching_files_with_hashes(tmp_path):
    root = fake_tree(tmp_path)
    manifest = launcher.prepare_payload(root, ("pkg/**/*.py", "configs/*.json", "pkg/*"))
    assert sorted(manifest["files"]) == ["configs/c.json", "pkg/a.py", "pkg/sub/b.py"]
    assert manifest["files"]["pkg/a.py"] == hashlib.sha256(b"A = 1\n").hexdigest()
    assert manifest["file_count"] == 3
    assert manifest["payload_sha256"] == common.json_sha256(manifest["files"])
    launcher.verify_payload(manifest)
    (root / "pkg" / "a.py").write_text("A = 2\n")
    with pytest.raises(ValueError, match="source changed"):
        launcher.verify_payload(manifest)


def test_payload_refuses_symlinks_missing_files_and_empty_sets(tmp_path):
    root = fake_tree(tmp_path)
    (root / "pkg" / "link.py").symlink_to(root / "notes.txt")
    with pytest.raises(ValueError, match="symlinks"):
        launcher.prepare_payload(root, ("pkg/**/*.py",))
    (root / "pkg" / "link.py").unlink()
    with pytest.raises(FileNotFoundError, match="missing"):
        launcher.prepare_payload(root, ("pkg/**/*.py", "bench.py"))
    with pytest.raises(ValueError, match="empty"):
        launcher.prepare_payload(root, ("nothing/*.py",))


@pytest.mark.parametrize("options, message", [
    ({"stage": "nightly", "gpus": 2}, "stage must be"),
    ({"stage": "smoke", "gpus": 3}, "gpus must be"),
    ({"stage": "smoke", "gpus": True}, "gpus must be"),
    ({"stage": "scale", "gpus": 2}, "needs 8 GPUs"),
    ({"stage": "smoke", "gpus": 2, "timeout_seconds": 0}, "finite and positive"),
    ({"stage": "smoke", "gpus": 2, "device": "tpu"}, "device must be"),
])
def test_options_are_validated(options, message):
    with pytest.raises(ValueError, match=message):
        launcher.validate_options(options)


def test_cost_estimate_is_every_case_at_its_timeout():
    checked = launcher.validate_options({"stage": "smoke", "gpus": 4})
    plan = checked["plan"]
    seconds = sum(case["timeout_seconds"] for case in plan["cases"])
    assert checked["estimate"]["worst_case_gpu_minutes"] == pytest.approx(seconds * 4 / 60)
    assert checked["estimate"]["cases"] == 10 and checked["estimate"]["allocated_gpus"] == 4
    assert checked["timeout_seconds"] == 3600.0 and checked["skip_tests"] is False


def run_preflight_script(tmp_path, fake_torch, fake_run, gpus):
    """Executes the embedded script with stand-ins for torch and subprocess.run."""
    report = tmp_path / "preflight.json"
    namespace = {"__name__": "__main__"}
    fake_subprocess = types.SimpleNamespace(run=fake_run, TimeoutExpired=subprocess.TimeoutExpired)
    saved = {name: sys.modules.get(name) for name in ("torch", "subprocess")}
    argv = sys.argv
    sys.modules["torch"], sys.modules["subprocess"] = fake_torch, fake_subprocess
    sys.argv = ["preflight.py", str(report), str(gpus)]
    try:
        exec(compile(launcher.PREFLIGHT_SCRIPT, "preflight.py", "exec"), namespace)
    finally:
        sys.argv = argv
        for name, module in saved.items():
            if module is None:
                sys.modules.pop(name, None)
            else:
                sys.modules[name] = module
    return json.loads(report.read_text())


def make_fake_torch(count=2, bf16=True, peer_error=False):
    properties = types.SimpleNamespace(name="NVIDIA B200", uuid="GPU-x", total_memory=183 << 30)

    def can_access(i, j):
        if peer_error:
            raise RuntimeError("peer query failed")
        return True

    cuda = types.SimpleNamespace(
        device_count=lambda: count, set_device=lambda index: None,
        is_bf16_supported=lambda including_emulation=False: bf16,
        get_device_properties=lambda index: properties,
        get_device_capability=lambda index: (10, 0), can_device_access_peer=can_access)
    return types.SimpleNamespace(cuda=cuda, __version__="2.11.0", version=types.SimpleNamespace(cuda="12.8"))


def test_preflight_records_devices_topology_and_peer_matrix(tmp_path, capsys):
    def fake_run(command, capture_output, text, timeout):
        return types.SimpleNamespace(returncode=0, stdout="GPU0 GPU1 NV18\n", stderr="")

    report = run_preflight_script(tmp_path, make_fake_torch(), fake_run, 2)
    assert [d["index"] for d in report["devices"]] == [0, 1]
    assert report["devices"][0]["capability"] == [10, 0]
    assert report["peer_access"] == [[True, True], [True, True]]
    assert report["nvidia_smi_topology"] == "GPU0 GPU1 NV18\n" and report["warnings"] == []
    capsys.readouterr()


def test_preflight_diagnostics_degrade_to_warnings(tmp_path, capsys):
    def fake_run(command, capture_output, text, timeout):
        if "topo" in command:
            raise OSError("nvidia-smi not found")
        raise subprocess.TimeoutExpired(command, timeout)

    report = run_preflight_script(tmp_path, make_fake_torch(peer_error=True), fake_run, 2)
    assert report["nvidia_smi_topology"] is None and report["nvidia_smi_identities"] is None
    assert report["peer_access"] == [[True, None], [None, True]]
    kinds = " ".join(report["warnings"])
    assert "unavailable" in kinds and "timeout" in kinds and "Peer-access query" in kinds
    capsys.readouterr()


def test_preflight_fails_on_too_few_gpus_or_missing_bf16(tmp_path):
    never = lambda *a, **k: pytest.fail("diagnostics ran after a fatal finding")  # noqa: E731
    with pytest.raises(RuntimeError, match="at least 4 CUDA GPUs"):
        run_preflight_script(tmp_path, make_fake_torch(count=2), never, 4)
    with pytest.raises(RuntimeError, match="lacks native BF16"):
        run_preflight_script(tmp_path, make_fake_torch(bf16=False), never, 2)


def test_junit_parser_counts_and_names_nonpassing_cases(tmp_path):
    path = tmp_path / "tests.xml"
    path.write_text("""<testsuites><testsuite tests="4" failures="1" errors="0" skipped="1">
      <testcase classname="t.a" name="ok"/>
      <testcase classname="t.a" name="bad"><failure message="x"/></testcase>
      <testcase classname="t.b" name="later"><skipped message="no gpu"/></testcase>
      <testcase classname="t.b" name="fine"/></testsuite></testsuites>""")
    report = launcher.parse_junit(path)
    assert (report["tests"], report["passed"], report["failures"], report["skipped"]) == (4, 2, 1, 1)
    assert {(c["name"], c["status"]) for c in report["nonpassing"]} == {("bad", "failure"),
                                                                      ("later", "skipped")}


@pytest.mark.parametrize("device, skipped, gate", [("cuda", 1, "failed"), ("cpu", 1, "passed"),
                                                   ("cuda", 0, "passed")])
def test_gate_requires_zero_skips_on_a_gpu_host(tmp_path, monkeypatch, device, skipped, gate):
    def fake_case(command, *, log_path, timeout, cwd, env):
        junit = next(a for a in command if a.startswith("--junitxml=")).split("=", 1)[1]
        Path(junit).write_text(f'<testsuite tests="3" failures="0" errors="0" skipped="{skipped}"/>')
        assert ("not gpu" in command) == (device == "cpu")
        return {"status": "completed", "returncode": 0}

    monkeypatch.setattr(common, "run_case", fake_case)
    report = launcher.run_gate(tmp_path, device=device, timeout=10)
    assert report["gate"] == gate and report["returncode"] == 0


def test_evidence_is_small_text_only_and_bounded(tmp_path):
    run = tmp_path / "run"
    (run / "cases" / "c1").mkdir(parents=True)
    (run / "cases" / "c1" / "summary.json").write_text('{"status": "completed"}')
    (run / "cases" / "c1" / "rank-0-metrics.jsonl").write_text('{"event": "train"}\n')
    (run / "cases" / "c1" / "final-state.pt").write_bytes(b"\0" * 1000)
    (run / "tests.log").write_text("x" * 50_000)
    (run / "outside.json").symlink_to(tmp_path / "secret.json")
    (tmp_path / "secret.json").write_text('{"token": 1}')
    evidence = launcher.collect_evidence(run, log_tail_bytes=1000)
    assert sorted(evidence["files"]) == ["cases/c1/rank-0-metrics.jsonl", "cases/c1/summary.json"]
    assert evidence["logs"]["tests.log"]["bytes"] == 50_000
    assert len(evidence["logs"]["tests.log"]["tail"]) == 1000
    assert evidence["evidence_sha256"] == common.json_sha256(
        {"files": evidence["files"], "logs": evidence["logs"]})


def test_pipeline_stops_before_the_study_when_the_gate_fails(tmp_path, monkeypatch):
    monkeypatch.setattr(launcher, "prepare_payload",
                        lambda: {"payload_sha256": "p", "files": {}, "root": str(tmp_path)})
    monkeypatch.setattr(launcher, "run_gate", lambda output, device, timeout:
                        {"gate": "failed", "failures": 2})
    monkeypatch.setattr(planner, "run_plan", lambda *a, **k: pytest.fail("study started"))
    summary = launcher.run_pipeline({"stage": "smoke", "gpus": 2, "device": "cpu"}, {},
                                    tmp_path / "launch")
    assert summary["status"] == "failed" and "test gate failed" in summary["error"]
    written = json.loads((tmp_path / "launch" / "launch-summary.json").read_text())
    assert written["status"] == "failed" and written["gpus"] == 2
    assert (tmp_path / "launch" / "evidence.json").is_file()
    with pytest.raises(FileExistsError):
        launcher.run_pipeline({"stage": "smoke", "gpus": 2, "device": "cpu"}, {},
                              tmp_path / "launch")


def test_pipeline_runs_the_stage_after_a_clean_gate(tmp_path, monkeypatch):
    monkeypatch.setattr(launcher, "prepare_payload",
                        lambda: {"payload_sha256": "p", "files": {}, "root": str(tmp_path)})
    monkeypatch.setattr(launcher, "run_gate", lambda output, device, timeout: {"gate": "passed"})
    seen = {}

    def fake_plan(plan, base, output, *, device, allocated_gpus):
        seen.update(stage=plan["stage"], device=device, gpus=allocated_gpus)
        return {"status": "completed"}

    monkeypatch.setattr(planner, "run_plan", fake_plan)
    summary = launcher.run_pipeline({"stage": "smoke", "gpus": 2, "device": "cpu"}, {},
                                    tmp_path / "launch")
    assert summary["status"] == "completed" and "preflight" not in summary
    assert seen == {"stage": "smoke", "device": "cpu", "gpus": 2}


# ------------------------------------------------------------------ campaign --
@pytest.fixture
def frozen(tmp_path, monkeypatch):
    monkeypatch.setattr(launcher, "prepare_payload", lambda: {
        "format_version": 1, "root": str(tmp_path), "file_count": 0, "files": {},
        "payload_sha256": "p"})
    config = tmp_path / "config.json"
    config.write_text(SMOKE_CONFIG.read_text())
    return campaign.prepare_campaign(config, tmp_path / "campaign"), config


def test_campaign_freezes_both_plans_and_checks_the_budget(frozen, tmp_path):
    record, config = frozen
    definition = record["definition"]
    assert record["status"] == "planned"
    assert record["definition_sha256"] == campaign.definition_hash(definition)
    assert [s["name"] for s in definition["stages"]] == ["smoke", "scale"]
    assert [len(s["plan"]["cases"]) for s in definition["stages"]] == [10, 38]
    assert definition["gpu_minutes_at_timeouts"] == pytest.approx(900 * 2 / 60 + 2400 * 8 / 60)
    assert not (tmp_path / "campaign").exists()                 # planning writes nothing
    with pytest.raises(ValueError, match="exceeds the working budget"):
        campaign.prepare_campaign(config, tmp_path / "other", budget_gpu_minutes=100)
    with pytest.raises(FileNotFoundError):
        campaign.prepare_campaign(tmp_path / "missing.json", tmp_path / "other")
    (tmp_path / "exists").mkdir()
    with pytest.raises(FileExistsError):
        campaign.prepare_campaign(config, tmp_path / "exists")


def test_smoke_gates_scale_and_nothing_is_retried(frozen, monkeypatch):
    record, _ = frozen
    calls = []

    def fake_stage(stage, base_config):
        calls.append(stage["name"])
        return {"status": "failed", "error": "test gate failed", "wall_seconds": 60.0}

    monkeypatch.setattr(campaign, "run_stage", fake_stage)
    result = campaign.execute_campaign(record)
    assert calls == ["smoke"] and result["status"] == "failed"
    assert result["stages"][0]["status"] == "failed"
    assert result["stages"][0]["gpu_minutes_used"] == pytest.approx(2.0)
    assert result["stages"][1] == {"name": "scale", "status": "not_run", "blocked_by": "smoke"}
    saved = json.loads((Path(record["definition"]["output_dir"]) / "campaign.json").read_text())
    assert saved["status"] == "failed"
    with pytest.raises(ValueError, match="only execute once"):
        campaign.execute_campaign(result)


def test_campaign_completes_when_both_stages_pass(frozen, monkeypatch):
    record, _ = frozen
    monkeypatch.setattr(campaign, "run_stage", lambda stage, base:
                        {"status": "completed", "wall_seconds": 30.0, "preflight": {"big": 1}})
    result = campaign.execute_campaign(record)
    assert result["status"] == "completed"
    assert all(stage["status"] == "completed" for stage in result["stages"])
    assert "preflight" not in result["stages"][0]["summary"]


def test_campaign_detects_changes_after_freezing(frozen, monkeypatch):
    record, config = frozen
    monkeypatch.setattr(campaign, "run_stage", lambda *a: pytest.fail("a stage ran"))
    tampered = copy.deepcopy(record)
    tampered["definition"]["stages"][1]["options"]["gpus"] = 4
    with pytest.raises(ValueError, match="definition changed"):
        campaign.execute_campaign(tampered)
    config.write_text(config.read_text() + "\n")
    with pytest.raises(RuntimeError, match="Config changed"):
        campaign.execute_campaign(record)


# --------------------------------------------------------------------- study --
def test_study_plans():
    development = study.build_plan("development")
    assert common.verify_seal(development)
    assert [job["name"] for job in development["jobs"]][-1] == "100m-1k-quality-dev"
    assert development["case_count"] == sum(job["case_count"] for job in development["jobs"])
    quality = development["jobs"][-1]
    assert quality["policies"] == ["sdpa:none:8", "sdpa:none:1", "sdpa:block:8"]
    assert quality["case_count"] == 3 and quality["overrides"]["max_steps"] == 1200
    assert development["jobs"][0]["case_count"] == 2 * 4          # full matrix, one seed
    confirmation = study.build_plan("confirmation")
    assert len(confirmation["jobs"]) == 5
    assert {job["seeds"][0] for job in confirmation["jobs"][:3]} == {2027, 2028, 2029}
    assert study.build_plan("development", synthetic=False)["jobs"][0]["config"].startswith(
        "configs/scale-")
    with pytest.raises(ValueError, match="Unknown stage"):
        study.build_plan("exploration")


def aggregate_of(rows, comparability="passed"):
    from collections import Counter
    return {"status_counts": dict(Counter(row["status"] for row in rows)),
            "comparability": {"status": comparability}, "cases": rows}


def test_job_classification():
    done = {"status": "completed"}
    oom = {"status": "failed", "failure_kind": "oom"}
    late = {"status": "timeout", "failure_kind": "timeout"}
    crash = {"status": "failed", "failure_kind": "process_error"}
    assert study.classify_job(aggregate_of([done, done]), False) == "completed"
    assert study.classify_job(aggregate_of([done, oom, late], "insufficient"), True) == \
        "completed_with_resource_limits"
    assert study.classify_job(aggregate_of([done, oom], "insufficient"), False) == "blocked"
    assert study.classify_job(aggregate_of([done, crash], "insufficient"), True) == "blocked"
    assert study.classify_job(aggregate_of([done, oom], "failed"), True) == "blocked"
    assert study.classify_job(aggregate_of([done, {"status": "invalid_output"}],
                                           "insufficient"), True) == "blocked"


def small_stage(jobs):
    return common.seal({"format_version": 1, "stage": "development", "jobs": jobs})


def test_stage_runs_jobs_in_order_and_a_blocked_job_stops_it(tmp_path, monkeypatch):
    monkeypatch.setattr(pilot, "source_identity", lambda: {"python_source_sha256": "aa" * 32})
    monkeypatch.setattr(study, "source_identity", lambda: {"python_source_sha256": "aa" * 32})
    job = dict(config="configs/smoke.json", microbatches=[2], effective_batch_size=4, seeds=[1],
               warmup_steps=2, case_timeout_seconds=30, job_timeout_seconds=60, overrides={},
               policies=["sdpa:none:2"], case_count=1)
    plan = small_stage([dict(job, name="first", allow_resource_limits=True),
                        dict(job, name="second", allow_resource_limits=False),
                        dict(job, name="third", allow_resource_limits=False)])
    outcomes = iter([aggregate_of([{"status": "completed"},
                                   {"status": "failed", "failure_kind": "oom"}], "insufficient"),
                     aggregate_of([{"status": "failed", "failure_kind": "oom"}], "insufficient")])
    roots = []

    def execute(root):
        roots.append(root.name)
        assert (root / "manifest.json").is_file()
        return next(outcomes)

    record = study.run_stage(plan, tmp_path / "study", device="cpu", execute_job=execute)
    assert roots == ["first", "second"]
    assert [job["status"] for job in record["jobs"]] == ["completed_with_resource_limits", "blocked"]
    assert record["status"] == "blocked"
    assert json.loads((tmp_path / "study" / "study.json").read_text()) == record
    with pytest.raises(FileExistsError):
        study.run_stage(plan, tmp_path / "study", device="cpu", execute_job=execute)


def test_stage_refuses_a_modified_plan_and_quality_stages_need_a_target(tmp_path):
    plan = study.build_plan("development")
    plan["jobs"][0]["case_timeout_seconds"] = 1
    with pytest.raises(ValueError, match="modified"):
        study.run_stage(plan, tmp_path / "a")
    with pytest.raises(ValueError, match="frozen target"):
        study.run_stage(study.build_plan("quality-confirmation"), tmp_path / "b")


# ------------------------------------------------------------ quality target --
@pytest.mark.parametrize("value, expected", [(2.349999, "2.35"), (2.35, "2.35"),
                                             (2.3500000000000001, "2.35"), (2.3500001, "2.40"),
                                             (2.0, "2.00"), (0.1 + 0.2, "0.35")])
def test_ceiling_is_exact_decimal_arithmetic(value, expected):
    """0.1 + 0.2 is 0.30000000000000004 in binary: the decimal ceiling must move up a step,
    while a value that prints as a multiple of the step must stay."""
    assert quality_target.ceiling_to_step(value) == expected


def test_ceiling_rejects_a_nonpositive_step():
    with pytest.raises(ValueError):
        quality_target.ceiling_to_step(1.0, "0")


@pytest.fixture
def development(tmp_path, monkeypatch):
    monkeypatch.setattr(pilot, "source_identity", lambda: {"python_source_sha256": "ab" * 32})
    from systems_for_llms_b200.config import load_config
    from dataclasses import replace
    plan = pilot.make_plan(replace(load_config(SMOKE_CONFIG), max_steps=6), microbatches=[2],
                           effective_batch_size=4, seeds=[1], warmup_steps=2, device="cpu",
                           policies=["sdpa:none:2", "sdpa:block:2"])
    root = pilot.write_plan(plan, tmp_path / "dev")
    losses = {}
    for index, case in enumerate(plan["cases"]):
        run = root / "runs" / case["case_id"]
        run.mkdir(parents=True)
        loss = 2.31 + 0.03 * index
        losses[case["case_id"]] = loss
        events = [{"event": "train", "step": 4, "train_seconds": 8.0},
                  {"event": "eval", "step": 4, "valid_loss": loss + 0.2},
                  {"event": "train", "step": 6, "train_seconds": 12.5},
                  {"event": "eval", "step": 6, "valid_loss": loss}]
        (run / "metrics.jsonl").write_text("".join(json.dumps(e) + "\n" for e in events))
    rows = [{"case_id": case["case_id"], "status": "completed", "batch_stream_sha256": "s" * 64,
             "data_identity_sha256": "d" * 64} for case in plan["cases"]]
    aggregate = {"plan_sha256": plan["plan_sha256"], "comparability": {"status": "passed"},
                 "cases": rows}
    (root / "aggregate.json").write_text(json.dumps(aggregate))
    return root, aggregate, losses


def test_target_is_frozen_once_and_revalidates(development, tmp_path):
    root, aggregate, losses = development
    output = tmp_path / "frozen-target.json"
    record = quality_target.freeze_target(root / "aggregate.json", output, target_step=6)
    assert record["target"]["max_development_loss"] == max(losses.values())
    assert record["target"]["target_validation_loss"] == "2.35"
    assert set(record["input_sha256"]) == {"aggregate.json", "manifest.json",
                                           *(f"runs/{c}/metrics.jsonl" for c in losses)}
    with pytest.raises(FileExistsError):
        quality_target.freeze_target(root / "aggregate.json", output, target_step=6)
    assert quality_target.validate_frozen(output, check_source=False)["target"] == record["target"]


def test_tampering_is_detected(development, tmp_path):
    root, aggregate, losses = development
    output = tmp_path / "frozen-target.json"
    quality_target.freeze_target(root / "aggregate.json", output, target_step=6)
    edited = json.loads(output.read_text())
    edited["target"]["target_validation_loss"] = "2.60"
    output.write_text(json.dumps(edited))
    with pytest.raises(ValueError, match="was modified"):
        quality_target.validate_frozen(output, check_source=False)
    output.unlink()
    quality_target.freeze_target(root / "aggregate.json", output, target_step=6)
    victim = root / "runs" / next(iter(losses)) / "metrics.jsonl"
    victim.write_text(victim.read_text().replace("2.31", "2.11"))
    with pytest.raises(ValueError, match="evidence changed"):
        quality_target.validate_frozen(output, check_source=False)


def test_target_needs_comparable_complete_development_runs(development):
    root, aggregate, _ = development
    broken = copy.deepcopy(aggregate)
    broken["comparability"]["status"] = "insufficient"
    with pytest.raises(ValueError, match="comparability"):
        quality_target.derive_target(broken, root / "runs", target_step=6)
    broken = copy.deepcopy(aggregate)
    broken["cases"][0]["status"] = "failed"
    with pytest.raises(ValueError, match="must complete"):
        quality_target.derive_target(broken, root / "runs", target_step=6)
    broken = copy.deepcopy(aggregate)
    broken["cases"][1]["batch_stream_sha256"] = "t" * 64
    with pytest.raises(ValueError, match="same batches"):
        quality_target.derive_target(broken, root / "runs", target_step=6)
    with pytest.raises(ValueError, match="exactly one evaluation"):
        quality_target.derive_target(aggregate, root / "runs", target_step=5)


def test_time_to_target_is_the_first_evaluation_at_or_below(development):
    root, _, losses = development
    case_id, loss = next(iter(losses.items()))
    hit = quality_target.time_to_target(root / "runs" / case_id, loss + 0.2)
    assert hit == {"step": 4, "valid_loss": loss + 0.2, "train_seconds": 8.0}
    assert quality_target.time_to_target(root / "runs" / case_id, loss)["step"] == 6
    assert quality_target.time_to_target(root / "runs" / case_id, loss - 0.5) is None


# ------------------------------------------------------------------ analysis --
def evidence_row(mode, world, seed, rate, *, ckpt="none", peak=10 << 30, state=2 << 30,
                 provenance="same", status="completed"):
    case = planner._case(mode, world, checkpointing=ckpt, seed=seed)
    return dict(case, status=status, tokens_per_second=rate, peak_cuda_allocated_bytes=peak,
                optimizer_state_bytes_max_rank=state, valid_loss=3.0 + 0.001 * world,
                active_gpu_seconds_per_update=world * 32768 / rate,
                measured_train_seconds=55 * 32768 / rate, provenance_sha256=provenance,
                checkpoint_comparison_provenance_sha256=provenance)


def study_rows():
    rows = []
    for seed, scale in ((2027, 1.0), (2028, 1.02), (2029, 0.98)):
        rows += [evidence_row("single", 1, seed, 100e3 * scale),
                 evidence_row("ddp", 8, seed, 600e3 * scale),
                 evidence_row("zero1", 8, seed, 540e3 * scale, peak=8 << 30, state=256 << 20),
                 evidence_row("fsdp", 8, seed, 300e3 * scale, peak=6 << 30, state=256 << 20),
                 evidence_row("ddp", 8, seed, 330e3 * scale, ckpt="block", peak=6 << 30),
                 evidence_row("tp", 8, seed, 80e3 * scale, peak=4 << 30)]
    return rows


def test_policy_statistics_summarise_across_seeds():
    rows = study_rows() + [evidence_row("naive", 8, 2027, 1.0, status="failed")]
    planner.add_scaling_metrics(rows, 8)
    entries = analyze.policy_statistics(rows)
    assert len(entries) == 6
    ddp = next(e for e in entries if e["policy"]["mode"] == "ddp"
               and e["policy"]["checkpointing"] == "none")
    assert ddp["seeds"] == [2027, 2028, 2029]
    assert ddp["metrics"]["tokens_per_second"]["mean"] == pytest.approx(600e3)
    assert ddp["metrics"]["tokens_per_second"]["sample_sd"] == pytest.approx(12e3)
    assert ddp["metrics"]["strong_scaling_efficiency"]["median"] == pytest.approx(0.75)
    with pytest.raises(ValueError, match="more than one case for a seed"):
        analyze.policy_statistics(rows + [evidence_row("ddp", 8, 2027, 1.0)])


def test_paired_comparisons_are_within_seed_and_need_matching_provenance():
    rows = study_rows()
    rows[1]["provenance_sha256"] = "other"                    # ddp, seed 2027: different data
    groups = {g["comparison"]: g for g in analyze.paired_comparisons(rows)}
    assert set(groups) == {"ddp_vs_single", "tp_vs_single", "zero1_vs_ddp", "fsdp_vs_ddp",
                           "ddp_block_vs_none"}
    assert groups["ddp_vs_single"]["seeds"] == [2028, 2029]   # the mismatched pair is dropped
    assert groups["zero1_vs_ddp"]["seeds"] == [2028, 2029]
    assert groups["tp_vs_single"]["paired_count"] == 3
    assert groups["ddp_vs_single"]["metrics"]["throughput_ratio"]["median"] == pytest.approx(6.0)
    assert groups["ddp_vs_single"]["metrics"]["strong_scaling_efficiency"]["median"] == \
        pytest.approx(0.75)
    assert groups["zero1_vs_ddp"]["metrics"]["optimizer_state_ratio"]["median"] == \
        pytest.approx(0.125)
    assert groups["fsdp_vs_ddp"]["metrics"]["allocated_memory_ratio"]["median"] == pytest.approx(0.6)
    block = groups["ddp_block_vs_none"]
    assert block["denominator"]["checkpointing"] == "none" and block["seeds"] == [2027, 2028, 2029]
    assert block["metrics"]["throughput_ratio"]["median"] == pytest.approx(0.55)


def test_cost_rows_from_launch_and_campaign_records(tmp_path):
    stage = tmp_path / "campaign" / "smoke"
    (stage / "study").mkdir(parents=True)
    common.write_json(stage / "launch-summary.json", {
        "stage": "smoke", "gpus": 2, "status": "completed", "wall_seconds": 300.0,
        "estimate": {"worst_case_gpu_minutes": 44.0}})
    cases = [{"active_gpu_seconds_measured": 30.0}, {"active_gpu_seconds_measured": 90.0},
             {"status": "failed"}]
    rows = analyze.cost_rows(stage / "study", cases)
    assert len(rows) == 1
    assert rows[0]["gpu_minutes_used"] == pytest.approx(10.0)
    assert rows[0]["gpu_minutes_at_timeouts"] == 44.0
    assert rows[0]["active_gpu_minutes_measured"] == pytest.approx(2.0)
    common.write_json(tmp_path / "campaign" / "campaign.json", {
        "definition": {"stages": [
            {"name": "smoke", "output_dir": str(stage), "options": {"gpus": 2},
             "estimate": {"worst_case_gpu_minutes": 44.0}},
            {"name": "scale", "output_dir": str(tmp_path / "campaign" / "scale"),
             "options": {"gpus": 8}, "estimate": {"worst_case_gpu_minutes": 1216.0}}]},
        "stages": [{"name": "smoke", "status": "completed"},
                   {"name": "scale", "status": "not_run"}]})
    rows = analyze.cost_rows(stage / "study", cases)
    assert [(r["stage"], r["status"]) for r in rows] == [("smoke", "completed"), ("scale", "not_run")]
    assert rows[1]["gpu_minutes_used"] is None and rows[1]["allocated_gpus"] == 8
    assert rows[1]["gpu_minutes_at_timeouts"] == 1216.0
    assert "active_gpu_minutes_measured" not in rows[1]
    common.write_json(stage / "launch-summary.json", {"stage": "smoke", "gpus": 2,
                                                      "wall_seconds": -1.0})
    with pytest.raises(ValueError, match="finite and positive"):
        analyze.cost_rows(stage / "study")


def test_report_renders_policies_pairs_cost_and_failures():
    rows = study_rows() + [evidence_row("naive", 8, 2027, 1.0, status="timeout")]
    rows[-1]["error"] = "case exceeded 240 seconds"
    planner.add_scaling_metrics(rows, 8)
    summary = {"stage": "confirmation", "plan_sha256": "f" * 64, "status": "failed",
               "timing_note": analyze.TIMING_NOTE, "cost_note": analyze.COST_NOTE, "cases": rows,
               "policies": analyze.policy_statistics(rows),
               "paired": analyze.paired_comparisons(rows),
               "cost": [{"stage": "scale", "status": "failed", "allocated_gpus": 8,
                         "wall_seconds": 600.0, "gpu_minutes_used": 80.0,
                         "gpu_minutes_at_timeouts": 1216.0, "active_gpu_minutes_measured": 12.5}],
               "input_sha256": {"aggregate.json": "a" * 64, "plan.json": "b" * 64}}
    text = analyze.render_report(summary)
    assert "| DDP | 8 | 1024 | none | 4 | 3 | 600,000 |" in text
    assert "| zero1_vs_ddp | 8 | 3 | 0.900 |" in text
    assert "| scale | failed | 8 | 600.0 | 80.00 | 1,216.0 | 12.50 |" in text
    assert "timeout case exceeded 240 seconds" in text
    series = analyze.plot_series(summary)
    assert series[("ddp", "none")] == [(8, pytest.approx(600e3))]
    assert series[("single", "none")] == [(1, pytest.approx(100e3))]


def test_summary_refuses_an_aggregate_of_another_plan(tmp_path):
    plan = planner.build_plan("smoke")
    common.write_json(tmp_path / "plan.json", plan)
    common.write_json(tmp_path / "aggregate.json", {"plan_sha256": "0" * 64, "cases": [],
                                                    "status": "failed", "allocated_gpus": 2})
    with pytest.raises(ValueError, match="different plan"):
        analyze.build_summary(tmp_path)


# --------------------------------------------------------------------- plots --
def test_plot_series_and_curves(tmp_path):
    aggregate = {"cases": [
        {"status": "completed", "attention_backend": "sdpa", "activation_checkpointing": "none",
         "batch_size": 8, "seed": 1, "tokens_per_second": 100.0,
         "peak_cuda_allocated_bytes": 3 << 30},
        {"status": "failed", "attention_backend": "eager", "activation_checkpointing": "none",
         "batch_size": 8, "seed": 1},
        {"status": "completed", "attention_backend": "eager", "activation_checkpointing": "block",
         "batch_size": 1, "seed": 1, "tokens_per_second": 10.0, "peak_cuda_allocated_bytes": None}]}
    series = plots.pilot_series(aggregate)
    assert [row["label"] for row in series] == ["eager/block/mb1/s1", "sdpa/none/mb8/s1"]
    assert series[1]["peak_gib"] == 3.0 and series[0]["peak_gib"] is None
    run = tmp_path / "job" / "runs" / "case-a"
    run.mkdir(parents=True)
    events = [{"event": "train", "step": 1, "train_seconds": 1.5},
              {"event": "eval", "step": 1, "valid_loss": 3.0},
              {"event": "train", "step": 2, "train_seconds": 3.0},
              {"event": "eval", "step": 2, "valid_loss": 2.5}]
    (run / "metrics.jsonl").write_text("".join(json.dumps(e) + "\n" for e in events))
    assert plots.quality_curves(tmp_path / "job") == {"case-a": [(1.5, 3.0), (3.0, 2.5)]}


def test_plots_are_written_when_matplotlib_is_present(tmp_path):
    pytest.importorskip("matplotlib")
    aggregate = {"cases": [{"status": "completed", "attention_backend": "sdpa",
                            "activation_checkpointing": "none", "batch_size": 8, "seed": 1,
                            "tokens_per_second": 100.0, "peak_cuda_allocated_bytes": 1 << 30}]}
    path = tmp_path / "aggregate.json"
    path.write_text(json.dumps(aggregate))
    assert plots.plot_pilot(path, tmp_path / "pilot.png").stat().st_size > 0
