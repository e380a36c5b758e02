"""Trainer behaviour: golden values, resume, cadence, accumulation (CPU)."""

import dataclasses
import json
from pathlib import Path

import pytest
import torch

from systems_for_llms_b200 import train as trainer
from systems_for_llms_b200.config import load_config
from systems_for_llms_b200.data import load_data

ROOT = Path(__file__).resolve().parents[1]


def metrics(path):
    return [json.loads(line) for line in (path / "metrics.jsonl").read_text().splitlines()]


def test_smoke_config_reproduces_reference_values(tmp_path):
    """configs/smoke.json on CPU: the numbers the reference produces from the same
    seed (construction order and initialisers are identical)."""
    config = load_config(ROOT / "configs" / "smoke.json")
    summary = trainer.run(config, tmp_path / "run")
    assert summary["status"] == "completed" and summary["step"] == 20
    assert summary["tokens_seen"] == 320
    assert summary["valid_loss"] == pytest.approx(3.8301379680633545, rel=1e-6)
    first = [row for row in metrics(tmp_path / "run") if row["event"] == "train"][0]
    assert first["loss"] == pytest.approx(3.3269598484039307, rel=1e-6)
    assert first["gradient_norm"] == pytest.approx(1.4130134582519531, rel=1e-6)
    assert first["learning_rate"] == pytest.approx(0.0015)
    assert first["batch_start_sha256"].startswith("5a68da16")
    for name in ("metadata.json", "metrics.jsonl", "summary.json", "checkpoint.pt"):
        assert (tmp_path / "run" / name).exists()
    checkpoint = torch.load(tmp_path / "run" / "checkpoint.pt", weights_only=True)
    assert {"format_version", "config", "data_identity", "source_sha256", "device_type", "step",
            "model", "optimizer", "sampler_rng_state", "torch_rng_state"} <= set(checkpoint)
    assert len(checkpoint["model"]) == 12
    state = checkpoint["optimizer"]["state"][0]
    assert set(state) == {"step", "exp_avg", "exp_avg_sq"}


@pytest.mark.parametrize("accum,ckpt", [(1, "none"), (3, "block")])
def test_resume_is_bit_exact(tmp_path, tiny_config, accum, ckpt):
    config = dataclasses.replace(
        tiny_config, grad_accum_steps=accum, max_steps=6, checkpoint_interval=3,
        model=dataclasses.replace(tiny_config.model, activation_checkpointing=ckpt))
    trainer.run(config, tmp_path / "straight")
    trainer.run(config, tmp_path / "first", stop_after=3)
    paused = json.loads((tmp_path / "first" / "summary.json").read_text())
    assert paused["status"] == "paused" and paused["step"] == 3
    trainer.run(config, tmp_path / "second", resume=tmp_path / "first" / "checkpoint.pt")
    a = torch.load(tmp_path / "straight" / "checkpoint.pt", weights_only=True)
    b = torch.load(tmp_path / "second" / "checkpoint.pt", weights_only=True)
    for name in a["model"]:
        assert torch.equal(a["model"][name], b["model"][name]), name
    for index, state in a["optimizer"]["state"].items():
        for key, value in state.items():
            assert torch.equal(value, b["optimizer"]["state"][index][key])
    assert torch.equal(a["sampler_rng_state"], b["sampler_rng_state"])
    assert torch.equal(a["torch_rng_state"], b["torch_rng_state"])


def test_eval_cadence_does_not_change_training(tmp_path, tiny_config):
    trainer.run(dataclasses.replace(tiny_config, eval_interval=1), tmp_path / "often")
    trainer.run(dataclasses.replace(tiny_config, eval_interval=4), tmp_path / "rare")
    a = torch.load(tmp_path / "often" / "checkpoint.pt", weights_only=True)["model"]
    b = torch.load(tmp_path / "rare" / "checkpoint.pt", weights_only=True)["model"]
    assert all(torch.equal(a[k], b[k]) for k in a)


def test_eval_is_batch_size_independent_and_rng_free(tiny_config):
    from dataclasses import asdict
    from systems_for_llms_b200.models.transformer import TransformerLM
    torch.manual_seed(0)
    model = TransformerLM(**asdict(tiny_config.model), dtype=torch.float32)
    _, valid, _ = load_data(tiny_config)
    device = torch.device("cpu")
    before = torch.get_rng_state()
    one = trainer.evaluate(model, valid, dataclasses.replace(tiny_config, eval_batch_size=1,
                                                             eval_batches=4), device)
    two = trainer.evaluate(model, valid, dataclasses.replace(tiny_config, eval_batch_size=2,
                                                             eval_batches=2), device)
    assert torch.equal(before, torch.get_rng_state())
    assert one == pytest.approx(two, rel=1e-6)


def test_resume_rejects_changed_config_and_data(tmp_path, tiny_config):
    trainer.run(tiny_config, tmp_path / "base", stop_after=2)
    checkpoint = tmp_path / "base" / "checkpoint.pt"
    with pytest.raises(ValueError, match="configuration"):
        trainer.run(dataclasses.replace(tiny_config, learning_rate=2e-3), tmp_path / "a",
                    resume=checkpoint)
    other_data = dataclasses.replace(tiny_config, data=dataclasses.replace(
        tiny_config.data, synthetic_tokens=300))
    with pytest.raises(ValueError):
        trainer.run(other_data, tmp_path / "b", resume=checkpoint)
    # cadence may change
    trainer.run(dataclasses.replace(tiny_config, eval_interval=1), tmp_path / "c",
                resume=checkpoint)


def test_failed_setup_writes_summary_and_never_overwrites(tmp_path, tiny_config):
    bad = dataclasses.replace(tiny_config, precision="bf16")   # bf16 needs CUDA
    with pytest.raises(ValueError):
        trainer.run(bad, tmp_path / "bad")
    summary = json.loads((tmp_path / "bad" / "summary.json").read_text())
    assert summary["status"] == "failed" and summary["phase"] == "setup"
    with pytest.raises(FileExistsError):
        trainer.run(tiny_config, tmp_path / "bad")


def test_accumulation_equals_full_batch(tmp_path, tiny_config):
    full = dataclasses.replace(tiny_config, batch_size=4, grad_accum_steps=1)
    split = dataclasses.replace(tiny_config, batch_size=1, grad_accum_steps=4)
    trainer.run(full, tmp_path / "full")
    trainer.run(split, tmp_path / "split")
    rows_a = [r for r in metrics(tmp_path / "full") if r["event"] == "train"]
    rows_b = [r for r in metrics(tmp_path / "split") if r["event"] == "train"]
    for a, b in zip(rows_a, rows_b):
        assert a["batch_start_sha256"] == b["batch_start_sha256"]
        assert a["gradient_norm"] == pytest.approx(b["gradient_norm"], rel=2e-5)
        assert a["gradient_norm"] > tiny_config.grad_clip   # clipping is active
    a = torch.load(tmp_path / "full" / "checkpoint.pt", weights_only=True)["model"]
    b = torch.load(tmp_path / "split" / "checkpoint.pt", weights_only=True)["model"]
    for name in a:
        torch.testing.assert_close(a[name], b[name], rtol=2e-5, atol=2e-6)


def test_learning_rate_schedule(tiny_config):
    config = dataclasses.replace(tiny_config, max_steps=10, warmup_steps=2, learning_rate=1.0,
                                 min_learning_rate=0.1)
    assert trainer.learning_rate(0, config) == pytest.approx(0.5)
    assert trainer.learning_rate(1, config) == pytest.approx(1.0)
    assert trainer.learning_rate(2, config) == pytest.approx(1.0)
    assert trainer.learning_rate(9, config) == pytest.approx(0.1)


def test_invalid_stop_after(tmp_path, tiny_config):
    with pytest.raises(ValueError):
        trainer.run(tiny_config, tmp_path / "x", stop_after=0)
