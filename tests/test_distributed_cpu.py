"""Distributed runner and wrappers on CPU: two gloo ranks against one process.

Mirrors the reference's strategy (distributed/tests/test_train.py,
test_optim_shard.py, test_tensor_parallel.py): every mode must reproduce the
single-process global-batch run - same batch stream, validation loss, per-step
gradient norms and final parameters.
"""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from systems_for_llms_b200.parallel.optim_shard import ShardedAdamW, assign_owners
from systems_for_llms_b200.parallel.train import validate_layout

ROOT = Path(__file__).resolve().parents[1]

CONFIG = {
    "model": {"vocab_size": 32, "context_length": 8, "d_model": 16, "num_layers": 2,
              "num_heads": 4, "d_ff": 32, "attention_backend": "sdpa"},
    "data": {"kind": "synthetic", "synthetic_tokens": 256},
    "seed": 1337, "device": "cpu", "num_threads": 1, "batch_size": 2, "max_steps": 4,
    "learning_rate": 0.001, "min_learning_rate": 0.0001, "warmup_steps": 1, "grad_clip": 0.15,
    "eval_interval": 4, "eval_batches": 4, "eval_batch_size": 1, "checkpoint_interval": 4,
}


def launch(tmp_path, name, mode, world, extra=(), config=None, timeout=180):
    config_path = tmp_path / f"{name}.json"
    config_path.write_text(json.dumps(config or CONFIG))
    out = tmp_path / name
    base = [sys.executable]
    if world > 1:
        base += ["-m", "torch.distributed.run", "--standalone", "--nnodes=1",
                 f"--nproc-per-node={world}", "--local-addr", "127.0.0.1", "--max-restarts=0",
                 "-m", "llmdist.train"]
    else:
        base += ["-m", "llmdist.train"]
    command = base + ["--config", str(config_path), "--output-dir", str(out), "--mode", mode,
                      "--global-batch-size", "4", "--warmup-steps", "1", "--save-final-state",
                      *extra]
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1", MASTER_ADDR="127.0.0.1")
    result = subprocess.run(command, cwd=ROOT, env=env, capture_output=True, text=True,
                            timeout=timeout)
    assert result.returncode == 0, result.stderr[-3000:]
    summary = json.loads((out / "summary.json").read_text())
    rows = [json.loads(line) for line in (out / "rank-0-metrics.jsonl").read_text().splitlines()]
    state = torch.load(out / "final-state.pt", weights_only=True)
    return summary, rows, state


@pytest.fixture(scope="module")
def single(tmp_path_factory):
    return launch(tmp_path_factory.mktemp("single"), "single", "single", 1,
                  ["--microbatch-size", "4"])


CASES = [("naive", []), ("ddp", []), ("ddp", ["--sync-policy", "every"]),
         ("ddp", ["--checkpointing", "block"]), ("zero1", []), ("tp", []),
         ("tp", ["--checkpointing", "block"]), ("fsdp", []), ("fsdp", ["--checkpointing", "block"])]


@pytest.mark.parametrize("mode,extra", CASES, ids=[f"{m}-{'-'.join(e) or 'plain'}" for m, e in CASES])
def test_mode_matches_single_process(tmp_path, single, mode, extra):
    ref_summary, ref_rows, ref_state = single
    summary, rows, state = launch(tmp_path, "case", mode, 2, ["--microbatch-size", "1", *extra])
    assert summary["status"] == "completed" and summary["world_size"] == 2
    assert summary["batch_stream_sha256"] == ref_summary["batch_stream_sha256"]
    assert summary["valid_loss"] == pytest.approx(ref_summary["valid_loss"], abs=2e-5)
    ref_train = [r for r in ref_rows if r["event"] == "train"]
    train = [r for r in rows if r["event"] == "train"]
    for a, b in zip(ref_train, train):
        assert b["gradient_norm"] == pytest.approx(a["gradient_norm"], rel=2e-5)
        assert b["loss"] == pytest.approx(a["loss"], rel=2e-5)
        assert a["gradient_norm"] > 0.15            # clipping active
    assert set(state["model"]) == set(ref_state["model"])
    for name, value in ref_state["model"].items():
        torch.testing.assert_close(state["model"][name], value, rtol=2e-5, atol=2e-6, msg=name)
    if mode == "zero1":
        assert summary["optimizer_state_bytes_max_rank"] < summary["optimizer_state_bytes_sum"]
        meta = state["optimizer"]["sharding"]
        assert meta["world_size"] == 2 and meta["owned_parameter_indices"]
    if mode in ("ddp", "naive"):
        ref_opt = ref_state["optimizer"]["state"]
        for index, entry in state["optimizer"]["state"].items():
            torch.testing.assert_close(entry["exp_avg"], ref_opt[index]["exp_avg"], rtol=2e-4,
                                       atol=1e-7)


def test_ddp_and_zero1_replicas_identical(tmp_path):
    _, _, ddp = launch(tmp_path, "ddp", "ddp", 2, ["--microbatch-size", "1"])
    _, _, zero = launch(tmp_path, "zero1", "zero1", 2, ["--microbatch-size", "1"])
    for name, value in ddp["model"].items():
        assert torch.equal(zero["model"][name], value), name


def test_inactive_clipping_variant(tmp_path):
    config = dict(CONFIG, grad_clip=1000.0)
    ref = launch(tmp_path, "s", "single", 1, ["--microbatch-size", "2"], config)
    got = launch(tmp_path, "d", "ddp", 2, ["--microbatch-size", "2"], config)
    for name, value in ref[2]["model"].items():
        torch.testing.assert_close(got[2]["model"][name], value, rtol=2e-5, atol=2e-6)


@pytest.mark.parametrize("args", [
    ("bogus", 2, 4, 1, "last"), ("single", 2, 4, 1, "last"), ("ddp", 1, 4, 1, "last"),
    ("ddp", 2, 5, 1, "last"), ("ddp", 2, 4, 3, "last"), ("tp", 2, 4, 1, "every"),
    ("ddp", 2, 4, 1, "sometimes"), ("ddp", 2, 4.0, 1, "last")])
def test_layout_validation_rejects(args):
    with pytest.raises(ValueError):
        validate_layout(*args)


def test_layout_validation_accumulation():
    assert validate_layout("ddp", 2, 8, 2, "last") == 2
    assert validate_layout("tp", 8, 32, 4, "last") == 8
    assert validate_layout("single", 1, 32, 4, "last") == 8


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_ownership_is_deterministic_and_balanced(world):
    sizes = [1024 * 1024] * 4 + [3 * 1024 * 1024, 2752 * 1024, 2752 * 1024, 1024, 1024] * 3
    owners, load = assign_owners(sizes, world)
    assert (owners, load) == assign_owners(sizes, world)
    assert sorted(set(owners)) == list(range(min(world, len(sizes))))[:len(set(owners))]
    assert sum(load) == sum(sizes)
    assert max(load) - min(load) <= max(sizes)


def test_sharded_adamw_single_rank_equals_adamw():
    torch.manual_seed(0)
    a = [torch.nn.Parameter(torch.randn(5, 3, dtype=torch.float64)),
         torch.nn.Parameter(torch.randn(7, dtype=torch.float64))]
    b = [torch.nn.Parameter(p.detach().clone()) for p in a]
    sharded = ShardedAdamW([{"params": [a[0]], "lr": 1e-2}, {"params": [a[1]], "weight_decay": 0}],
                           lr=1e-3)
    plain = torch.optim.AdamW([{"params": [b[0]], "lr": 1e-2}, {"params": [b[1]], "weight_decay": 0}],
                              lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    for step in range(5):
        for pa, pb in zip(a, b):
            g = torch.randn_like(pa)
            pa.grad, pb.grad = g.clone(), g.clone()
        sharded.step()
        plain.step()
    for pa, pb in zip(a, b):
        torch.testing.assert_close(pa, pb, rtol=1e-11, atol=0)
    assert sharded.local_state_bytes() > 0
    restored = ShardedAdamW([{"params": [a[0]], "lr": 1e-2}, {"params": [a[1]], "weight_decay": 0}],
                            lr=1e-3)
    restored.load_state_dict(sharded.state_dict())
    bad = sharded.state_dict()
    bad["sharding"] = dict(bad["sharding"], world_size=2)
    with pytest.raises(ValueError):
        restored.load_state_dict(bad)
    with pytest.raises(ValueError):
        ShardedAdamW([])
    with pytest.raises(ValueError):
        ShardedAdamW([a[0], a[0]])


def test_zero_grad_keeps_bucket_views():
    buffer = torch.ones(6)
    p = torch.nn.Parameter(torch.zeros(6))
    p.grad = buffer.view(6)
    optimizer = ShardedAdamW([p])
    optimizer.zero_grad(set_to_none=False)
    assert p.grad.data_ptr() == buffer.data_ptr() and buffer.sum() == 0
    optimizer.zero_grad()
    assert p.grad is None
