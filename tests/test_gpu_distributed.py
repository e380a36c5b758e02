"""Peer-memory collectives and fused data-parallel modes on two B200s."""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = Path(__file__).resolve().parents[1]

CONFIG = {
    "model": {"vocab_size": 1000, "context_length": 128, "d_model": 128, "num_layers": 2,
              "num_heads": 2, "d_ff": 352, "attention_backend": "sdpa"},
    "data": {"kind": "synthetic", "synthetic_tokens": 20000},
    "seed": 1337, "device": "cuda", "precision": "bf16", "num_threads": 1, "batch_size": 2,
    "max_steps": 4, "learning_rate": 0.001, "min_learning_rate": 0.0001, "warmup_steps": 1,
    "grad_clip": 0.5, "eval_interval": 4, "eval_batches": 4, "eval_batch_size": 1,
    "checkpoint_interval": 4,
}
PORT = 29600


def launch(tmp_path, name, mode, world, extra=()):
    global PORT
    PORT += 1
    config_path = tmp_path / f"{name}.json"
    config_path.write_text(json.dumps(CONFIG))
    out = tmp_path / name
    command = [sys.executable]
    if world > 1:
        command += ["-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                    "--master-addr", "127.0.0.1", "--master-port", str(PORT), "--max-restarts=0",
                    "-m", "llmdist.train"]
    else:
        command += ["-m", "llmdist.train"]
    command += ["--config", str(config_path), "--output-dir", str(out), "--mode", mode,
                "--global-batch-size", "8", "--warmup-steps", "1", "--save-final-state", *extra]
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1", NCCL_NVLS_ENABLE="0")
    result = subprocess.run(command, cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stderr[-3000:]
    summary = json.loads((out / "summary.json").read_text())
    meta = json.loads((out / "rank-0-metadata.json").read_text())
    state = torch.load(out / "final-state.pt", weights_only=True)
    return summary, meta, state


@pytest.fixture(scope="module")
def single(tmp_path_factory):
    return launch(tmp_path_factory.mktemp("single"), "single", "single", 1,
                  ["--microbatch-size", "4"])


@pytest.mark.parametrize("mode,extra", [("ddp", []), ("ddp", ["--sync-policy", "every"]),
                                        ("ddp", ["--bucket-cap-mb", "1"]), ("zero1", []),
                                        ("naive", []), ("tp", []), ("tp", ["--checkpointing", "block"]),
                                        ("fsdp", []), ("fsdp", ["--checkpointing", "block"])])
def test_two_gpu_mode_matches_single(tmp_path, single, mode, extra):
    ref_summary, ref_meta, ref_state = single
    summary, meta, state = launch(tmp_path, "case", mode, 2, ["--microbatch-size", "2", *extra])
    assert summary["batch_stream_sha256"] == ref_summary["batch_stream_sha256"]
    assert summary["valid_loss"] == pytest.approx(ref_summary["valid_loss"], rel=2e-2)
    if mode in ("ddp", "zero1", "tp", "fsdp"):
        assert meta["execution_path"] == "sm_100a fused engine"
        assert meta["gradient_reduction"] == "peer-memory kernels over NVLink"
    for name, value in ref_state["model"].items():
        # bf16 compute: different reduction orders move low-order bits of the update
        torch.testing.assert_close(state["model"][name], value, rtol=0, atol=5e-3, msg=name)
    if mode in ("zero1", "fsdp"):
        assert summary["optimizer_state_bytes_max_rank"] * 2 <= summary["optimizer_state_bytes_sum"] + 64


def test_two_gpu_tensor_parallel_fused_gemm_allreduce_matches_single(tmp_path, monkeypatch):
    """d_model of 256 lets the row-parallel products and the column-parallel input
    gradients run as one GEMM + all-reduce kernel each, issued by the native block
    runner; the result must match a single GPU like every other mode."""
    wide = dict(CONFIG, model=dict(CONFIG["model"], d_model=256, num_heads=4, d_ff=704))
    monkeypatch.setitem(globals(), "CONFIG", wide)
    ref_summary, _, ref_state = launch(tmp_path, "one", "single", 1, ["--microbatch-size", "4"])
    for extra in ([], ["--checkpointing", "block"]):
        summary, meta, state = launch(tmp_path, "tp" + str(len(extra)), "tp", 2,
                                      ["--microbatch-size", "2", *extra])
        assert meta["tensor_parallel_reduction"].startswith("inside the GEMM kernels")
        assert summary["batch_stream_sha256"] == ref_summary["batch_stream_sha256"]
        assert summary["valid_loss"] == pytest.approx(ref_summary["valid_loss"], rel=2e-2)
        for name, value in ref_state["model"].items():
            torch.testing.assert_close(state["model"][name], value, rtol=0, atol=5e-3, msg=name)


@pytest.mark.parametrize("one_shot", ["1", "0"])
def test_comm_kernels_against_nccl(tmp_path, one_shot):
    """``one_shot`` picks the variant of the fused GEMM + all-reduce: both ranks finish
    every row (the default for two ranks) or tiles owned round-robin (larger groups)."""
    script = ROOT / "tests" / "helpers" / "comm_check.py"
    global PORT
    PORT += 1
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
               "--master-addr", "127.0.0.1", "--master-port", str(PORT), str(script),
               str(tmp_path / "out.json")]
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0", SFL_TP_ONE_SHOT=one_shot)
    result = subprocess.run(command, cwd=ROOT, env=env, capture_output=True, text=True, timeout=300)
    assert result.returncode == 0, result.stderr[-3000:]
    out = json.loads((tmp_path / "out.json").read_text())
    assert out["allreduce_maxerr"] < 1e-6 and out["replicas_equal"]
    assert out["norm"] == pytest.approx(out["norm_ref"], rel=1e-5)
    assert out["zero_param_maxerr"] < 2e-6 and out["zero_shadow_ok"]
    assert out["allgather_ok"] and out["tp_reduce_maxerr"] < 1e-6
    assert out["tp_fused_equal"] and out["tp_fused_replicas_equal"]
    assert out["tp_fused_maxerr"] < 0.15      # bf16 partials of a K = 384 reduction, |x| ~ 1
    assert out["timeout_status"] == 5 and out["recovered_after_timeout"]
