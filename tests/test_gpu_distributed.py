"""Peer-memory collectives and fused parallel modes against one GPU, on 2, 4 and 8 B200s.

Parity is checked where a wrong run cannot hide: the per-step loss and gradient norm
of every update, and the parameter UPDATE (final - initial) tensor by tensor with a
relative bound.  (Four AdamW steps at lr <= 1e-3 move a weight by at most a few 1e-3,
so an absolute tolerance on the final parameters would also accept a run that never
updated.)  Cases for more GPUs than the machine has are skipped.
"""

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]
ROOT = Path(__file__).resolve().parents[1]

SMALL = {"vocab_size": 1000, "context_length": 128, "d_model": 128, "num_layers": 2,
         "num_heads": 2, "d_ff": 352, "attention_backend": "sdpa"}
# eight heads and a feed-forward width divisible by eight ranks; d_model is a multiple of 256,
# so tensor-parallel products can run as one GEMM + all-reduce kernel
WIDE = {"vocab_size": 1000, "context_length": 128, "d_model": 512, "num_layers": 2,
        "num_heads": 8, "d_ff": 1408, "attention_backend": "sdpa"}
TRAIN = {
    "data": {"kind": "synthetic", "synthetic_tokens": 20000},
    "seed": 1337, "device": "cuda", "precision": "bf16", "num_threads": 1, "batch_size": 2,
    "max_steps": 4, "learning_rate": 0.001, "min_learning_rate": 0.0001, "warmup_steps": 1,
    "grad_clip": 0.5, "eval_interval": 4, "eval_batches": 8, "eval_batch_size": 1,
    "checkpoint_interval": 4,
}
PORT = 29600


def gpus() -> int:
    return torch.cuda.device_count() if torch.cuda.is_available() else 0


def need(world: int) -> None:
    if gpus() < world:
        pytest.skip(f"needs {world} CUDA devices")


def launch(tmp_path, name, mode, world, model, extra=(), env_extra=None):
    global PORT
    PORT += 1
    config_path = tmp_path / f"{name}.json"
    config_path.write_text(json.dumps(dict(TRAIN, model=model)))
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
    env = dict(os.environ, PYTHONPATH=str(ROOT), OMP_NUM_THREADS="1", NCCL_NVLS_ENABLE="0",
               **(env_extra or {}))
    result = subprocess.run(command, cwd=ROOT, env=env, capture_output=True, text=True, timeout=420)
    assert result.returncode == 0, result.stderr[-3000:]
    rows = [json.loads(line) for line in (out / "rank-0-metrics.jsonl").read_text().splitlines()]
    return {"summary": json.loads((out / "summary.json").read_text()),
            "meta": json.loads((out / "rank-0-metadata.json").read_text()),
            "train": [row for row in rows if row["event"] == "train"],
            "initial": torch.load(out / "initial-state.pt", weights_only=True)["model"],
            "final": torch.load(out / "final-state.pt", weights_only=True)["model"]}


# Relative L2 bound on a tensor's update.  Data-parallel modes reduce fp32 gradients and differ
# from one GPU only in summation order; tensor parallelism sums bf16 partial activations and
# the sharded modes round at different points, and Adam's normalised early steps amplify that
# for near-zero gradients.  A run that never updated (or updated with the wrong sign) is at 1.
UPDATE_TOLERANCE = {"tp": 0.12, "fsdp": 0.08}


def assert_same_training(run, reference, *, update_tolerance=5e-2):
    assert run["summary"]["batch_stream_sha256"] == reference["summary"]["batch_stream_sha256"]
    assert len(run["train"]) == len(reference["train"]) == TRAIN["max_steps"]
    for ours, theirs in zip(run["train"], reference["train"]):
        assert ours["loss"] == pytest.approx(theirs["loss"], rel=1e-2), ours["step"]
        assert ours["gradient_norm"] == pytest.approx(theirs["gradient_norm"], rel=1e-2), ours["step"]
    assert run["summary"]["valid_loss"] == pytest.approx(reference["summary"]["valid_loss"], rel=5e-3)
    for name, start in reference["initial"].items():
        assert torch.equal(run["initial"][name], start), f"{name}: different initial parameters"
        expected = reference["final"][name].double() - start.double()
        actual = run["final"][name].double() - run["initial"][name].double()
        size = expected.norm().item()
        assert size > 0, f"{name} never moved in the reference run"
        assert (actual - expected).norm().item() <= update_tolerance * size, name


_single_cache: dict = {}


def single_run(tmp_path_factory, model_name: str):
    if model_name not in _single_cache:
        model = SMALL if model_name == "small" else WIDE
        _single_cache[model_name] = launch(tmp_path_factory.mktemp(f"single-{model_name}"),
                                           "single", "single", 1, model, ["--microbatch-size", "4"])
    return _single_cache[model_name]


@pytest.mark.parametrize("mode,extra", [("ddp", []), ("ddp", ["--sync-policy", "every"]),
                                        ("ddp", ["--bucket-cap-mb", "1"]), ("zero1", []),
                                        ("naive", []), ("tp", []), ("tp", ["--checkpointing", "block"]),
                                        ("fsdp", []), ("fsdp", ["--checkpointing", "block"])])
def test_two_gpu_mode_matches_single(tmp_path, tmp_path_factory, mode, extra):
    reference = single_run(tmp_path_factory, "small")
    run = launch(tmp_path, "case", mode, 2, SMALL, ["--microbatch-size", "2", *extra])
    assert_same_training(run, reference, update_tolerance=UPDATE_TOLERANCE.get(mode, 5e-2))
    if mode in ("ddp", "zero1", "tp", "fsdp"):
        assert run["meta"]["execution_path"] == "sm_100a fused engine"
        assert run["meta"]["gradient_reduction"] == "peer-memory kernels over NVLink"
    summary = run["summary"]
    if mode in ("zero1", "fsdp"):
        assert summary["optimizer_state_bytes_max_rank"] * 2 <= summary["optimizer_state_bytes_sum"] + 64
    if mode != "naive":
        # peer-mapped buffers are outside PyTorch's allocator and are reported on top
        assert (summary["peak_cuda_allocated_with_symmetric_bytes"]
                > summary["peak_cuda_allocated_bytes"])


@pytest.mark.parametrize("world", [4, 8])
@pytest.mark.parametrize("mode,extra", [("ddp", []), ("zero1", []), ("fsdp", []),
                                        ("fsdp", ["--checkpointing", "block"]), ("tp", []),
                                        ("tp", ["--checkpointing", "block"])])
def test_wider_groups_match_single(tmp_path, tmp_path_factory, world, mode, extra):
    """Four and eight ranks: the 4- and 8-way reduction kernels, eighth-size optimizer
    slices, and tensor parallelism with one head per rank."""
    need(world)
    reference = single_run(tmp_path_factory, "wide")
    micro = "1" if mode != "tp" else "2"
    # tensor parallelism here stays on GEMM + reduction kernel; the fused form has its own test
    env = {"SFL_TP_FUSE_WIDE": "0"} if mode == "tp" else None
    run = launch(tmp_path, "case", mode, world, WIDE, ["--microbatch-size", micro, *extra],
                 env_extra=env)
    assert_same_training(run, reference, update_tolerance=UPDATE_TOLERANCE.get(mode, 5e-2))
    assert run["meta"]["execution_path"] == "sm_100a fused engine"
    if mode in ("zero1", "fsdp"):
        summary = run["summary"]
        assert (summary["optimizer_state_bytes_max_rank"] * world
                <= summary["optimizer_state_bytes_sum"] * 1.05 + 64 * world)


def test_two_gpu_tensor_parallel_fused_gemm_allreduce_matches_single(tmp_path, tmp_path_factory):
    """A d_model that is a multiple of 256 lets the row-parallel products and the
    column-parallel input gradients run as one GEMM + all-reduce kernel each, issued by
    the native block runner; the result must match a single GPU like every other mode."""
    reference = single_run(tmp_path_factory, "wide")
    for extra in ([], ["--checkpointing", "block"]):
        run = launch(tmp_path, "tp" + str(len(extra)), "tp", 2, WIDE,
                     ["--microbatch-size", "2", *extra])
        assert run["meta"]["tensor_parallel_reduction"].startswith("inside the GEMM kernels")
        assert_same_training(run, reference, update_tolerance=UPDATE_TOLERANCE["tp"])


@pytest.mark.parametrize("world", [4, 8])
def test_tensor_parallel_fused_owned_tiles_match_single(tmp_path, tmp_path_factory, world):
    """More than two ranks: the owned-tile form of the fused GEMM + all-reduce."""
    need(world)
    reference = single_run(tmp_path_factory, "wide")
    run = launch(tmp_path, "tp", "tp", world, WIDE, ["--microbatch-size", "2"])
    assert run["meta"]["tensor_parallel_reduction"].startswith("inside the GEMM kernels")
    assert_same_training(run, reference, update_tolerance=UPDATE_TOLERANCE["tp"])


def run_comm_check(tmp_path, world, env_extra):
    script = ROOT / "tests" / "helpers" / "comm_check.py"
    global PORT
    PORT += 1
    command = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1",
               f"--nproc-per-node={world}", "--master-addr", "127.0.0.1", "--master-port",
               str(PORT), str(script), str(tmp_path / "out.json")]
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0", **env_extra)
    result = subprocess.run(command, cwd=ROOT, env=env, capture_output=True, text=True, timeout=420)
    assert result.returncode == 0, result.stderr[-3000:]
    return json.loads((tmp_path / "out.json").read_text())


def check_comm_results(out):
    assert out["allreduce_maxerr"] < 1e-6 and out["replicas_equal"]
    assert out["norm"] == pytest.approx(out["norm_ref"], rel=1e-5)
    assert out["zero_param_maxerr"] < 2e-6 and out["zero_shadow_ok"]
    assert out["allgather_ok"] and out["tp_reduce_maxerr"] < 1e-6
    assert out["tp_fused_equal"] and out["tp_fused_replicas_equal"]
    assert out["tp_fused_maxerr"] < 0.15      # bf16 partials of a K = 384 reduction, |x| ~ 1
    assert out["timeout_status"] == 5 and out["recovered_after_timeout"]


@pytest.mark.parametrize("one_shot", ["1", "0"])
def test_comm_kernels_against_nccl(tmp_path, one_shot):
    """``one_shot`` picks the variant of the fused GEMM + all-reduce: both ranks finish
    every row (the default for two ranks) or tiles owned round-robin (larger groups)."""
    check_comm_results(run_comm_check(tmp_path, 2, {"SFL_TP_ONE_SHOT": one_shot}))


@pytest.mark.parametrize("world", [4, 8])
def test_comm_kernels_against_nccl_wider_groups(tmp_path, world):
    """The 4- and 8-way reduce kernels, eighth-size AdamW slices, the owned-tile fused
    GEMM + all-reduce, and the timeout / recovery path with more than one waiting peer."""
    need(world)
    check_comm_results(run_comm_check(tmp_path, world, {}))
