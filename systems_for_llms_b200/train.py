"""Single-device training: controlled batching, evaluation, checkpoints, resume.

Command line and artefacts match the reference (src/llmlab/train.py:139-326):
``python -m llmlab.train --config ... --output-dir ...`` writes ``metadata.json``,
``metrics.jsonl`` (start / train / eval / checkpoint / finish events),
``checkpoint.pt`` (atomic, format_version 1) and ``summary.json``; ``--resume``
continues bit-exactly after verifying configuration, data, source and device
identity; ``--stop-after`` pauses early.

What differs is the step itself on a B200: the model's fused engine runs the
forward/backward chain, ``FusedAdamW.clip_and_step`` replaces clip + optimizer,
token windows arrive through pinned memory, and loss / gradient norm are read
back once per step.
"""

from __future__ import annotations

import argparse
import hashlib
import importlib.metadata
import json
import math
import os
import platform
import subprocess
import time
from contextlib import nullcontext
from dataclasses import asdict, replace
from pathlib import Path

import numpy as np
import torch

from .config import TrainConfig, load_config
from .data import batch_at, file_sha256, load_data
from .models.transformer import TransformerLM
from .optim import FusedAdamW
from .training.loss import cross_entropy  # noqa: F401  (re-exported for API parity)

TIMING_SCOPE = ("run() entry to summary construction; excludes interpreter/import startup, "
                "final output writes, and parent invocations")


# ------------------------------------------------------------------ devices --
def get_device(name: str) -> torch.device:
    if name == "auto":
        if torch.cuda.is_available():
            name = "cuda"
        elif torch.backends.mps.is_available():
            name = "mps"
        else:
            name = "cpu"
    if name == "cuda" and not torch.cuda.is_available():
        raise RuntimeError("CUDA requested but unavailable")
    if name == "mps" and not torch.backends.mps.is_available():
        raise RuntimeError("MPS requested but unavailable")
    return torch.device(name)


def synchronize(device: torch.device) -> None:
    if device.type == "cuda":
        torch.cuda.synchronize(device)
    elif device.type == "mps":
        torch.mps.synchronize()


def check_precision(config: TrainConfig, device: torch.device) -> None:
    if config.precision != "bf16":
        return
    if device.type != "cuda":
        raise ValueError("bf16 training requires a CUDA device")
    if not torch.cuda.is_bf16_supported(including_emulation=False):
        raise ValueError("bf16 requires native hardware support on the selected CUDA device")


def autocast(config: TrainConfig, device: torch.device):
    if config.precision == "bf16":
        return torch.autocast(device_type=device.type, dtype=torch.bfloat16)
    return nullcontext()


# ----------------------------------------------------------------- schedule --
def learning_rate(step: int, config: TrainConfig) -> float:
    """Linear warm-up, then cosine decay; ``step`` counts completed updates."""
    peak, floor = config.learning_rate, config.min_learning_rate
    if step < config.warmup_steps:
        return peak * (step + 1) / config.warmup_steps
    span = max(1, config.max_steps - config.warmup_steps - 1)
    progress = (step - config.warmup_steps) / span
    return floor + 0.5 * (peak - floor) * (1 + math.cos(math.pi * progress))


def make_optimizer(model: TransformerLM, config: TrainConfig) -> FusedAdamW:
    return FusedAdamW(model.parameters(), lr=config.learning_rate, betas=(0.9, 0.95),
                      weight_decay=config.weight_decay, engine=None)


def _attach_engine(model: TransformerLM, optimizer, config: TrainConfig, device) -> None:
    """Give the optimizer the model's fused engine once it exists."""
    if isinstance(optimizer, FusedAdamW) and optimizer.engine is None and device.type == "cuda":
        with autocast(config, device):
            optimizer.engine = model.fused_engine()


# --------------------------------------------------------------------- step --
def train_step(model: TransformerLM, optimizer: torch.optim.Optimizer, data: np.ndarray,
               config: TrainConfig, sampler: torch.Generator, device: torch.device) -> dict:
    """One update: sample the effective batch once, then split it into microbatches."""
    accumulation = config.grad_accum_steps
    effective = config.batch_size * accumulation
    starts = torch.randint(len(data) - config.model.context_length, (effective,),
                           generator=sampler)
    stream_hash = hashlib.sha256(starts.numpy().astype("<i8", copy=False).tobytes()).hexdigest()
    optimizer.zero_grad(set_to_none=True)
    running = torch.zeros((), device=device)
    for begin in range(0, effective, config.batch_size):
        x, y = batch_at(data, starts[begin:begin + config.batch_size].tolist(),
                        config.model.context_length, device)
        with autocast(config, device):
            loss = model.loss(x, y, 1.0 / accumulation)
        running += loss.detach()
        loss.backward()
        del x, y, loss
    _attach_engine(model, optimizer, config, device)
    if isinstance(optimizer, FusedAdamW):
        norm = optimizer.clip_and_step(config.grad_clip)
    else:
        norm = torch.nn.utils.clip_grad_norm_(model.parameters(), config.grad_clip,
                                              error_if_nonfinite=True)
        optimizer.step()
    from .ops.gemm import raise_on_status, status_report
    loss_value, norm_value, status_code = torch.cat(
        [torch.stack([running.float(), norm.float().to(device)]), status_report(device)]).tolist()
    raise_on_status(status_code, device)
    if not math.isfinite(loss_value):
        raise FloatingPointError("non-finite training loss")
    if not math.isfinite(norm_value):
        raise RuntimeError("non-finite gradient norm")
    return {"loss": loss_value, "gradient_norm": norm_value, "batch_start_sha256": stream_hash}


@torch.no_grad()
def evaluate(model: TransformerLM, data: np.ndarray, config: TrainConfig,
             device: torch.device) -> float:
    """Mean loss over fixed, evenly spaced validation windows (no RNG involved)."""
    context = config.model.context_length
    windows = np.linspace(0, len(data) - context - 1,
                          config.eval_batch_size * config.eval_batches, dtype=np.int64)
    was_training = model.training
    model.eval()
    weighted, count = 0.0, 0
    try:
        for begin in range(0, len(windows), config.eval_batch_size):
            x, y = batch_at(data, windows[begin:begin + config.eval_batch_size].tolist(),
                            context, device)
            with autocast(config, device):
                loss = model.loss(x, y)
            weighted += loss.item() * y.numel()
            count += y.numel()
    finally:
        model.train(was_training)
    return weighted / count


# ----------------------------------------------------------------- identity --
def source_identity() -> dict:
    """Hash of this package's Python and CUDA sources plus the git state."""
    package = Path(__file__).resolve().parent
    digest = hashlib.sha256()
    for path in sorted(package.rglob("*")):
        if path.suffix in (".py", ".cu", ".cuh", ".h") and "build" not in path.parts:
            digest.update(str(path.relative_to(package)).encode())
            digest.update(path.read_bytes())

    def git(*args: str) -> str | None:
        try:
            return subprocess.check_output(["git", *args], cwd=package.parent,
                                           stderr=subprocess.DEVNULL, text=True).strip()
        except (OSError, subprocess.CalledProcessError):
            return None

    return {"python_source_sha256": digest.hexdigest(), "git_head": git("rev-parse", "HEAD"),
            "git_status": git("status", "--porcelain")}


def resume_config(config: dict) -> dict:
    """Fields that must match on resume; cadence and data paths may change."""
    return {k: v for k, v in config.items()
            if k not in ("eval_interval", "checkpoint_interval", "data")}


def _rng_snapshot(device: torch.device, sampler: torch.Generator) -> dict:
    state = {"sampler_rng_state": sampler.get_state(), "torch_rng_state": torch.get_rng_state()}
    if device.type == "cuda":
        state["cuda_rng_states"] = torch.cuda.get_rng_state_all()
    elif device.type == "mps":
        state["mps_rng_state"] = torch.mps.get_rng_state()
    return state


def _rng_restore(checkpoint: dict, device: torch.device, sampler: torch.Generator) -> None:
    sampler.set_state(checkpoint["sampler_rng_state"])
    torch.set_rng_state(checkpoint["torch_rng_state"])
    if device.type == "cuda":
        torch.cuda.set_rng_state_all(checkpoint["cuda_rng_states"])
    elif device.type == "mps":
        torch.mps.set_rng_state(checkpoint["mps_rng_state"])


def save_checkpoint(path: Path, payload: dict) -> None:
    """Write-then-rename so a crash never leaves a truncated checkpoint."""
    temporary = path.with_name(path.name + ".tmp")
    torch.save(payload, temporary)
    os.replace(temporary, path)


# ---------------------------------------------------------------------- run --
def run(config: TrainConfig, output_dir: str | Path, resume: str | Path | None = None,
        stop_after: int | None = None) -> dict:
    started = time.perf_counter()
    output_dir = Path(output_dir)
    output_dir.mkdir(parents=True, exist_ok=False)
    try:
        return _run(config, output_dir, resume, stop_after, started)
    except Exception as error:
        summary_path = output_dir / "summary.json"
        if not summary_path.exists():
            summary_path.write_text(json.dumps(
                {"status": "failed", "phase": "setup", "step": 0, "error": str(error),
                 "requested_config": repr(config),
                 "wall_seconds": time.perf_counter() - started}, indent=2) + "\n")
        raise


def _metadata(config, config_dict, device, model, data_identity, source, parent) -> dict:
    cuda = device.type == "cuda"
    tokens = config.batch_size * config.grad_accum_steps * config.model.context_length
    properties = torch.cuda.get_device_properties(device) if cuda else None
    return {
        "config": config_dict,
        "config_sha256": hashlib.sha256(json.dumps(config_dict, sort_keys=True).encode()).hexdigest(),
        "data_identity": data_identity, "source": source, "parent_checkpoint": parent,
        "parameter_count": sum(p.numel() for p in model.parameters()),
        "device": str(device), "gpu_count": int(cuda),
        "gpu_name": torch.cuda.get_device_name(device) if cuda else None,
        "platform": platform.platform(), "python": platform.python_version(),
        "packages": {name: importlib.metadata.version(name) for name in ("torch", "numpy", "einops")},
        "precision": config.precision, "parameter_dtype": "float32",
        "effective_batch_size": config.batch_size * config.grad_accum_steps,
        "tokens_per_optimizer_step": tokens,
        "attention_dispatch": ("sm_100a flash attention (fused engine) or PyTorch SDPA"
                               if config.model.attention_backend == "sdpa"
                               else "explicit eager attention"),
        "matmul_precision": torch.get_float32_matmul_precision(),
        "deterministic_algorithms": torch.are_deterministic_algorithms_enabled(),
        "cuda_version": torch.version.cuda,
        "cuda_device_capability": torch.cuda.get_device_capability(device) if cuda else None,
        "cuda_total_memory_bytes": properties.total_memory if cuda else None,
        "timing_scope": TIMING_SCOPE,
        "peak_memory_scope": "training and evaluation after model initialization",
        "workload": ("synthetic pipeline check" if config.data.kind == "synthetic"
                     else "tokenized language modeling"),
        # which of the two code paths this configuration selects (the portable path is
        # the numerical oracle; a run that silently fell back to it is not a
        # measurement of the kernels)
        "execution_path": execution_path(model, config, device),
    }


def execution_path(model: TransformerLM, config: TrainConfig, device: torch.device) -> str:
    if device.type != "cuda" or config.precision != "bf16":
        return "portable PyTorch operators"
    from .models import fused
    return "sm_100a fused engine" if fused.eligible(model) else "portable PyTorch operators"


def _run(config: TrainConfig, output_dir: Path, resume, stop_after, started: float) -> dict:
    config.validate()
    target = config.max_steps if stop_after is None else stop_after
    if type(target) is not int or not 0 < target <= config.max_steps:
        raise ValueError("stop_after must be an integer in [1, max_steps]")
    torch.set_num_threads(config.num_threads)
    device = get_device(config.device)
    check_precision(config, device)
    torch.set_float32_matmul_precision("highest")
    torch.manual_seed(config.seed)
    train_data, valid_data, data_identity = load_data(config)
    model = TransformerLM(**asdict(config.model), device=device, dtype=torch.float32)
    optimizer = make_optimizer(model, config)
    sampler = torch.Generator(device="cpu").manual_seed(config.seed + 1)
    source = source_identity()
    config_dict = config.to_dict()
    step, parent = 0, None
    if resume is not None:
        checkpoint = torch.load(resume, map_location="cpu", weights_only=True)
        if resume_config(checkpoint["config"]) != resume_config(config_dict):
            raise ValueError("resume configuration does not match checkpoint")
        if checkpoint["data_identity"] != data_identity:
            raise ValueError("resume data/tokenizer identity does not match checkpoint")
        if checkpoint["source_sha256"] != source["python_source_sha256"]:
            raise ValueError("resume source differs from checkpoint")
        if checkpoint["device_type"] != device.type:
            raise ValueError("resume device type differs from checkpoint")
        model.load_state_dict(checkpoint["model"])
        optimizer.load_state_dict(checkpoint["optimizer"])
        _rng_restore(checkpoint, device, sampler)
        step = checkpoint["step"]
        if step >= target:
            raise ValueError("checkpoint is already at or beyond the requested stop step")
        parent = {"path": str(Path(resume).resolve()), "sha256": file_sha256(resume), "step": step}
    first_step = step
    metadata = _metadata(config, config_dict, device, model, data_identity, source, parent)
    (output_dir / "metadata.json").write_text(json.dumps(metadata, indent=2) + "\n")
    synchronize(device)
    setup_seconds = time.perf_counter() - started
    seconds = {"train": 0.0, "eval": 0.0, "checkpoint": 0.0}
    last_valid_loss = None
    if device.type == "cuda":
        torch.cuda.reset_peak_memory_stats(device)
    tokens_per_step = config.batch_size * config.grad_accum_steps * config.model.context_length
    stream = (output_dir / "metrics.jsonl").open("w")

    def record(event: str, **fields) -> None:
        row = {"event": event, "step": step, "wall_seconds": time.perf_counter() - started}
        row.update(fields)
        stream.write(json.dumps(row, allow_nan=False) + "\n")
        stream.flush()

    def timed(phase: str, action):
        synchronize(device)
        tick = time.perf_counter()
        result = action()
        synchronize(device)
        elapsed = time.perf_counter() - tick
        seconds[phase] += elapsed
        return result, elapsed

    try:
        model.train()
        record("start", start_step=step)
        while step < target:
            lr = learning_rate(step, config)
            for group in optimizer.param_groups:
                group["lr"] = lr
            values, elapsed = timed("train", lambda: train_step(model, optimizer, train_data,
                                                                config, sampler, device))
            step += 1
            record("train", **values, learning_rate=lr, tokens_seen=step * tokens_per_step,
                   step_seconds=elapsed, train_seconds=seconds["train"],
                   tokens_per_second=tokens_per_step / elapsed)
            last = step == target
            if step % config.eval_interval == 0 or last:
                last_valid_loss, elapsed = timed(
                    "eval", lambda: evaluate(model, valid_data, config, device))
                record("eval", valid_loss=last_valid_loss, eval_seconds=elapsed,
                       valid_tokens=(config.eval_batches * config.eval_batch_size
                                     * config.model.context_length))
            if step % config.checkpoint_interval == 0 or last:
                def write():
                    payload = {"format_version": 1, "config": config_dict,
                               "data_identity": data_identity,
                               "source_sha256": source["python_source_sha256"],
                               "device_type": device.type, "step": step,
                               "model": model.state_dict(), "optimizer": optimizer.state_dict()}
                    payload.update(_rng_snapshot(device, sampler))
                    save_checkpoint(output_dir / "checkpoint.pt", payload)
                _, elapsed = timed("checkpoint", write)
                record("checkpoint", checkpoint_seconds=elapsed, path="checkpoint.pt")
        cuda = device.type == "cuda"
        summary = {
            "status": "completed" if step == config.max_steps else "paused",
            "step": step, "tokens_seen": step * tokens_per_step,
            "invocation_tokens": (step - first_step) * tokens_per_step,
            "valid_loss": last_valid_loss, "setup_seconds": setup_seconds,
            "train_seconds": seconds["train"], "eval_seconds": seconds["eval"],
            "checkpoint_seconds": seconds["checkpoint"],
            "wall_seconds": time.perf_counter() - started, "timing_scope": TIMING_SCOPE,
            "peak_cuda_allocated_bytes": torch.cuda.max_memory_allocated(device) if cuda else None,
            "peak_cuda_reserved_bytes": torch.cuda.max_memory_reserved(device) if cuda else None,
            "execution_path": ("sm_100a fused engine" if getattr(model, "_fused", None) is not None
                               else "portable PyTorch operators"),
        }
        record("finish", status=summary["status"])
        (output_dir / "summary.json").write_text(
            json.dumps(summary, indent=2, allow_nan=False) + "\n")
        return summary
    except Exception as error:
        (output_dir / "summary.json").write_text(json.dumps(
            {"status": "failed", "step": step, "error": str(error),
             "wall_seconds": time.perf_counter() - started}, indent=2) + "\n")
        raise
    finally:
        stream.close()


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--config", required=True, type=Path)
    parser.add_argument("--output-dir", required=True, type=Path)
    parser.add_argument("--resume", type=Path)
    parser.add_argument("--stop-after", type=int)
    parser.add_argument("--attention-backend", choices=["eager", "sdpa"])
    parser.add_argument("--device", choices=["cpu", "cuda", "mps", "auto"])
    parser.add_argument("--precision", choices=["fp32", "bf16"])
    parser.add_argument("--batch-size", type=int, help="sequences per microbatch")
    parser.add_argument("--grad-accum-steps", type=int)
    parser.add_argument("--activation-checkpointing", choices=["none", "block"])
    args = parser.parse_args()
    config = load_config(args.config)
    model_overrides = {}
    if args.attention_backend is not None:
        model_overrides["attention_backend"] = args.attention_backend
    if args.activation_checkpointing is not None:
        model_overrides["activation_checkpointing"] = args.activation_checkpointing
    if model_overrides:
        config = replace(config, model=replace(config.model, **model_overrides))
    top = {name: getattr(args, name) for name in ("device", "precision", "batch_size",
                                                  "grad_accum_steps")
           if getattr(args, name) is not None}
    config = replace(config, **top)
    summary = run(config, args.output_dir, args.resume, args.stop_after)
    print(json.dumps(summary, indent=2))


if __name__ == "__main__":
    main()
