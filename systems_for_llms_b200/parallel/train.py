"""Matched-global-batch training under ``torch.distributed.run``.

Command line, modes, artefacts and measurement protocol follow the reference
runner (distributed/llmdist/train.py:28-460): ``--mode single|naive|ddp|zero1|
fsdp|tp``; every rank builds the same fp32 model from the same seed and the
initial hashes are compared; one global batch is sampled per update with the same
CPU generator on every rank and sliced by rank (tensor parallelism consumes all
of it); each step is timed after a barrier between device synchronisations and
the maximum over ranks is recorded; per-rank ``metadata`` / ``metrics`` /
``summary`` files plus ``summary.json`` on rank 0, optional ``final-state.pt`` and
profiler traces; a failure writes ``rank-R-failure.json``.

On B200 the wrappers take their fused paths:

  ddp    BucketedDDP over peer memory (bucket all-reduce kernels overlapped with
         backward, scale + gradient norm fused) and FusedAdamW
  zero1  BucketedDDP in scatter mode and ShardedAdamW flat slices
         (reduce-scatter -> fused AdamW -> all-gather stores)
  fsdp   per-block sharding (parallel/fsdp.py)
  tp     head / feed-forward sharding (parallel/tensor_parallel.py)

On other devices (CPU with gloo in the tests) the same wrappers run on
``torch.distributed`` collectives.
"""

from __future__ import annotations

import argparse
import hashlib
import importlib.metadata
import json
import math
import os
import platform
import statistics
import time
from contextlib import nullcontext
from dataclasses import asdict, replace
from datetime import timedelta
from pathlib import Path

import numpy as np
import torch
import torch.distributed as dist

from ..config import TrainConfig, load_config
from ..data import batch_at, load_data
from ..models.transformer import TransformerLM
from ..optim import FusedAdamW
from ..train import autocast, check_precision, learning_rate, synchronize

MODES = ("single", "naive", "ddp", "zero1", "fsdp", "tp")
TIMING_SCOPE = ("max rank synchronized optimizer-step time after an inter-rank barrier; "
                "includes data, backward synchronization, clipping, update and loss reduction; "
                "excludes timing-max reduction, evaluation, setup and checkpoint writes")


def validate_layout(mode, world_size, global_batch_size, microbatch_size, sync_policy) -> int:
    """Checks the batch geometry and returns the accumulation steps per update."""
    if mode not in MODES:
        raise ValueError(f"Unknown mode: {mode}")
    if sync_policy not in ("last", "every"):
        raise ValueError("sync_policy must be last or every")
    if mode == "single" and world_size != 1:
        raise ValueError("single mode requires one rank")
    if mode != "single" and world_size < 2:
        raise ValueError("Distributed modes require at least two ranks")
    for value in (world_size, global_batch_size, microbatch_size):
        if type(value) is not int or value <= 0:
            raise ValueError("World, global batch and microbatch sizes must be positive integers")
    replicas = 1 if mode == "tp" else world_size
    if global_batch_size % (replicas * microbatch_size):
        raise ValueError("Global batch must be divisible by data-parallel ranks times microbatch")
    if sync_policy == "every" and mode not in ("ddp", "zero1"):
        raise ValueError("sync-policy every applies to DDP and zero1 only")
    return global_batch_size // replicas // microbatch_size


def source_identity() -> dict:
    package = Path(__file__).resolve().parents[1]
    files = {}
    for path in sorted(package.rglob("*")):
        if path.suffix in (".py", ".cu", ".cuh", ".h") and "build" not in path.parts:
            files[str(path.relative_to(package))] = hashlib.sha256(path.read_bytes()).hexdigest()
    digest = hashlib.sha256(json.dumps(files, sort_keys=True).encode()).hexdigest()
    return {"files": files, "sha256": digest}


def _local(tensor):
    return tensor.to_local() if hasattr(tensor, "to_local") else tensor


def state_hash(model) -> str:
    """sha256 over (name, shape, bytes) of every parameter this rank holds."""
    digest = hashlib.sha256()
    for name, parameter in model.named_parameters():
        value = _local(parameter.detach()).to(device="cpu").contiguous()
        digest.update(name.encode())
        digest.update(str(tuple(value.shape)).encode())
        digest.update(value.view(torch.uint8).numpy().tobytes())
    return digest.hexdigest()


def tensor_bytes(value) -> int:
    if isinstance(value, torch.Tensor):
        local = _local(value)
        return local.numel() * local.element_size()
    if isinstance(value, dict):
        return sum(tensor_bytes(item) for item in value.values())
    if isinstance(value, (tuple, list)):
        return sum(tensor_bytes(item) for item in value)
    return 0


def _cpu_tree(value):
    if isinstance(value, torch.Tensor):
        return _local(value.detach()).cpu()
    if isinstance(value, dict):
        return {key: _cpu_tree(item) for key, item in value.items()}
    if isinstance(value, list):
        return [_cpu_tree(item) for item in value]
    if isinstance(value, tuple):
        return tuple(_cpu_tree(item) for item in value)
    return value


def _all_reduce(value, op=dist.ReduceOp.SUM):
    if dist.is_initialized():
        dist.all_reduce(value, op=op)
    return value


def fsdp_clip_grad_norm(model, max_norm):
    """Global-norm clip for the sharded model (each element counted once)."""
    from .fsdp import clip_grad_norm_sharded
    return clip_grad_norm_sharded(model.parameters(), max_norm)


class Strategy:
    """Everything mode-specific: wrapping, the per-microbatch context, reduction, update."""

    def __init__(self, mode, base_model, config, device, *, world, rank, sync_policy,
                 bucket_cap_mb):
        self.mode, self.base, self.config, self.device = mode, base_model, config, device
        self.world, self.rank, self.sync_policy = world, rank, sync_policy
        self.model = base_model
        self.ddp = None
        self.engine = None
        self.sharding = None
        kwargs = dict(lr=config.learning_rate, betas=(0.9, 0.95), weight_decay=config.weight_decay)
        fused_possible = device.type == "cuda" and config.precision == "bf16"
        if mode == "tp":
            from .tensor_parallel import describe_sharding, parallelize_model
            parallelize_model(base_model)
            self.sharding = describe_sharding(base_model)
            if fused_possible:
                from .tensor_parallel import enable_fused
                self.engine = enable_fused(base_model, autocast(config, device))
        elif mode == "fsdp":
            if fused_possible:
                with autocast(config, device):
                    self.engine = base_model.fused_engine()
            if self.engine is not None:
                from .fsdp_fused import FusedShardedTransformer
                self.model = FusedShardedTransformer(base_model, self.engine)
            else:
                from .fsdp import shard_model
                self.model = shard_model(base_model)
        if fused_possible and mode in ("single", "naive", "ddp", "zero1"):
            with autocast(config, device):
                self.engine = base_model.fused_engine()
        if mode in ("ddp", "zero1"):
            from .ddp import BucketedDDP
            scatter = mode == "zero1" and self.engine is not None
            self.ddp = BucketedDDP(base_model, bucket_cap_mb=bucket_cap_mb,
                                   mode="scatter" if scatter else "allreduce")
            if self.engine is not None:
                self.ddp.enable_peer_memory(self.engine)
            self.model = self.ddp
        if mode == "zero1":
            from .optim_shard import ShardedAdamW
            self.optimizer = ShardedAdamW(base_model.parameters(), **kwargs)
            if self.engine is not None:
                self.optimizer.attach_flat(self.ddp, self.engine)
        elif mode == "fsdp" and self.engine is not None:
            from .fsdp_fused import ShardedStepper
            self.optimizer = ShardedStepper(self.model, **kwargs)
        elif mode == "fsdp":
            self.optimizer = torch.optim.AdamW(self.model.parameters(), **kwargs)
        else:
            self.optimizer = FusedAdamW(base_model.parameters(), engine=self.engine, **kwargs)

    @property
    def trainable(self):
        return self.model if self.mode == "fsdp" else self.base

    def microbatch_context(self, last: bool):
        if self.mode in ("ddp", "zero1") and self.sync_policy == "last" and not last:
            return self.ddp.no_sync()
        if self.mode == "fsdp":
            self.model.set_requires_gradient_sync(last)
        return nullcontext()

    def after_backward(self) -> None:
        """Called after every microbatch's backward."""
        if self.mode == "fsdp" and self.engine is not None:
            self.model.end_microbatch()

    def optimizer_state_bytes(self) -> int:
        if self.mode == "zero1":
            return self.optimizer.local_state_bytes()
        return tensor_bytes(self.optimizer.state)

    def reduce_and_update(self) -> torch.Tensor:
        """After the last backward: synchronise gradients, clip, step.  Returns the norm."""
        config, mode = self.config, self.mode
        if mode == "naive":
            for parameter in self.base.parameters():
                if parameter.grad is None:
                    raise RuntimeError("The naive reducer requires every parameter to have a gradient")
                _all_reduce(parameter.grad).div_(self.world)
        if mode in ("ddp", "zero1"):
            stats = self.ddp.finish(config.grad_clip)
            if stats is not None:                      # peer-memory path
                if mode == "zero1":
                    self.optimizer.step_flat(stats)
                    return stats[0]
                return self.optimizer.step_with_stats(stats)
        if mode == "tp" and self.engine is not None:
            from .tensor_parallel import fused_grad_stats
            stats = fused_grad_stats(self.base, self.engine, config.grad_clip)
            return self.optimizer.step_with_stats(stats)
        if mode == "tp":
            from .tensor_parallel import clip_grad_norm_tp
            norm = clip_grad_norm_tp(self.base, config.grad_clip, error_if_nonfinite=True)
            self.optimizer.step()
            return norm
        if mode == "fsdp" and self.engine is not None:
            return self.optimizer.clip_and_step(config.grad_clip)
        if mode == "fsdp":
            norm = fsdp_clip_grad_norm(self.model, config.grad_clip)
            self.optimizer.step()
            return norm
        if isinstance(self.optimizer, FusedAdamW):
            return self.optimizer.clip_and_step(config.grad_clip)
        norm = torch.nn.utils.clip_grad_norm_(self.base.parameters(), config.grad_clip,
                                              error_if_nonfinite=True)
        self.optimizer.step()
        return norm

    def full_state(self):
        if self.mode == "tp":
            from .tensor_parallel import reconstruct_state_dict
            return reconstruct_state_dict(self.base)
        if self.mode == "fsdp":
            return self.model.full_state_dict()
        return self.base.state_dict()

    def close(self) -> None:
        if self.mode == "zero1" and hasattr(self.optimizer, "close"):
            self.optimizer.close()
        if self.ddp is not None:
            self.ddp.close()
        if self.mode == "fsdp" and hasattr(self.model, "close"):
            self.model.close()
        if self.engine is not None and self.engine.tp is not None:
            self.engine.tp.close()
            self.engine.tp = None


def train_step(strategy: Strategy, data, config, sampler, device, *, global_batch_size,
               microbatch_size) -> dict:
    mode, rank, world = strategy.mode, strategy.rank, strategy.world
    accumulation = validate_layout(mode, world, global_batch_size, microbatch_size,
                                   strategy.sync_policy)
    starts = torch.randint(len(data) - config.model.context_length, (global_batch_size,),
                           generator=sampler)
    stream_hash = hashlib.sha256(starts.numpy().astype("<i8", copy=False).tobytes()).hexdigest()
    local_batch = global_batch_size if mode == "tp" else global_batch_size // world
    mine = starts if mode == "tp" else starts[rank * local_batch:(rank + 1) * local_batch]
    strategy.optimizer.zero_grad(set_to_none=True)
    loss_sum = torch.zeros((), device=device)
    for index, begin in enumerate(range(0, local_batch, microbatch_size)):
        with strategy.microbatch_context(last=index == accumulation - 1):
            x, y = batch_at(data, mine[begin:begin + microbatch_size].tolist(),
                            config.model.context_length, device)
            with autocast(config, device):
                loss = strategy.model.loss(x, y, 1.0 / accumulation)
            loss_sum += loss.detach()
            loss.backward()
            strategy.after_backward()
            del x, y, loss
    # Reference order: vote on finiteness, then clip and update.  The fused
    # update skips itself on a non-finite norm, so the vote can ride along with
    # the single read-back at the end of the step without changing the outcome.
    norm = strategy.reduce_and_update()
    # The device status word rides along: a peer or pipeline wait that ran out during this
    # step must stop the run here, not after the last step.
    from ..ops.gemm import raise_on_status, status_report
    report = torch.cat([torch.stack([loss_sum.float(), torch.isfinite(loss_sum).float(),
                                     norm.float().to(device)]), status_report(device)])
    if world > 1:
        # one collective: the loss sums, and so do the finiteness votes (all ranks
        # finite <=> the votes add up to the world size)
        votes = report[:2].clone()
        dist.all_reduce(votes)
        report[:2] = votes
        report[1] = (votes[1] >= world - 0.5).float()
    mean_loss, finite, norm_value, status_code = report.tolist()
    raise_on_status(status_code, device)
    if not finite:
        raise FloatingPointError("Non-finite training loss on a rank")
    if not math.isfinite(norm_value):
        raise RuntimeError("Non-finite global gradient norm")
    return {"loss": mean_loss / world, "gradient_norm": norm_value,
            "batch_start_sha256": stream_hash}


@torch.no_grad()
def evaluate(model, data, config, device, *, rank, world_size, mode) -> float:
    windows = config.eval_batches * config.eval_batch_size
    if mode != "tp" and config.eval_batches % world_size:
        raise ValueError("eval_batches must be divisible by the number of data-parallel ranks")
    starts = np.linspace(0, len(data) - config.model.context_length - 1, windows, dtype=np.int64)
    if mode != "tp":
        starts = starts[rank * windows // world_size:(rank + 1) * windows // world_size]
    was_training = model.training
    model.eval()
    totals = torch.zeros(2, device=device, dtype=torch.float64)
    try:
        for begin in range(0, len(starts), config.eval_batch_size):
            x, y = batch_at(data, starts[begin:begin + config.eval_batch_size].tolist(),
                            config.model.context_length, device)
            with autocast(config, device):
                loss = model.loss(x, y)
            totals[0] += loss.double() * y.numel()
            totals[1] += y.numel()
    finally:
        model.train(was_training)
    _all_reduce(totals)
    return (totals[0] / totals[1]).item()


def _environment() -> tuple[int, int, int]:
    return tuple(int(os.environ.get(key, default)) for key, default in
                 (("RANK", "0"), ("WORLD_SIZE", "1"), ("LOCAL_RANK", "0")))


def run(config: TrainConfig, output_dir, *, mode="single", global_batch_size=8,
        microbatch_size=1, warmup_steps=5, sync_policy="last", bucket_cap_mb=25.,
        save_final_state=False, profile_steps=0):
    rank, world, local_rank = _environment()
    accumulation = validate_layout(mode, world, global_batch_size, microbatch_size, sync_policy)
    config.validate()
    if not 0 <= warmup_steps < config.max_steps:
        raise ValueError("Timing warmup must be smaller than the update count")
    if bucket_cap_mb <= 0 or not np.isfinite(bucket_cap_mb) or profile_steps < 0:
        raise ValueError("Bucket capacity must be finite and positive; profile steps nonnegative")
    if config.device not in ("cpu", "cuda"):
        raise ValueError("Distributed runner supports explicit cpu or cuda devices")
    if mode != "tp" and config.eval_batches % world:
        raise ValueError("eval_batches must be divisible by data-parallel ranks")
    torch.set_num_threads(config.num_threads)
    if config.device == "cuda":
        if not torch.cuda.is_available() or local_rank >= torch.cuda.device_count():
            raise RuntimeError("Requested CUDA device is unavailable")
        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
    else:
        device = torch.device("cpu")
    check_precision(config, device)
    torch.set_float32_matmul_precision("highest")
    output = Path(output_dir)
    initialized_here = output_ready = False
    strategy = None
    started = time.perf_counter()
    try:
        if world > 1 and not dist.is_initialized():
            dist.init_process_group(backend="nccl" if device.type == "cuda" else "gloo",
                                    init_method="env://", timeout=timedelta(seconds=120))
            initialized_here = True
        if rank == 0:
            output.mkdir(parents=True, exist_ok=False)
            output_ready = True
        if world > 1:
            dist.barrier()
        output_ready = True
        torch.manual_seed(config.seed)
        train_data, valid_data, data_identity = load_data(config)
        base_model = TransformerLM(**asdict(config.model), device=device, dtype=torch.float32)
        parameter_count = sum(p.numel() for p in base_model.parameters())
        initial_hash = state_hash(base_model)
        if world > 1:
            hashes = [None] * world
            dist.all_gather_object(hashes, initial_hash)
            if len(set(hashes)) != 1:
                raise RuntimeError("Initial full-model parameters differ across ranks")
        strategy = Strategy(mode, base_model, config, device, world=world, rank=rank,
                            sync_policy=sync_policy, bucket_cap_mb=bucket_cap_mb)
        optimizer = strategy.optimizer
        trainable = strategy.trainable
        sampler = torch.Generator(device="cpu").manual_seed(config.seed + 1)
        cuda = device.type == "cuda"

        def local_parameter_bytes():
            return sum(_local(p).numel() * p.element_size() for p in trainable.parameters())

        def local_gradient_bytes():
            return sum(tensor_bytes(p.grad) for p in trainable.parameters() if p.grad is not None)

        metadata = {
            "format_version": 1, "config": config.to_dict(), "mode": mode, "rank": rank,
            "local_rank": local_rank, "world_size": world,
            "data_parallel_size": 1 if mode == "tp" else world,
            "global_batch_size": global_batch_size, "microbatch_size": microbatch_size,
            "accumulation_steps": accumulation, "sync_policy": sync_policy,
            "bucket_cap_mb": bucket_cap_mb, "timing_warmup_steps": warmup_steps,
            "profile_steps": profile_steps, "parameter_count": parameter_count,
            "local_parameter_bytes": local_parameter_bytes(),
            "local_gradient_bytes_before_training": local_gradient_bytes(),
            "optimizer_state_bytes_before_training": strategy.optimizer_state_bytes(),
            "cuda_allocated_bytes_before_training": torch.cuda.memory_allocated(device) if cuda else None,
            "cuda_reserved_bytes_before_training": torch.cuda.memory_reserved(device) if cuda else None,
            "initial_parameter_sha256": initial_hash, "data_identity": data_identity,
            "source": source_identity(), "sharding": strategy.sharding,
            "optimizer_ownership": optimizer.ownership_metadata() if mode == "zero1" else None,
            "python": platform.python_version(),
            "packages": {n: importlib.metadata.version(n) for n in ("torch", "numpy", "einops")},
            "device": str(device),
            "gpu_name": torch.cuda.get_device_name(device) if cuda else None,
            "cuda_version": torch.version.cuda,
            "gpu_total_memory_bytes": torch.cuda.get_device_properties(device).total_memory if cuda else None,
            "timing_scope": TIMING_SCOPE,
            "peak_memory_scope": ("training and evaluation after model/wrapper setup; "
                                  "final state export excluded"),
            "execution_path": ("sm_100a fused engine" if strategy.engine is not None
                               else "portable PyTorch operators"),
            "gradient_reduction": ("peer-memory kernels over NVLink"
                                   if (strategy.ddp is not None and strategy.ddp._peer_active())
                                   or (strategy.engine is not None and strategy.engine.tp is not None)
                                   or (mode == "fsdp" and strategy.engine is not None)
                                   else "torch.distributed collectives"),
            "tensor_parallel_reduction": (
                None if strategy.engine is None or strategy.engine.tp is None
                else "inside the GEMM kernels (tile by tile over peer memory)"
                if strategy.engine.tp.can_fuse(strategy.engine.d_model)
                else "separate peer-memory kernel after each GEMM"),
            "checkpoint_scope": ("optional final model/optimizer state for correctness checks; "
                                 "resume unsupported"),
        }
        (output / f"rank-{rank}-metadata.json").write_text(json.dumps(metadata, indent=2) + "\n")
        if save_final_state:
            # The state before the first update, gathered like the final one: parity checks
            # compare the UPDATE (final - initial), which a tolerance on raw parameters
            # cannot resolve after a handful of small steps.
            state = strategy.full_state()
            if rank == 0:
                torch.save({"model": {name: value.detach().cpu() for name, value in state.items()}},
                           output / "initial-state.pt")
            del state
        synchronize(device)
        if world > 1:
            dist.barrier()
        setup_seconds = time.perf_counter() - started
        if cuda:
            torch.cuda.reset_peak_memory_stats(device)
        rows, measured = [], []
        first_update_memory = last_valid_loss = None
        tokens_per_step = global_batch_size * config.model.context_length
        strategy.model.train()
        profile = nullcontext()
        if profile_steps:
            activities = [torch.profiler.ProfilerActivity.CPU]
            if cuda:
                activities.append(torch.profiler.ProfilerActivity.CUDA)
            profile = torch.profiler.profile(
                activities=activities,
                schedule=torch.profiler.schedule(wait=warmup_steps, warmup=1, active=profile_steps,
                                                 repeat=1),
                on_trace_ready=lambda p: p.export_chrome_trace(str(output / f"rank-{rank}-trace.json")),
                record_shapes=True, profile_memory=True)
        with (output / f"rank-{rank}-metrics.jsonl").open("w") as stream, profile as profiler:
            def record(event, step, **values):
                row = {"event": event, "step": step,
                       "wall_seconds": time.perf_counter() - started, **values}
                stream.write(json.dumps(row, allow_nan=False) + "\n")
                stream.flush()
                rows.append(row)

            for step in range(1, config.max_steps + 1):
                if world > 1:
                    dist.barrier()
                synchronize(device)
                tick = time.perf_counter()
                lr = learning_rate(step - 1, config)
                for group in optimizer.param_groups:
                    group["lr"] = lr
                values = train_step(strategy, train_data, config, sampler, device,
                                    global_batch_size=global_batch_size,
                                    microbatch_size=microbatch_size)
                synchronize(device)
                local_seconds = time.perf_counter() - tick
                slowest = _all_reduce(torch.tensor(local_seconds, device=device, dtype=torch.float64),
                                      dist.ReduceOp.MAX).item()
                record("train", step, **values, learning_rate=lr,
                       tokens_seen=step * tokens_per_step, step_seconds=slowest,
                       local_step_seconds=local_seconds)
                if step == 1:
                    first_update_memory = {
                        "optimizer_state_bytes": strategy.optimizer_state_bytes(),
                        "local_gradient_bytes": local_gradient_bytes(),
                        "cuda_allocated_bytes": torch.cuda.memory_allocated(device) if cuda else None,
                        "cuda_reserved_bytes": torch.cuda.memory_reserved(device) if cuda else None,
                    }
                if step > warmup_steps:
                    measured.append(slowest)
                if step % config.eval_interval == 0 or step == config.max_steps:
                    synchronize(device)
                    tick = time.perf_counter()
                    eval_model = strategy.model if mode == "fsdp" else base_model
                    last_valid_loss = evaluate(eval_model, valid_data, config, device, rank=rank,
                                               world_size=world, mode=mode)
                    synchronize(device)
                    record("eval", step, valid_loss=last_valid_loss,
                           eval_seconds=time.perf_counter() - tick,
                           valid_tokens=(config.eval_batches * config.eval_batch_size
                                         * config.model.context_length))
                if profiler is not None:
                    profiler.step()
        if cuda:
            from ..ops.gemm import check_status
            check_status(device)
        batch_stream_hash = hashlib.sha256("".join(
            row["batch_start_sha256"] for row in rows if row["event"] == "train").encode()).hexdigest()
        symmetric_peak = 0
        if cuda:
            from .comm import symmetric_memory_bytes
            symmetric_peak = symmetric_memory_bytes()["peak"]
        rank_result = {
            "rank": rank,
            "peak_cuda_allocated_bytes": torch.cuda.max_memory_allocated(device) if cuda else None,
            # peer-mapped buffers are allocated outside PyTorch's allocator
            "symmetric_buffer_bytes": symmetric_peak if cuda else None,
            "peak_cuda_allocated_with_symmetric_bytes":
                torch.cuda.max_memory_allocated(device) + symmetric_peak if cuda else None,
            "peak_cuda_reserved_bytes": torch.cuda.max_memory_reserved(device) if cuda else None,
            "optimizer_state_bytes": strategy.optimizer_state_bytes(),
            "local_parameter_bytes": local_parameter_bytes(),
            "local_gradient_bytes": local_gradient_bytes(),
            "first_update_memory": first_update_memory,
            "batch_stream_sha256": batch_stream_hash,
            "final_parameter_sha256": state_hash(trainable),
            "parameter_hash_scope": ("rank-local shard" if mode in ("fsdp", "tp")
                                     else "full replicated model"),
        }
        ranks = [None] * world
        if world > 1:
            dist.all_gather_object(ranks, rank_result)
        else:
            ranks = [rank_result]
        if len({item["batch_stream_sha256"] for item in ranks}) != 1:
            raise RuntimeError("Global batch streams differ across ranks")
        if mode in ("naive", "ddp", "zero1") and len({item["final_parameter_sha256"] for item in ranks}) != 1:
            raise RuntimeError("Final replicated parameters differ across ranks")
        if save_final_state:
            state = strategy.full_state()
            if rank == 0:
                torch.save({"model": {name: value.detach().cpu() for name, value in state.items()},
                            "optimizer": _cpu_tree(optimizer.state_dict()),
                            "sampler_rng_state": sampler.get_state()}, output / "final-state.pt")
        summary = {
            "status": "completed", "mode": mode, "world_size": world,
            "global_batch_size": global_batch_size, "microbatch_size": microbatch_size,
            "accumulation_steps": accumulation, "sync_policy": sync_policy,
            "step": config.max_steps, "tokens_seen": config.max_steps * tokens_per_step,
            "tokens_per_step": tokens_per_step, "measured_steps": len(measured),
            "step_seconds_median": statistics.median(measured),
            "step_seconds_p90": float(np.percentile(measured, 90)),
            "tokens_per_second": len(measured) * tokens_per_step / sum(measured),
            "measured_train_seconds": sum(measured), "setup_seconds": setup_seconds,
            "valid_loss": last_valid_loss, "profiled": bool(profile_steps), "ranks": ranks,
            "peak_cuda_allocated_bytes": max(i["peak_cuda_allocated_bytes"] for i in ranks) if cuda else None,
            "peak_cuda_reserved_bytes": max(i["peak_cuda_reserved_bytes"] for i in ranks) if cuda else None,
            "peak_cuda_allocated_with_symmetric_bytes":
                max(i["peak_cuda_allocated_with_symmetric_bytes"] for i in ranks) if cuda else None,
            "optimizer_state_bytes_max_rank": max(i["optimizer_state_bytes"] for i in ranks),
            "optimizer_state_bytes_sum": sum(i["optimizer_state_bytes"] for i in ranks),
            "batch_stream_sha256": batch_stream_hash,
            "wall_seconds": time.perf_counter() - started, "timing_scope": TIMING_SCOPE,
        }
        text = json.dumps(summary, indent=2, allow_nan=False) + "\n"
        (output / f"rank-{rank}-summary.json").write_text(text)
        if rank == 0:
            (output / "summary.json").write_text(text)
        return summary
    except Exception as error:
        if output_ready:
            failure = {"status": "failed", "rank": rank, "mode": mode, "error": str(error),
                       "wall_seconds": time.perf_counter() - started}
            (output / f"rank-{rank}-failure.json").write_text(json.dumps(failure, indent=2) + "\n")
            if rank == 0:
                (output / "summary.json").write_text(json.dumps(failure, indent=2) + "\n")
        raise
    finally:
        if strategy is not None:
            try:
                if world > 1 and dist.is_initialized():
                    synchronize(device)
                strategy.close()
            except Exception:
                pass
        if initialized_here:
            dist.destroy_process_group()


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("--config", required=True, type=Path)
    parser.add_argument("--output-dir", required=True, type=Path)
    parser.add_argument("--mode", choices=MODES, default="single")
    parser.add_argument("--global-batch-size", type=int, default=8)
    parser.add_argument("--microbatch-size", type=int, default=1)
    parser.add_argument("--seed", type=int)
    parser.add_argument("--steps", type=int)
    parser.add_argument("--warmup-steps", type=int, default=5,
                        help="training updates excluded from timing")
    parser.add_argument("--sync-policy", choices=["last", "every"], default="last")
    parser.add_argument("--bucket-cap-mb", type=float, default=25.)
    parser.add_argument("--checkpointing", choices=["none", "block"])
    parser.add_argument("--device", choices=["cpu", "cuda"])
    parser.add_argument("--precision", choices=["fp32", "bf16"])
    parser.add_argument("--save-final-state", action="store_true")
    parser.add_argument("--profile-steps", type=int, default=0)
    args = parser.parse_args()
    config = load_config(args.config)
    overrides = {key: value for key, value in (("seed", args.seed), ("max_steps", args.steps),
                                               ("device", args.device),
                                               ("precision", args.precision)) if value is not None}
    config = replace(config, **overrides)
    if args.checkpointing is not None:
        config = replace(config, model=replace(config.model,
                                               activation_checkpointing=args.checkpointing))
    result = run(config, args.output_dir, mode=args.mode,
                 global_batch_size=args.global_batch_size, microbatch_size=args.microbatch_size,
                 warmup_steps=args.warmup_steps, sync_policy=args.sync_policy,
                 bucket_cap_mb=args.bucket_cap_mb, save_final_state=args.save_final_state,
                 profile_steps=args.profile_steps)
    if int(os.environ.get("RANK", "0")) == 0:
        print(json.dumps(result, indent=2))


if __name__ == "__main__":
    main()
