"""Headline benchmark: training throughput of the 324M decoder at sequence 1024.

    python bench.py --gpus N --steps K --warmup W [--impl ours|reference] [--mode MODE]
                    [--checkpointing none|block] [--seq-len S --global-batch B --microbatch M]

Metric and configuration are the reference's distributed protocol (324,092,928
parameters, bf16 autocast with fp32 parameters and AdamW state, global batch 32 x
1024 tokens per update, microbatch 4, AdamW + clip 1.0, cosine schedule): one
process drives one GPU (``--mode single``, 8 accumulation steps); N processes
under ``torch.distributed.run`` train data-parallel (``ddp`` by default; ``zero1``,
``fsdp`` and ``tp`` selectable) on the same global batch, so scaling is strong.
Token ids are synthetic uniform-random, weights are randomly initialised.
``--seq-len 4096 --global-batch 8 --microbatch 1`` is the reference's long-context
workload (same model, same tokens per update); both arms honour the three flags.

Two numbers are reported.  ``value`` is timed on the device with CUDA events
around exactly K optimizer steps whose token batches already sit in device
memory; ``e2e.value`` goes through the public step function
(``parallel.train.train_step``): per step it samples the global batch, copies
each microbatch from pinned host memory, and reads loss and gradient norm back;
that loop runs W warm-up steps of its own before its K timed ones.
Both are the maximum over ranks.  ``--impl reference`` runs the unmodified
reference package installed under ``baseline/_ref`` through its own runner and
reports its own throughput figure in the same JSON shape.
"""

from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
METRIC = "tokens/s 324M s1024 @1/2/4/8 B200 (DDP/shard/FSDP/TP), max over ranks; peak GiB"
GLOBAL_BATCH, MICROBATCH, SEQ = 32, 4, 1024      # defaults; main() applies the flags
PUBLISHED = {  # tokens/s on 8xH200 / 1xH200 from the reference's confirmation study
    ("single", 1): 67021.0, ("ddp", 2): 126224.0, ("ddp", 4): 226220.0, ("ddp", 8): 397738.0,
    ("zero1", 2): 121692.0, ("zero1", 4): 218501.0, ("zero1", 8): 353293.0,
    ("fsdp", 2): 70471.0, ("fsdp", 4): 134447.0, ("fsdp", 8): 231534.0,
    ("tp", 2): 60115.0, ("tp", 4): 57363.0, ("tp", 8): 55733.0,
}
PUBLISHED_BLOCK = {("single", 1): 35587.0, ("ddp", 8): 213460.0, ("fsdp", 2): 44347.0,
                   ("fsdp", 4): 80889.0, ("fsdp", 8): 150249.0, ("tp", 2): 31988.0,
                   ("tp", 4): 30117.0, ("tp", 8): 27414.0}
PUBLISHED_S4096 = {("single", 1, "none"): 63273.0, ("single", 1, "block"): 34239.0,
                   ("ddp", 8, "none"): 395309.0, ("ddp", 8, "block"): 195089.0,
                   ("zero1", 8, "block"): 183612.0, ("fsdp", 8, "block"): 147702.0,
                   ("tp", 8, "block"): 27775.0}


def published_for(mode: str, world: int, checkpointing: str):
    """The reference's published tokens/s for this workload (H200), or None."""
    if (GLOBAL_BATCH, MICROBATCH, SEQ) == (32, 4, 1024):
        table = PUBLISHED if checkpointing == "none" else PUBLISHED_BLOCK
        return table.get((mode, world))
    if (GLOBAL_BATCH, MICROBATCH, SEQ) == (8, 1, 4096):
        return PUBLISHED_S4096.get((mode, world, checkpointing))
    return None


def model_config() -> dict:
    return {"vocab_size": 10000, "context_length": SEQ, "d_model": 1024, "num_layers": 24,
            "num_heads": 16, "d_ff": 2752, "rope_theta": 10000.0, "attention_backend": "sdpa",
            "activation_checkpointing": "none"}


def train_config_dict(steps: int, checkpointing: str) -> dict:
    model = model_config()
    model["activation_checkpointing"] = checkpointing
    return {"model": model, "data": {"kind": "synthetic", "synthetic_tokens": 4_000_000},
            "seed": 1337, "device": "cuda", "num_threads": 4, "batch_size": MICROBATCH,
            "grad_accum_steps": 1, "precision": "bf16", "max_steps": max(steps, 7),
            "learning_rate": 3e-4, "min_learning_rate": 3e-5, "warmup_steps": 5,
            "weight_decay": 0.1, "grad_clip": 1.0, "eval_interval": 10 ** 6, "eval_batches": 8,
            "eval_batch_size": 1, "checkpoint_interval": 10 ** 6}


class ClockSampler:
    """Samples SM clock and throttle reasons while the timed region runs (reads only).

    NVML is polled from a thread every 25 ms, so even a timed region of a tenth of
    a second gets samples; ``nvidia-smi -lms`` is the fallback when the NVML
    binding cannot be loaded.  Only rank 0 samples (``enabled``): management
    queries from eight processes at once take driver locks that kernel launches
    also need, which slowed the launch-heavy sharded modes inside the timed
    region.
    """

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self, index: int, uuid: str | None = None, enabled: bool = True):
        self.index, self.uuid, self.enabled = index, uuid, enabled
        self.samples, self.process, self.thread = [], None, None
        self.stop = threading.Event()

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        if self.uuid:
            try:
                return pynvml, pynvml.nvmlDeviceGetHandleByUUID(f"GPU-{self.uuid}".encode())
            except pynvml.NVMLError:
                pass
        return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.index)

    def _poll_nvml(self, nvml, handle):
        bits = (nvml.nvmlClocksThrottleReasonHwSlowdown,
                nvml.nvmlClocksThrottleReasonHwThermalSlowdown,
                nvml.nvmlClocksThrottleReasonSwThermalSlowdown,
                nvml.nvmlClocksThrottleReasonSwPowerCap)
        peak = nvml.nvmlDeviceGetMaxClockInfo(handle, nvml.NVML_CLOCK_SM)
        while not self.stop.is_set():
            try:
                clock = nvml.nvmlDeviceGetClockInfo(handle, nvml.NVML_CLOCK_SM)
                mask = nvml.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.samples.append([str(clock), str(peak)]
                                    + ["Active" if mask & bit else "Not Active" for bit in bits])
            except nvml.NVMLError:
                pass
            self.stop.wait(0.025)

    def __enter__(self):
        if not self.enabled:
            return self
        try:
            nvml, handle = self._nvml_handle()
            self.thread = threading.Thread(target=self._poll_nvml, args=(nvml, handle), daemon=True)
            self.thread.start()
            return self
        except Exception:
            self.thread = None
        try:
            self.process = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.process = None
        return self

    def _read(self):
        for line in self.process.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.samples.append(parts)

    def __exit__(self, *exc):
        self.stop.set()
        if self.thread is not None:
            self.thread.join(timeout=1.0)
        if self.process is not None:
            self.process.terminate()
        return False

    def summary(self) -> dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        clocks = sorted(int(s[0]) for s in self.samples)
        reasons = [name for i, name in enumerate(self.NAMES)
                   if any(s[2 + i].lower().startswith("active") for s in self.samples)]
        return {"sm_mhz": clocks[len(clocks) // 2], "sm_max_mhz": int(self.samples[0][1]),
                "reasons": reasons, "samples": len(self.samples)}


def device_uuid(index: int) -> str | None:
    try:
        import torch
        return str(torch.cuda.get_device_properties(index).uuid)
    except Exception:
        return None


def env_ranks() -> tuple[int, int, int]:
    return (int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)),
            int(os.environ.get("LOCAL_RANK", 0)))


def emit(payload: dict) -> None:
    print(json.dumps(payload), flush=True)


# ------------------------------------------------------------------ ours ------
def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    sys.path.insert(0, str(ROOT))
    from systems_for_llms_b200.config import DataConfig, ModelConfig, TrainConfig
    from systems_for_llms_b200.data import gather_windows, load_data
    from systems_for_llms_b200.ops import lib as kernel_lib
    from systems_for_llms_b200.ops.gemm import check_status
    from systems_for_llms_b200.parallel import train as runner
    from systems_for_llms_b200.train import autocast, learning_rate

    rank, world, local_rank = env_ranks()
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}; launch with torch.distributed.run")
    mode = args.mode or ("single" if world == 1 else "ddp")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    raw = train_config_dict(args.steps + args.warmup, args.checkpointing)
    config = TrainConfig(model=ModelConfig(**raw.pop("model")), data=DataConfig(**raw.pop("data")),
                         **raw)
    config.validate()
    torch.set_float32_matmul_precision("highest")
    torch.manual_seed(config.seed)
    train_data, _, _ = load_data(config)
    from dataclasses import asdict
    from systems_for_llms_b200.models.transformer import TransformerLM
    base = TransformerLM(**asdict(config.model), device=device, dtype=torch.float32)
    strategy = runner.Strategy(mode, base, config, device, world=world, rank=rank,
                               sync_policy="last", bucket_cap_mb=args.bucket_cap_mb)
    if strategy.engine is None:
        # the portable PyTorch-operator path is the oracle, not the product: never time it
        raise SystemExit("the sm_100a fused engine did not engage for this model and mode; "
                         "refusing to benchmark the portable path")
    from systems_for_llms_b200.parallel.comm import reset_symmetric_peak, symmetric_memory_bytes
    accumulation = runner.validate_layout(mode, world, GLOBAL_BATCH, MICROBATCH, "last")
    sampler = torch.Generator(device="cpu").manual_seed(config.seed + 1)
    tokens_per_step = GLOBAL_BATCH * SEQ
    strategy.model.train()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def set_lr(step):
        for group in strategy.optimizer.param_groups:
            group["lr"] = learning_rate(step, config)

    # ---- device-timed loop: batches already on the device ----------------------
    local_batch = GLOBAL_BATCH if mode == "tp" else GLOBAL_BATCH // world
    starts = torch.randint(len(train_data) - SEQ, (GLOBAL_BATCH,), generator=sampler)
    mine = starts if mode == "tp" else starts[rank * local_batch:(rank + 1) * local_batch]
    resident = gather_windows(train_data, mine.tolist(), SEQ).to(device)
    micro = [(resident[b:b + MICROBATCH, :-1], resident[b:b + MICROBATCH, 1:])
             for b in range(0, local_batch, MICROBATCH)]

    def device_step():
        strategy.optimizer.zero_grad(set_to_none=True)
        for index, (x, y) in enumerate(micro):
            with strategy.microbatch_context(last=index == accumulation - 1):
                with autocast(config, device):
                    loss = strategy.model.loss(x, y, 1.0 / accumulation)
                loss.backward()
                strategy.after_backward()
        return strategy.reduce_and_update()

    for step in range(args.warmup):
        set_lr(step)
        device_step()
    barrier()
    check_status(device)
    torch.cuda.reset_peak_memory_stats(device)
    reset_symmetric_peak()
    launches_before = kernel_lib.launch_count()
    begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local_rank, device_uuid(local_rank), enabled=rank == 0) as clocks:
        begin.record()
        for step in range(args.steps):
            set_lr(args.warmup + step)
            device_step()
        end.record()
        barrier()
    device_ms = begin.elapsed_time(end)
    launches = kernel_lib.launch_count() - launches_before
    check_status(device)

    # ---- end-to-end loop through the public step function ----------------------
    # Its own warm-up: the first call through this path pays one-time costs the
    # device loop never met (pinned staging buffers, NCCL's first all-reduce of the
    # step statistics), which would otherwise be spread over a handful of timed steps.
    for step in range(args.warmup):
        set_lr(args.warmup + args.steps)
        runner.train_step(strategy, train_data, config, sampler, device,
                          global_batch_size=GLOBAL_BATCH, microbatch_size=MICROBATCH)
    barrier()
    e2e_begin, e2e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    tick = time.perf_counter()
    e2e_begin.record()
    for step in range(args.steps):
        set_lr(args.warmup + args.steps + step)
        values = runner.train_step(strategy, train_data, config, sampler, device,
                                   global_batch_size=GLOBAL_BATCH, microbatch_size=MICROBATCH)
    e2e_end.record()
    barrier()
    # every step ends with a host read of its result, so the device's clock and the
    # host's agree; report the longer of the two
    e2e_seconds = max(time.perf_counter() - tick, e2e_begin.elapsed_time(e2e_end) / 1e3)
    peak = torch.cuda.max_memory_allocated(device)
    symmetric = symmetric_memory_bytes()["peak"]
    optimizer_bytes = strategy.optimizer_state_bytes()
    if world > 1:
        stats = torch.tensor([device_ms, e2e_seconds, float(peak), float(peak + symmetric),
                              float(optimizer_bytes)], device=device, dtype=torch.float64)
        dist.all_reduce(stats, op=dist.ReduceOp.MAX)
        device_ms, e2e_seconds, peak, true_peak, optimizer_bytes = stats.tolist()
    else:
        true_peak = peak + symmetric
    if rank == 0:
        value = args.steps * tokens_per_step / (device_ms / 1e3)
        published = published_for(mode, world, args.checkpointing)
        emit({
            "metric": METRIC, "value": value, "unit": "tokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": device_ms / args.steps,
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": value / published if published else None, "dtype": "bf16",
            "data": "synthetic uniform-random token ids, random-init weights", "impl": "ours",
            "config": {"model": "324M decoder (24 layers, d_model 1024, 16 heads, d_ff 2752, vocab 10000)",
                       "global_batch": GLOBAL_BATCH, "seq_len": SEQ, "microbatch": MICROBATCH,
                       "parallelism": f"{mode}-{world}gpu" if world > 1 else "single",
                       "checkpointing": args.checkpointing,
                       "cache": "working set (weights, gradients, optimizer state, activations: "
                                "several GB) far exceeds the 126 MB L2 between steps"},
            "clocks": clocks.summary(),
            "e2e": {"value": args.steps * tokens_per_step / e2e_seconds, "unit": "tokens/s",
                    "h2d_bytes_per_step": GLOBAL_BATCH * (SEQ + 1) * 8,
                    "d2h_bytes_per_step": 4 * 4 * world, "last_loss": values["loss"]},
            "gpu_launches": launches, "peak_allocated_gib": peak / 2 ** 30,
            # buffers mapped on peer GPUs are allocated outside PyTorch's allocator
            "peak_with_symmetric_gib": true_peak / 2 ** 30,
            "optimizer_state_gib_max_rank": optimizer_bytes / 2 ** 30,
            "execution_path": "sm_100a fused engine",
            "published_reference_tokens_per_s": published,
        })
    strategy.close()
    if world > 1:
        dist.destroy_process_group()


# ------------------------------------------------------------- reference ------
def run_reference(args) -> None:
    rank, world, _ = env_ranks()
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "llmlab").is_dir() or not (ref / "llmdist").is_dir():
        if rank == 0:
            emit({"impl": "reference", "unavailable": "baseline/_ref does not contain the reference packages"})
        return
    # Nothing of this repository may be importable on this path.
    sys.path[:] = [str(ref)] + [p for p in sys.path if Path(p or ".").resolve() != ROOT]
    for name in list(sys.modules):
        if name.split(".")[0] in ("llmlab", "llmdist", "systems_for_llms_b200"):
            del sys.modules[name]
    try:
        import llmdist.train as ref_runner
        from llmlab.config import DataConfig, ModelConfig, TrainConfig
    except Exception as error:  # pragma: no cover - depends on the box
        if rank == 0:
            emit({"impl": "reference", "unavailable": f"import failed: {error!r}"[:200]})
        return
    mode = args.mode or ("single" if world == 1 else "ddp")
    raw = train_config_dict(args.steps + args.warmup, args.checkpointing)
    raw["max_steps"] = max(args.steps + args.warmup, 7)
    raw["eval_interval"] = raw["max_steps"]
    raw["eval_batches"] = 8
    config = TrainConfig(model=ModelConfig(**raw.pop("model")), data=DataConfig(**raw.pop("data")),
                         **raw)
    workdir = Path(tempfile.mkdtemp(prefix="ref-bench-")) / "run" if rank == 0 else None
    if world > 1:
        # every rank needs the same path; rank 0's temp name is passed through a file
        marker = Path(tempfile.gettempdir()) / f"ref-bench-{os.environ.get('MASTER_PORT', '0')}"
        if rank == 0:
            marker.write_text(str(workdir))
        else:
            for _ in range(600):
                if marker.exists() and marker.read_text():
                    break
                time.sleep(0.1)
            workdir = Path(marker.read_text())
    with ClockSampler(env_ranks()[2], device_uuid(env_ranks()[2]), enabled=rank == 0) as clocks:
        summary = ref_runner.run(config, workdir, mode=mode, global_batch_size=GLOBAL_BATCH,
                                 microbatch_size=MICROBATCH, warmup_steps=args.warmup,
                                 sync_policy="last", bucket_cap_mb=25.0)
    if rank == 0:
        published = published_for(mode, world, args.checkpointing)
        emit({
            "metric": METRIC, "value": summary["tokens_per_second"], "unit": "tokens/s",
            "n_gpus": world, "steps": summary["measured_steps"], "warmup": args.warmup,
            "ms_per_step": 1e3 * summary["measured_train_seconds"] / summary["measured_steps"],
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": summary["tokens_per_second"] / published if published else None,
            "dtype": "bf16", "data": "synthetic uniform-random token ids, random-init weights",
            "impl": "reference",
            "config": {"model": "324M decoder (24 layers, d_model 1024, 16 heads, d_ff 2752, vocab 10000)",
                       "global_batch": GLOBAL_BATCH, "seq_len": SEQ, "microbatch": MICROBATCH,
                       "parallelism": f"{mode}-{world}gpu" if world > 1 else "single",
                       "checkpointing": args.checkpointing,
                       "timing": "the reference's own host-timed synchronized steps, max over ranks"},
            "clocks": clocks.summary(),
            "e2e": {"value": summary["tokens_per_second"], "unit": "tokens/s",
                    "h2d_bytes_per_step": GLOBAL_BATCH * (SEQ + 1) * 8,
                    "d2h_bytes_per_step": 3 * 4 * world},
            "peak_allocated_gib": (summary["peak_cuda_allocated_bytes"] or 0) / 2 ** 30,
            "optimizer_state_gib_max_rank":
                (summary.get("optimizer_state_bytes_max_rank") or 0) / 2 ** 30,
        })


def main() -> None:
    global GLOBAL_BATCH, MICROBATCH, SEQ
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", choices=["ours", "reference"], default="ours")
    parser.add_argument("--mode", choices=["single", "naive", "ddp", "zero1", "fsdp", "tp"])
    parser.add_argument("--checkpointing", choices=["none", "block"], default="none")
    parser.add_argument("--bucket-cap-mb", type=float, default=25.0)
    parser.add_argument("--seq-len", type=int, default=SEQ)
    parser.add_argument("--global-batch", type=int, default=GLOBAL_BATCH)
    parser.add_argument("--microbatch", type=int, default=MICROBATCH)
    args = parser.parse_args()
    if args.warmup < 3:
        parser.error("--warmup must be at least 3")
    if min(args.seq_len, args.global_batch, args.microbatch) < 1:
        parser.error("--seq-len, --global-batch and --microbatch must be positive")
    GLOBAL_BATCH, MICROBATCH, SEQ = args.global_batch, args.microbatch, args.seq_len
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
