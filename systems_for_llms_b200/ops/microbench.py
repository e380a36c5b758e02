"""Kernel-level timings of this library at the shapes of the 324M training step.

    python -m systems_for_llms_b200.ops.microbench gemm        # every GEMM of one layer
    python -m systems_for_llms_b200.ops.microbench attention   # fwd / bwd at B4 H16 N1024 D64
    python -m systems_for_llms_b200.ops.microbench elementwise # norms, loss, optimizer
    python -m systems_for_llms_b200.ops.microbench decode      # split-KV decode, B8 GQA 32/4 N16384
    python -m systems_for_llms_b200.ops.microbench step        # per-kernel table of one step
    python -m systems_for_llms_b200.ops.microbench once NAME   # a few launches of one op
    python -m systems_for_llms_b200.ops.microbench mma         # tcgen05.mma issue-rate test
    python -m systems_for_llms_b200.ops.microbench sfu         # exponentials per tile: ex2 forms, polynomials
    SFL_LIBRARY=/tmp/libsfl_trace.so python -m systems_for_llms_b200.ops.microbench \
        attention-phases                                       # phase timers, needs a library built with
                                                               # ops.build -DSFL_ATTN_TRACE --output /tmp/libsfl_trace.so
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m systems_for_llms_b200.ops.microbench tp             # GEMM + all-reduce, one kernel vs two
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \
        -m systems_for_llms_b200.ops.microbench comm           # peer-memory collectives vs NCCL

Each timing is the median of CUDA-event measurements with a 256 MB buffer
written between launches, so operands come from HBM rather than from a warm L2.
Rates are printed next to their fraction of a roofline denominator: the measured
cuBLAS bf16 throughput and copy bandwidth in ``MEASURED_PEAKS.json`` at the
repository root when that file exists, otherwise 1590 TFLOP/s and 6650 GB/s.
``once`` exists so that a profiler can capture a named kernel from a process that
does little else; ``--json`` prints one machine-readable line instead of a table.
"""

from __future__ import annotations

import argparse
import json
import statistics
from pathlib import Path

import torch

M_TOKENS, D_MODEL, D_FF, SEQ, HEADS, VOCAB = 4096, 1024, 2752, 1024, 16, 10000
FALLBACK_PEAKS = {"bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "hbm_gbs": 6650.0}


def peaks() -> tuple[dict, str]:
    path = Path(__file__).resolve().parents[2] / "MEASURED_PEAKS.json"
    if path.is_file():
        data = json.loads(path.read_text())
        if all(key in data for key in FALLBACK_PEAKS):
            return {key: float(data[key]) for key in FALLBACK_PEAKS}, "of measured"
    return dict(FALLBACK_PEAKS), "of fallback"


def rnd(*shape, scale=1.0):
    return (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)


def timeit(fn, iters: int = 30, warmup: int = 5) -> float:
    """Median microseconds per call, L2 flushed between calls."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    flush = torch.empty(256 * 2 ** 20, dtype=torch.uint8, device="cuda")
    samples = []
    for _ in range(iters):
        flush.zero_()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        fn()
        end.record()
        end.synchronize()
        samples.append(begin.elapsed_time(end) * 1000)
    return statistics.median(samples)


def rope_tables(seq: int, dim: int):
    inv = 1.0 / (10000.0 ** (torch.arange(0, dim, 2, device="cuda").float() / dim))
    angles = torch.arange(seq, device="cuda").float()[:, None] * inv[None]
    return tuple(f(angles).bfloat16().float().contiguous() for f in (torch.cos, torch.sin))


def gemm_ops() -> dict:
    """name -> (callable, flops, algorithmic bytes) for every GEMM of one block + the head."""
    from . import gemm as G
    M, C, F, dk = M_TOKENS, D_MODEL, D_FF, D_MODEL // HEADS
    x, res = rnd(M, C), torch.randn(M, C, device="cuda")
    wqkv, wo = rnd(3 * C, C, scale=0.03), rnd(C, C, scale=0.03)
    w13, w2 = rnd(2 * F, C, scale=0.03), rnd(C, F, scale=0.03)
    cos, sin = rope_tables(SEQ, dk)
    qkv = torch.empty(M, 3 * C, dtype=torch.bfloat16, device="cuda")
    ro = torch.empty(M, C, device="cuda")
    g, a13 = G.swiglu_fwd(x, w13, F)
    dy = rnd(M, C)
    d13 = G.swiglu_bwd(dy, w2, a13)
    dx = torch.empty(M, C, dtype=torch.bfloat16, device="cuda")
    G.linear_fwd_rope(x, wqkv, cos, sin, SEQ, 2 * C, dk, qkv)
    logits = torch.empty(M, VOCAB, dtype=torch.bfloat16, device="cuda")
    whead = rnd(VOCAB, C, scale=0.03)
    grads = {"qkv": torch.zeros(3 * C, C, device="cuda"), "wo": torch.zeros(C, C, device="cuda"),
             "w13": torch.zeros(2 * F, C, device="cuda"), "w2": torch.zeros(C, F, device="cuda")}
    group = [(dy, g, grads["w2"], True), (d13, x, grads["w13"], True),
             (dy, x, grads["wo"], True), (qkv, x, grads["qkv"], True)]
    b16, b32 = 2, 4

    def flops(m, n, k):
        return 2.0 * m * n * k

    ops = {
        "qkv_rope": (lambda: G.linear_fwd_rope(x, wqkv, cos, sin, SEQ, 2 * C, dk, qkv),
                     flops(M, 3 * C, C), b16 * (M * C + 3 * C * C + M * 3 * C)),
        "wo_resid": (lambda: G.linear_fwd_resid(x, wo, res, ro),
                     flops(M, C, C), b16 * (M * C + C * C) + 2 * b32 * M * C),
        "w13_swiglu": (lambda: G.swiglu_fwd(x, w13, F),
                       flops(M, 2 * F, C), b16 * (M * C + 2 * F * C + 3 * M * F)),
        "w2_resid": (lambda: G.linear_fwd_resid(g, w2, res, ro),
                     flops(M, C, F), b16 * (M * F + C * F) + 2 * b32 * M * C),
        "swiglu_bwd": (lambda: G.swiglu_bwd(dy, w2, a13),
                       flops(M, F, C), b16 * (M * C + C * F + 4 * M * F)),
        "dgrad_w13": (lambda: G.linear_dgrad(d13, w13, dx),
                      flops(M, C, 2 * F), b16 * (2 * M * F + 2 * F * C + M * C)),
        "dgrad_qkv": (lambda: G.linear_dgrad(qkv, wqkv, dx),
                      flops(M, C, 3 * C), b16 * (3 * M * C + 3 * C * C + M * C)),
        "dgrad_wo": (lambda: G.linear_dgrad(dy, wo, dx),
                     flops(M, C, C), b16 * (2 * M * C + C * C)),
        "wgrad_group": (lambda: G.wgrad_grouped(group),
                        flops(M, C, F) + flops(M, 2 * F, C) + flops(M, C, C) + flops(M, 3 * C, C),
                        b16 * M * (C + F + 2 * F + C + C + C + 3 * C + C)
                        + 2 * b32 * (3 * C * C + C * C + 3 * F * C)),
        "head": (lambda: G.linear_fwd(x, whead, logits),
                 flops(M, VOCAB, C), b16 * (M * C + VOCAB * C + M * VOCAB)),
    }
    return ops


def attention_ops(B=4, H=HEADS, N=SEQ, D=64) -> dict:
    from ..attention import flash, masks
    q, k, v, upstream = (torch.randn(B, H, N, D, device="cuda").bfloat16() for _ in range(4))
    out = torch.empty_like(q)
    lse = torch.empty(B, H, N, device="cuda")
    mask = flash.prepare_mask(q, None, masks.MaskSpec(causal=True), None, "interval")
    grads = [torch.empty_like(q) for _ in range(3)]
    cos, sin = rope_tables(N, D)
    scale = D ** -0.5
    flash.flash_fwd(q, k, v, out, lse, mask, scale)
    causal = 4.0 * B * H * N * N * D * 0.5
    io = 2 * B * H * N * D
    return {
        "attn_fwd": (lambda: flash.flash_fwd(q, k, v, out, lse, mask, scale), causal, 4 * io),
        "attn_bwd": (lambda: flash.flash_bwd(q, k, v, out, upstream, lse, *grads, mask, scale,
                                             rope=(cos, sin)), 2.5 * causal, 8 * io),
    }


def elementwise_ops() -> dict:
    from . import functional as K
    M, C = M_TOKENS, D_MODEL
    x = torch.randn(M, C, device="cuda")
    w = torch.ones(C, device="cuda")
    h, rstd = K.rmsnorm(x, w, 1e-5)
    dy, dres = rnd(M, C), torch.randn(M, C, device="cuda")
    dw = torch.zeros(C, device="cuda")
    logits = rnd(M, VOCAB)
    dlogits = torch.empty_like(logits)
    targets = torch.randint(0, VOCAB, (M,), device="cuda")
    n_opt = 64 * 2 ** 20                     # 64M parameters: 1.2 GB over the five streams
    param, grad, m1, m2 = (torch.randn(n_opt, device="cuda") * 0.01 for _ in range(4))
    m2.abs_()
    shadow = torch.empty(n_opt, dtype=torch.bfloat16, device="cuda")
    return {
        "adamw": (lambda: K.adamw_step(param, grad, m1, m2, shadow, step=3, lr=1e-4, beta1=0.9,
                                       beta2=0.95, eps=1e-8, weight_decay=0.1), 0.0,
                  n_opt * (4 * 4 + 3 * 4 + 2)),
        "rmsnorm_fwd": (lambda: K.rmsnorm(x, w, 1e-5), 0.0, M * C * (4 + 2)),
        "rmsnorm_bwd": (lambda: K.rmsnorm_bwd(dy, x, w, rstd, dres, dw, True, want_bf16=True),
                        0.0, M * C * (2 + 4 + 4 + 4 + 2)),
        "cross_entropy": (lambda: K.cross_entropy_rows(logits, targets, VOCAB, dlogits, 1.0), 0.0,
                          2 * M * VOCAB * 2),
    }


def decode_ops() -> dict:
    """Split-KV decode at a batched GQA serving shape (B8, 32 query / 4 KV heads, D 128,
    16,384 cached tokens: 268 MB of K and V, so every call streams from HBM)."""
    from ..attention.decode import prepare
    B, Hq, Hkv, N, D = 8, 32, 4, 16384, 128
    q = rnd(B, Hq, D)
    k, v = rnd(B, Hkv, N, D), rnd(B, Hkv, N, D)
    nbytes = 2 * B * Hkv * N * D * 2
    ops = {}
    for variant, splits in (("mma", 4), ("tile", 4)):
        ops[f"decode_{variant}"] = (prepare(q, k, v, splits=splits, variant=variant), 0.0, nbytes)
    return ops


SUITES = {"gemm": gemm_ops, "attention": attention_ops, "elementwise": elementwise_ops,
          "decode": decode_ops}


def run_suite(name: str) -> list[dict]:
    from .gemm import check_status
    reference, label = peaks()
    rows = []
    for op, (fn, flops, nbytes) in SUITES[name]().items():
        micros = timeit(fn)
        row = {"op": op, "us": micros, "denominator": label}
        if flops:
            row["tflops"] = flops / micros / 1e6
            row["frac_bf16_burst"] = row["tflops"] / reference["bf16_tflops"]
            row["frac_bf16_sustained"] = row["tflops"] / reference["bf16_tflops_sustained"]
        row["gbs"] = nbytes / micros / 1e3
        row["frac_hbm"] = row["gbs"] / reference["hbm_gbs"]
        rows.append(row)
    torch.cuda.synchronize()
    check_status()
    return rows


def print_rows(rows: list[dict]) -> None:
    print(f"{'op':14s} {'us':>9s} {'TFLOP/s':>9s} {'burst':>7s} {'sust.':>7s} {'GB/s':>8s} "
          f"{'hbm':>6s}   ({rows[0]['denominator']})")
    for row in rows:
        tf = f"{row['tflops']:9.1f} {row['frac_bf16_burst']:7.2f} {row['frac_bf16_sustained']:7.2f}" \
            if "tflops" in row else f"{'':9s} {'':7s} {'':7s}"
        print(f"{row['op']:14s} {row['us']:9.1f} {tf} {row['gbs']:8.0f} {row['frac_hbm']:6.2f}")
    print(f"{'total':14s} {sum(r['us'] for r in rows):9.1f}")


def step_table(steps: int = 3) -> dict:
    """Wall time of the flagship training step and its per-kernel device time."""
    import time

    from ..models.transformer import TransformerLM
    from ..optim import FusedAdamW
    from .gemm import check_status
    torch.manual_seed(0)
    model = TransformerLM(vocab_size=VOCAB, context_length=SEQ, d_model=D_MODEL, num_layers=24,
                          num_heads=HEADS, d_ff=D_FF, rope_theta=10000.0, attention_backend="sdpa",
                          device="cuda", dtype=torch.float32)
    optimizer = FusedAdamW(model.parameters(), lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    x = torch.randint(0, VOCAB, (4, SEQ), device="cuda")
    y = torch.randint(0, VOCAB, (4, SEQ), device="cuda")

    def step(accumulation=8):
        optimizer.zero_grad(set_to_none=True)
        for _ in range(accumulation):
            with torch.autocast("cuda", dtype=torch.bfloat16):
                loss = model.loss(x, y, 1.0 / accumulation)
            loss.backward()
        optimizer.engine = model._fused
        return optimizer.clip_and_step(1.0)

    for _ in range(2):
        step()
    torch.cuda.synchronize()
    check_status()
    begin = time.perf_counter()
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    seconds = (time.perf_counter() - begin) / steps
    from torch.profiler import ProfilerActivity, profile
    with profile(activities=[ProfilerActivity.CUDA]) as prof:
        step()
        torch.cuda.synchronize()
    events = sorted(prof.key_averages(), key=lambda e: -e.device_time_total)[:24]
    return {"step_ms": seconds * 1e3, "tokens_per_s": 32 * SEQ / seconds,
            "peak_gib": torch.cuda.max_memory_allocated() / 2 ** 30,
            "note": "kernel times come from a profiled step; the wall time does not",
            "kernels": [{"name": e.key[:90], "ms": e.device_time_total / 1e3, "launches": e.count}
                        for e in events]}


def tensor_parallel_table(iters: int = 30) -> dict:
    """The four sharded-reduction products of a tensor-parallel layer (one process per
    GPU): the GEMM followed by the peer-memory reduction kernel against the single
    kernel that does both, CUDA-event time per call as the max over ranks, and the
    fused kernel's own phase times (CTA 0, first tile)."""
    import ctypes
    import os

    import torch.distributed as dist

    from ..parallel.tensor_parallel import TensorParallelComm
    from . import gemm as G
    from . import lib as L
    from .gemm import check_status
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    tp = TensorParallelComm(device, None, num_layers=1)
    M, d = M_TOKENS, D_MODEL
    aw, dff = D_MODEL // world, D_FF // world
    torch.manual_seed(rank)
    resid = torch.randn(M, d, device=device)
    cases = {   # name: (activations, weight, weight is [K, N])
        "wo_resid": (rnd(M, aw), rnd(d, aw, scale=aw ** -0.5), False),
        "w2_resid": (rnd(M, dff), rnd(d, dff, scale=dff ** -0.5), False),
        "dgrad_w13": (rnd(M, 2 * dff), rnd(2 * dff, d, scale=d ** -0.5), True),
        "dgrad_qkv": (rnd(M, 3 * aw), rnd(3 * aw, d, scale=d ** -0.5), True),
    }

    def two_kernels(a, w, b_mn):
        if b_mn:
            return tp.reduce_bf16(G.linear_dgrad(a, w, tp.partial(M, d)))
        return tp.reduce_residual(G.linear_fwd(a, w, tp.partial(M, d)), resid, 0)

    def one_kernel(a, w, b_mn):
        return tp.gemm_reduce_bf16(a, w) if b_mn else tp.gemm_reduce_residual(a, w, resid, 1)

    def timed(fn, args) -> float:
        for _ in range(5):
            fn(*args)
        samples = []
        for _ in range(iters):
            dist.barrier()
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            for _ in range(4):          # back to back, as inside a layer
                fn(*args)
            end.record()
            end.synchronize()
            samples.append(begin.elapsed_time(end) * 250)
        worst = torch.tensor(statistics.median(samples), device=device)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        return worst.item()

    rows = []
    for name, args in cases.items():
        K = args[0].shape[1]
        rows.append({"op": name, "k_per_rank": K, "two_kernels_us": timed(two_kernels, args),
                     "one_kernel_us": timed(one_kernel, args),
                     "link_mb_per_rank": M * d * 2 / 2 ** 20 if world == 2
                     else M * d * (2 + (2 if args[2] else 4)) * (world - 1) / world / 2 ** 20})
    counters = torch.zeros(6, dtype=torch.int64, device=device)
    handle = L.lib()._handle
    handle.sfl_gemm_tp_set_trace.argtypes = [ctypes.c_void_p]
    handle.sfl_gemm_tp_set_trace(counters.data_ptr())
    for _ in range(50):
        one_kernel(*cases["w2_resid"])
    torch.cuda.synchronize()
    handle.sfl_gemm_tp_set_trace(None)
    check_status()
    values = counters.tolist()
    phases = {name: values[i] / max(values[5], 1) / 1e3 for i, name in enumerate(
        ("accumulator_ready", "peers_entered", "strip_sent", "peer_strips_arrived", "rows_finished"))}
    dist.barrier()
    tp.close()
    dist.destroy_process_group()
    return {"rank": rank, "world": world, "rows": rows, "w2_resid_phase_us": phases}


LINK_GBS = 770.0      # measured peer copy, per direction per GPU, on this pool's NVLink 5


def collective_table(iters: int = 10) -> dict:
    """The data-parallel collectives at the size of the 324M gradient (one process per
    GPU): this library's peer-memory kernels against ``torch.distributed`` (NCCL),
    CUDA-event time as the max over ranks, and the fraction of the link roofline
    (bytes that must enter each GPU over NVLink / 770 GB/s)."""
    import os

    import torch.distributed as dist

    from ..parallel.comm import PeerComm, SymmetricBuffer
    from .gemm import check_status
    rank, world, local = (int(os.environ[k]) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK"))
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=device)
    comm = PeerComm(device, ctas=32)
    n = 324_000_000 // (4 * world * 64) * (4 * world * 64)      # fp32 elements, sliceable
    grads = SymmetricBuffer(n * 4, device)
    params, shadows = SymmetricBuffer(n * 4, device), SymmetricBuffer(n * 2, device)
    flat = grads.view(torch.float32, n)
    flat.normal_()
    per = n // world
    shard, m, v = (torch.zeros(per, device=device) for _ in range(3))
    plain = torch.randn(n, device=device)
    pieces = torch.empty(n, device=device, dtype=torch.bfloat16)
    piece = torch.randn(per, device=device).bfloat16()
    stats = torch.tensor([1.0, 1.0, 1.0], device=device)
    slots = iter(range(0, 48))

    def timed(fn) -> float:
        for _ in range(2):
            fn()
        samples = []
        for _ in range(iters):
            dist.barrier()
            torch.cuda.synchronize()
            begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            begin.record()
            fn()
            end.record()
            end.synchronize()
            samples.append(begin.elapsed_time(end) * 1000)
        worst = torch.tensor(statistics.median(samples), device=device)
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        return worst.item()

    s_ar, s_rs, s_ag, s_gather = (next(slots) for _ in range(4))
    share = (world - 1) / world
    cases = [
        # name, ours, NCCL, bytes entering each GPU
        ("allreduce_f32 (+1/W scale, norm partials)",
         lambda: comm.allreduce(grads, 0, n, 1.0 / world, s_ar),
         lambda: dist.all_reduce(plain), 2 * share * n * 4),
        ("reduce_scatter_f32 (+scale, norm partials)",
         lambda: comm.reduce_scatter(grads, 0, n, 1.0 / world, shard, s_rs),
         lambda: dist.reduce_scatter_tensor(shard, plain), share * n * 4),
        ("adamw + all-gather (fp32 params, bf16 copies)",
         lambda: comm.adamw_allgather(params, shadows, 0, n, shard, m, v, step=1, lr=1e-3,
                                      beta1=0.9, beta2=0.95, eps=1e-8, weight_decay=0.1,
                                      coef=stats[1:2], ok=stats[2:3], slot=s_ag),
         lambda: dist.all_gather_into_tensor(plain, shard), share * n * 6),
        ("all-gather of bf16 shards (pull)",
         lambda: comm.allgather_bytes(shadows, 0, per * 2, s_gather),
         lambda: dist.all_gather_into_tensor(pieces, piece), share * n * 2),
    ]
    rows = []
    for name, ours, nccl, link_bytes in cases:
        mine, theirs = timed(ours), timed(nccl)
        floor = link_bytes / (LINK_GBS * 1e9) * 1e6
        rows.append({"op": name, "us": mine, "nccl_us": theirs, "link_mb": link_bytes / 2 ** 20,
                     "link_floor_us": floor, "frac_of_link_roofline": floor / mine})
    torch.cuda.synchronize()
    check_status()
    dist.barrier()
    for buffer in (grads, params, shadows):
        buffer.close()
    comm.close()
    dist.destroy_process_group()
    return {"rank": rank, "world": world, "elements": n, "rows": rows}


def mma_issue_rate(name: str = "mma_issue_rate") -> str:
    """Compile ops/<name>.cu for sm_100a into a temporary directory and run it."""
    import subprocess
    import tempfile

    from . import build as builder
    source = Path(__file__).with_name(f"{name}.cu")
    with tempfile.TemporaryDirectory() as scratch:
        binary = Path(scratch) / name
        subprocess.run(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17",
                        "--expt-relaxed-constexpr", "-I", str(builder.CSRC), "-o", str(binary),
                        str(source)], check=True)
        return subprocess.run([str(binary)], check=True, capture_output=True, text=True,
                              timeout=120).stdout


def attention_phases(batch: int = 8, heads: int = 16, length: int = 4096, dim: int = 64,
                     repeats: int = 5) -> str:
    """Phase timers of the attention kernels (cycles of one traced CTA, per tile).

    Needs a library built with ``-DSFL_ATTN_TRACE`` (``SFL_LIBRARY`` points at it); the
    ordinary build has no timers and the readers return -1.
    """
    import ctypes

    from ..attention import flash, masks
    from . import lib as L
    handle = L.lib()
    q, k, v, d_out = (torch.randn(batch, heads, length, dim, device="cuda").bfloat16()
                      for _ in range(4))
    out, lse = torch.empty_like(q), torch.empty(batch, heads, length, device="cuda")
    dq, dk, dv = (torch.empty_like(q) for _ in range(3))
    mask = flash.prepare_mask(q, None, masks.MaskSpec(causal=True), None, "interval")
    scale = dim ** -0.5

    def forward():
        flash.flash_fwd(q, k, v, out, lse, mask, scale)

    def backward():
        flash.flash_bwd(q, k, v, out, d_out, lse, dq, dk, dv, mask, scale)

    for _ in range(2):
        forward()
        backward()
    torch.cuda.synchronize()
    fwd, bwd = (ctypes.c_ulonglong * 16)(), (ctypes.c_ulonglong * 32)()
    if handle.sfl_attn_trace_read(fwd) != 0 or handle.sfl_attn_bwd_trace_read(bwd) != 0:
        raise SystemExit("this library has no phase timers: build one with "
                         "python -m systems_for_llms_b200.ops.build -DSFL_ATTN_TRACE --output PATH "
                         "and point SFL_LIBRARY at it")
    lines = []
    pairs = batch * heads * (length // 128) * (length // 128 + 1) / 2
    for name, call, reader, buffer in (("forward", forward, handle.sfl_attn_trace_read, fwd),
                                       ("backward", backward, handle.sfl_attn_bwd_trace_read, bwd)):
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(repeats):
            call()
        end.record()
        torch.cuda.synchronize()
        ms = begin.elapsed_time(end) / repeats
        reader(buffer)
        lines.append(f"{name}: B{batch} H{heads} N{length} D{dim} causal, {ms:.3f} ms per call, "
                     f"{ms * 1e6 * 148 / pairs:.0f} ns per 128 x 128 tile and SM")
        if name == "forward":
            t = [x / repeats for x in buffer]
            tiles, products = max(t[5], 1), max(t[12], 1)
            lines.append(f"  softmax warp, per tile: wait scores {t[0] / tiles:.0f}, load {t[1] / tiles:.0f}, "
                         f"maximum {t[2] / tiles:.0f}, wait P V {t[6] / tiles:.0f}, exponentials + store "
                         f"{t[3] / tiles:.0f} cycles ({tiles:.0f} tiles)")
            lines.append(f"  MMA warp, per tile: wait P / V {t[8] / products:.0f}, issue P V "
                         f"{t[9] / products:.0f}, wait K / free scores {t[10] / products:.0f}, issue Q K "
                         f"{t[11] / products:.0f} cycles")
            continue
        for kernel, base in (("dQ kernel", 0), ("dK/dV kernel", 16)):
            t = [x / repeats for x in buffer[base:base + 16]]
            tiles, halves = max(t[5], 1), max(t[12], 1)
            lines.append(f"  {kernel}, compute warpgroup 0, per tile: set-up {t[0] / tiles:.0f}, wait scores "
                         f"{t[1] / tiles:.0f}, load S and dP {t[3] / tiles:.0f}, exponentials + dS + store "
                         f"{t[4] / tiles:.0f}, publish {t[2] / tiles:.0f} cycles ({tiles:.0f} tiles)")
            lines.append(f"  {kernel}, MMA warp, per 64-column half: wait P / dS {t[9] / halves:.0f}, issue "
                         f"accumulation {t[10] / halves:.0f}, wait tile + issue scores {t[8] / halves:.0f} "
                         f"cycles; SM clock {t[13] / max(t[15], 1):.2f} GHz")
            if t[7] or t[11] or t[14]:      # library also built with -DSFL_ATTN_TRACE_SERIAL
                lines.append(f"  {kernel}, MMA warp waiting for each batch it issued: a score batch takes "
                             f"{t[7] / halves:.0f} cycles to issue into the idle pipe and completes "
                             f"{t[11] / halves:.0f} later; an accumulation batch completes "
                             f"{t[14] / halves:.0f} after its issue")
    return "\n".join(lines) + "\n"


def main() -> None:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("what", choices=[*SUITES, "step", "once", "mma", "sfu", "tp", "comm",
                                         "attention-phases"])
    parser.add_argument("name", nargs="?", help="operation for 'once' (e.g. w13_swiglu, attn_bwd)")
    parser.add_argument("--repeat", type=int, default=3)
    parser.add_argument("--json", action="store_true")
    args = parser.parse_args()
    if not torch.cuda.is_available():
        raise SystemExit("a CUDA GPU is required")
    if args.what == "mma":
        print(mma_issue_rate(), end="")
        return
    if args.what == "sfu":
        print(mma_issue_rate("sfu_rate"), end="")
        return
    if args.what == "attention-phases":
        print(attention_phases(), end="")
        return
    if args.what == "comm":
        table = collective_table()
        if table["rank"] == 0:
            if args.json:
                print(json.dumps(table))
                return
            print(f"{table['world']} ranks, {table['elements']} fp32 elements; microseconds, max over "
                  f"ranks; link roofline = bytes entering a GPU / {LINK_GBS:.0f} GB/s")
            for row in table["rows"]:
                print(f"{row['op']:46s} {row['us']:9.1f}  NCCL {row['nccl_us']:9.1f}  "
                      f"{row['link_mb']:8.1f} MB  floor {row['link_floor_us']:8.1f}  "
                      f"{row['frac_of_link_roofline']:.2f} of link roofline")
        return
    if args.what == "tp":
        table = tensor_parallel_table()
        if table["rank"] == 0:
            if args.json:
                print(json.dumps(table))
                return
            print(f"{table['world']} ranks, M {M_TOKENS}, N {D_MODEL}; microseconds per call, max over ranks")
            for row in table["rows"]:
                print(f"{row['op']:10s} K/rank {row['k_per_rank']:5d}  GEMM + reduce kernel "
                      f"{row['two_kernels_us']:7.1f}   one kernel {row['one_kernel_us']:7.1f}   "
                      f"({row['link_mb_per_rank']:.1f} MB per rank over NVLink)")
            print("w2_resid, CTA 0, first tile, microseconds per phase: " + ", ".join(
                f"{k} {v:.1f}" for k, v in table["w2_resid_phase_us"].items()))
        return
    if args.what == "once":
        from .gemm import check_status
        name = args.name or ""
        first = ("attention" if name.startswith("attn_") else "decode" if name.startswith("decode_")
                 else "elementwise" if name in ("adamw", "rmsnorm_fwd", "rmsnorm_bwd", "cross_entropy")
                 else "gemm")
        # the likely suite first, so that a profiler sees few launches before the one it wants
        for suite in [SUITES[first]] + [v for k, v in SUITES.items() if k != first]:
            ops = suite()
            if args.name in ops:
                for _ in range(args.repeat):
                    ops[args.name][0]()
                torch.cuda.synchronize()
                check_status()
                print(f"ran {args.name} x{args.repeat}")
                return
        raise SystemExit(f"unknown operation {args.name!r}")
    if args.what == "step":
        table = step_table()
        if args.json:
            print(json.dumps(table))
            return
        print(f"step {table['step_ms']:.1f} ms  {table['tokens_per_s']:.0f} tokens/s  "
              f"peak {table['peak_gib']:.2f} GiB")
        for row in table["kernels"]:
            print(f"{row['ms']:8.2f} ms {row['launches']:6d}  "
                  f"{row['ms'] / row['launches'] * 1000:8.1f} us  {row['name']}")
        return
    rows = run_suite(args.what)
    if args.json:
        print(json.dumps(rows))
    else:
        print_rows(rows)


if __name__ == "__main__":
    main()
