"""Bounded study of the differentiable attention: numerics, fwd+bwd timing, one optimizer step.

Three kinds of case, as in the reference's training study
(attention_lab/backward_study.py:86-337):

* ``numerical_case``        output, dQ, dK, dV of ``training_attention`` against a
                            dense fp32 autograd oracle that never reads a schedule.
* ``performance_case``      backward-only and forward+backward latency of the
                            structured kernel against SDPA (and, when asked,
                            compiled FlexAttention), each first checked against
                            the oracle; retained forward, warm-ups, capture and
                            replay all live on one explicit non-default stream.
* ``transformer_step_case`` a whole pre-norm block - loss, backward, SGD on fp32
                            master weights, weights restored on every call so each
                            timed step does identical work - timed eagerly for
                            every variant and checked by scale-aware comparison of
                            loss, output, gradients and update deltas.

The time budget is checked between cases.  A failed CUDA-graph capture raises
``TrainingCaptureError`` and ends the run, since the stream state after it is
not trustworthy.  Negative results are written like any other.
"""

from __future__ import annotations

import argparse
import gc
import json
import math
import platform
import statistics
import time
import traceback
from dataclasses import asdict
from pathlib import Path

from .masks import MaskSpec

CUSTOM = "structured_sm100"


def dense_attention(q, k, v, spec: MaskSpec, documents=None):
    """Differentiable oracle built from the spec alone."""
    import torch
    n = q.shape[-2]
    position = torch.arange(n, device=q.device)
    distance = position[:, None] - position[None, :]
    mask = torch.ones(n, n, dtype=torch.bool, device=q.device)
    if spec.causal:
        mask &= distance >= 0
    if spec.window_left is not None:
        mask &= distance <= spec.window_left
    if spec.window_right is not None:
        mask &= distance >= -spec.window_right
    if spec.same_document:
        labels = torch.tensor(list(documents), device=q.device)
        mask &= labels[:, None] == labels[None, :]
    scores = q @ k.transpose(-2, -1) * q.shape[-1] ** -0.5
    return scores.masked_fill(~mask, -float("inf")).softmax(-1) @ v


def comparison(actual, expected, dtype) -> dict:
    import torch
    atol, rtol = (0.025, 0.035) if dtype == torch.bfloat16 else (0.004, 0.006)
    delta = actual.detach().float() - expected.detach().float()
    finite = bool(torch.isfinite(delta).all())
    rms = float(delta.square().mean().sqrt()) if finite else None
    scale = float(expected.detach().float().square().mean().sqrt().clamp_min(1e-12))
    return {"correct": finite and bool(torch.allclose(actual.float(), expected.float(),
                                                      atol=atol, rtol=rtol)),
            "max_abs_error": float(delta.abs().max()) if finite else None, "rms_error": rms,
            "relative_rms_error": rms / scale if finite else None, "atol": atol, "rtol": rtol}


def scale_aware_comparison(actual, expected, relative_tolerance=0.05, absolute_floor=1e-8) -> dict:
    """RMS error relative to the reference's RMS: a zero gradient cannot pass by
    hiding under an absolute tolerance, and weight updates are compared as deltas."""
    import torch
    value, reference = actual.detach().float(), expected.detach().float()
    finite = bool(torch.isfinite(value).all() and torch.isfinite(reference).all())
    reference_rms = float(reference.square().mean().sqrt())
    error_rms = float((value - reference).square().mean().sqrt())
    return {"correct": finite and error_rms <= relative_tolerance * reference_rms + absolute_floor,
            "actual_rms": float(value.square().mean().sqrt()), "reference_rms": reference_rms,
            "rms_error": error_rms, "relative_rms_error": error_rms / max(reference_rms, 1e-30),
            "actual_norm": float(value.norm()), "reference_norm": float(reference.norm()),
            "relative_rms_tolerance": relative_tolerance, "absolute_rms_floor": absolute_floor}


def values_for(n, d, dtype, seed, heads=2):
    import torch
    torch.manual_seed(seed)
    values = tuple(torch.randn(1, heads, n, d, device="cuda", dtype=dtype, requires_grad=True)
                   for _ in range(3))
    return values, torch.randn_like(values[0])


def _errors(outputs, references, dtype) -> dict:
    return {name: comparison(value, target, dtype)
            for name, value, target in zip(("output", "dq", "dk", "dv"), outputs, references)}


def numerical_case(n, d, dtype, spec, docs, seed=17, tile_q=64, tile_k=64) -> dict:
    import torch
    from .backward import training_attention
    result = {"kind": "correctness", "n": n, "d": d, "dtype": str(dtype), "spec": asdict(spec),
              "seed": seed, "block_q": tile_q, "block_k": tile_k,
              "document_pattern": "repeated labels" if docs else None}
    values, upstream = values_for(n, d, dtype, seed)
    oracle_values = tuple(v.detach().float().requires_grad_() for v in values)
    actual = training_attention(*values, spec, docs, block_q=tile_q, block_k=tile_k)
    reference = dense_attention(*oracle_values, spec, docs)
    grads = torch.autograd.grad(actual, values, upstream)
    oracle_grads = torch.autograd.grad(reference, oracle_values, upstream.float())
    result["errors"] = _errors((actual, *grads), (reference, *oracle_grads), dtype)
    good = all(e["correct"] for e in result["errors"].values())
    result["status"] = "passed" if good else "failed_correctness"
    return result


class TrainingCaptureError(RuntimeError):
    """Capture or replay failed; the CUDA stream state can no longer be trusted."""


def time_training_graph(function, *, repeats, warmup=2, inner_repeats=3) -> dict:
    """Capture on the stream that built the retained autograd graph.

    Backward nodes run on the stream of their forward; capturing on another
    stream would make the capture depend on uncaptured work.
    """
    import torch
    stream = torch.cuda.current_stream()
    if stream == torch.cuda.default_stream():
        raise ValueError("training graph timing needs an explicit non-default stream")
    for _ in range(warmup):
        function()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    try:
        with torch.cuda.graph(graph, stream=stream):
            for _ in range(inner_repeats):
                function()
        for _ in range(3):
            graph.replay()
        torch.cuda.synchronize()
        events = []
        for _ in range(repeats):
            begin, end = (torch.cuda.Event(enable_timing=True) for _ in range(2))
            begin.record(stream)
            graph.replay()
            end.record(stream)
            events.append((begin, end))
        stream.synchronize()
        samples = [begin.elapsed_time(end) / inner_repeats for begin, end in events]
    except Exception as error:
        raise TrainingCaptureError("training CUDA-graph capture or replay failed") from error
    if any(not math.isfinite(s) or s <= 0 for s in samples):
        raise RuntimeError("CUDA timing produced non-positive or non-finite samples")
    return {"median_ms": statistics.median(samples), "min_ms": min(samples),
            "max_ms": max(samples), "samples_ms": samples, "mode": "cuda_graph",
            "calls_per_sample": inner_repeats}


def time_eager(function, *, repeats, warmup=2) -> dict:
    import torch
    for _ in range(warmup):
        function()
    samples = []
    for _ in range(repeats):
        begin, end = (torch.cuda.Event(enable_timing=True) for _ in range(2))
        begin.record()
        function()
        end.record()
        end.synchronize()
        samples.append(begin.elapsed_time(end))
    return {"median_ms": statistics.median(samples), "min_ms": min(samples),
            "max_ms": max(samples), "samples_ms": samples, "mode": "eager", "calls_per_sample": 1}


def timing_and_memory(function, repeats, *, timing_mode="cuda_graph") -> dict:
    import torch
    function()
    torch.cuda.synchronize()
    gc.collect()
    baseline = torch.cuda.memory_allocated()
    torch.cuda.reset_peak_memory_stats()
    function()
    torch.cuda.synchronize()
    peak = torch.cuda.max_memory_allocated()
    timing = (time_training_graph(function, repeats=repeats) if timing_mode == "cuda_graph"
              else time_eager(function, repeats=repeats))
    return {"timing": timing, "baseline_allocated_bytes": baseline, "peak_allocated_bytes": peak,
            "peak_increment_bytes": max(0, peak - baseline),
            "memory_scope": ("one eager call after warm-up; live inputs and retained graph count "
                             "toward the baseline; the CUDA-graph pool is excluded")}


def variants_for(n, spec, docs, *, include_flex=False) -> list:
    import torch
    import torch.nn.functional as F
    from .backward import training_attention
    variants = [(CUSTOM, lambda q, k, v: training_attention(q, k, v, spec, docs))]
    if not spec.same_document and spec.window_left is None and spec.window_right is None:
        name = "pytorch_sdpa_native_causal" if spec.causal else "pytorch_sdpa_native_dense"
        variants.append((name, lambda q, k, v: F.scaled_dot_product_attention(
            q, k, v, is_causal=spec.causal)))
    else:
        from .benchmark import dense_mask
        mask = dense_mask(n, spec, docs).cuda()
        variants.append(("pytorch_sdpa_bool_mask", lambda q, k, v: F.scaled_dot_product_attention(
            q, k, v, attn_mask=mask)))
    if include_flex:
        from torch.nn.attention.flex_attention import create_block_mask, flex_attention
        import torch._functorch.config as functorch_config
        functorch_config.donated_buffer = False   # retained backward reuses saved buffers
        labels = None if docs is None else torch.tensor(list(docs), device="cuda")

        def predicate(b, h, qi, ki):
            ok = qi >= 0
            if spec.causal:
                ok = ok & (ki <= qi)
            if spec.window_left is not None:
                ok = ok & (ki >= qi - spec.window_left)
            if spec.window_right is not None:
                ok = ok & (ki <= qi + spec.window_right)
            if spec.same_document:
                ok = ok & (labels[qi] == labels[ki])
            return ok

        block_mask = create_block_mask(predicate, None, None, n, n, device="cuda")
        compiled = torch.compile(flex_attention, dynamic=False)
        variants.append(("flex_attention", lambda q, k, v: compiled(q, k, v,
                                                                    block_mask=block_mask)))
    return variants


def performance_case(n, d, dtype, spec, docs, seed=19, repeats=15, include_flex=False) -> dict:
    import torch
    caller = torch.cuda.current_stream()
    stream = torch.cuda.Stream()
    stream.wait_stream(caller)
    with torch.cuda.stream(stream):
        result = _performance_on_stream(n, d, dtype, spec, docs, seed, repeats, include_flex)
    caller.wait_stream(stream)
    return result


def _performance_on_stream(n, d, dtype, spec, docs, seed, repeats, include_flex) -> dict:
    import torch
    result = {"kind": "attention_training", "n": n, "d": d, "batch": 1, "heads": 2,
              "dtype": str(dtype), "spec": asdict(spec), "seed": seed, "variants": {},
              "scope": ("CUDA-graph replay without Python dispatch; inputs, retained forward, "
                        "warm-ups, capture and replay share one explicit stream; identical "
                        "Q/K/V, mask and upstream gradient for every variant")}
    values, upstream = values_for(n, d, dtype, seed)
    oracle_values = tuple(v.detach().float().requires_grad_() for v in values)
    reference = dense_attention(*oracle_values, spec, docs)
    reference_grads = torch.autograd.grad(reference, oracle_values, upstream.float())
    for name, function in variants_for(n, spec, docs, include_flex=include_flex):
        record = result["variants"][name] = {}
        try:
            torch.cuda.synchronize()
            begin = time.perf_counter()
            output = function(*values)
            grads = torch.autograd.grad(output, values, upstream, retain_graph=True)
            torch.cuda.synchronize()
            record["first_forward_backward_ms"] = (time.perf_counter() - begin) * 1000
            record["errors"] = _errors((output, *grads), (reference, *reference_grads), dtype)
            if not all(e["correct"] for e in record["errors"].values()):
                record["status"] = "failed_correctness"
                continue

            def backward_only():
                return torch.autograd.grad(output, values, upstream, retain_graph=True)

            def forward_backward():
                return torch.autograd.grad(function(*values), values, upstream)

            record["backward_only"] = timing_and_memory(backward_only, repeats)
            record["forward_backward"] = timing_and_memory(forward_backward, repeats)
            record["status"] = "passed"
            del output, grads
        except TrainingCaptureError:
            raise
        except Exception as error:
            record.update(status="failed", error_type=type(error).__name__, error=str(error),
                          traceback=traceback.format_exc())
    add_ratios(result, ("backward_only", "forward_backward"))
    return result


def add_ratios(result: dict, operations) -> None:
    custom = result["variants"].get(CUSTOM, {})
    if custom.get("status") == "passed":
        for name, variant in result["variants"].items():
            if name == CUSTOM or variant.get("status") != "passed":
                continue
            for operation in operations:
                variant[operation]["baseline_over_custom_speedup"] = (
                    variant[operation]["timing"]["median_ms"]
                    / custom[operation]["timing"]["median_ms"])
    good = all(v.get("status") == "passed" for v in result["variants"].values())
    result["status"] = "passed" if good else "failed"


STEP_LABELS = ("loss", "output", "qkv_gradient", "projection_gradient", "up_gradient",
               "down_gradient", "qkv_update_delta", "projection_update_delta", "up_update_delta",
               "down_update_delta")


def transformer_step_case(n, d, dtype, spec, docs, repeats=12, include_flex=False) -> dict:
    import torch
    import torch.nn.functional as F
    heads, width = 2, 2 * d
    torch.manual_seed(73)
    x = torch.randn(1, n, width, device="cuda", dtype=dtype)
    shapes = [(3 * width, width), (width, width), (4 * width, width), (width, 4 * width)]
    initial = [torch.randn(shape, device="cuda") * shape[1] ** -0.5 for shape in shapes]
    result = {"kind": "transformer_optimizer_step", "n": n, "d": d, "heads": heads,
              "dtype": str(dtype), "spec": asdict(spec), "variants": {}, "timing_mode": "eager",
              "architecture": ("one pre-norm block, 2 heads, GELU MLP of width 4C, mean squared "
                               "output loss, fp32 master weights cast to the activation dtype for "
                               "the linears, SGD lr 0.01"),
              "scope": ("eager CUDA-event timing for every variant, Python submission gaps "
                        "included: weight restore, forward, loss, backward, SGD")}
    baseline = None
    # a library implementation runs first and becomes the comparator, so the
    # kernel under study is never its own oracle
    for name, attend in reversed(variants_for(n, spec, docs, include_flex=include_flex)):
        record = result["variants"][name] = {}
        try:
            weights = [torch.nn.Parameter(value.clone()) for value in initial]

            def step():
                with torch.no_grad():
                    for weight, source in zip(weights, initial):
                        weight.copy_(source)
                        weight.grad = None
                cast = [w.to(dtype) for w in weights]
                qkv = F.linear(F.layer_norm(x, (width,)), cast[0])
                q, k, v = (t.contiguous() for t in
                           qkv.view(1, n, 3, heads, d).permute(2, 0, 3, 1, 4).unbind(0))
                hidden = x + F.linear(attend(q, k, v).transpose(1, 2).reshape(1, n, width), cast[1])
                output = hidden + F.linear(
                    F.gelu(F.linear(F.layer_norm(hidden, (width,)), cast[2])), cast[3])
                loss = output.float().square().mean()
                loss.backward()
                with torch.no_grad():
                    for weight in weights:
                        weight.add_(weight.grad, alpha=-0.01)
                return loss, output

            begin = time.perf_counter()
            loss, output = step()
            torch.cuda.synchronize()
            record["first_step_ms"] = (time.perf_counter() - begin) * 1000
            observed = (loss.detach(), output.detach(), *(w.grad.detach().clone() for w in weights),
                        *((w.detach() - source).clone() for w, source in zip(weights, initial)))
            if baseline is None:
                baseline = observed
                result["optimizer_correctness_reference"] = name
            record["errors"] = {label: scale_aware_comparison(value, reference)
                                for label, value, reference in zip(STEP_LABELS, observed, baseline)}
            record["optimizer_observability"] = {
                label: {"changed_fraction": float((update != 0).float().mean()),
                        "update_norm": float(update.norm()), "gradient_norm": float(grad.norm()),
                        "nonzero_gradient_and_update": bool(grad.norm() > 0 and update.norm() > 0)}
                for label, grad, update in zip(("qkv", "projection", "up", "down"),
                                               observed[2:6], observed[6:10])}
            record["loss"] = float(loss.detach())
            good = (all(e["correct"] for e in record["errors"].values())
                    and all(o["nonzero_gradient_and_update"]
                            for o in record["optimizer_observability"].values()))
            if good:
                record["step"] = timing_and_memory(step, repeats, timing_mode="eager")
            record["status"] = "passed" if good else "failed_correctness"
        except Exception as error:
            record.update(status="failed", error=str(error), traceback=traceback.format_exc())
    add_ratios(result, ("step",))
    return result


def planned_jobs(stage: str, *, include_flex: bool = False) -> list:
    """(kind, thunk) pairs in run order; building the list touches no GPU."""
    import torch
    half, bf16 = torch.float16, torch.bfloat16
    cases = [(17, 64, half, MaskSpec(), None, 32, 64),
             (65, 128, bf16, MaskSpec(causal=True), None, 64, 32),
             (129, 64, half, MaskSpec(window_left=11, window_right=5), None, 32, 64),
             (129, 128, bf16, MaskSpec(causal=True, same_document=True),
              tuple((i // 7) % 3 - 1 for i in range(129)), 64, 64),
             (65, 64, bf16, MaskSpec(window_left=0, window_right=0), None, 64, 64)]
    if stage == "study":
        cases += [(257, 128, half, MaskSpec(causal=True, window_left=63, same_document=True),
                   tuple((i // 31) % 4 for i in range(257)), 32, 64),
                  (129, 128, half, MaskSpec(same_document=True), tuple(i % 5 for i in range(129)),
                   64, 32),
                  (65, 64, bf16, MaskSpec(window_left=1, window_right=3), None, 64, 64)]
    jobs = [("correctness", lambda c=c: numerical_case(*c[:5], tile_q=c[5], tile_k=c[6]))
            for c in cases]
    # the whole optimizer step runs before the longer sweeps so that a bounded
    # run always yields one integrated training result
    jobs.append(("transformer", lambda: transformer_step_case(
        512, 64, bf16, MaskSpec(causal=True), None, include_flex=include_flex)))
    sweeps = [(1024, 64, MaskSpec(causal=True), None, 19),
              (1024, 64, MaskSpec(causal=True, window_left=127), None, 19)]
    if stage == "study":
        sweeps += [(4096, 64, MaskSpec(causal=True, window_left=255), None, 29),
                   (2048, 128, MaskSpec(causal=True, same_document=True),
                    tuple((i // 256) % 3 for i in range(2048)), 29)]
    for n, d, spec, docs, seed in sweeps:
        jobs.append(("performance", lambda n=n, d=d, spec=spec, docs=docs, seed=seed:
                     performance_case(n, d, bf16, spec, docs, seed=seed,
                                      include_flex=include_flex)))
    if stage == "study":
        jobs.append(("transformer", lambda: transformer_step_case(
            1024, 128, bf16, MaskSpec(causal=True, window_left=127), None,
            include_flex=include_flex)))
    return jobs


def run_jobs(jobs, output_dir: Path, report: dict, budget_seconds: float) -> dict:
    """Runs jobs in order, one evidence file each; separated from ``main`` for tests."""
    started = time.perf_counter()
    report.update(planned_cases=len(jobs), cases=[])

    def save():
        report["elapsed_seconds"] = time.perf_counter() - started
        scratch = output_dir / "summary.tmp"
        scratch.write_text(json.dumps(report, indent=2))
        scratch.replace(output_dir / "summary.json")

    save()
    for index, (kind, job) in enumerate(jobs):
        if time.perf_counter() - started >= budget_seconds:
            report["stopped_for_budget"] = True
            break
        fatal = False
        try:
            item = job()
        except Exception as error:
            item = {"kind": kind, "status": "failed", "error": str(error),
                    "traceback": traceback.format_exc()}
            fatal = isinstance(error, TrainingCaptureError) or "CUDA error" in str(error)
            if fatal:
                item["fatal_cuda_state"] = True
                report["stopped_after_cuda_failure"] = True
        item["case_index"] = index
        report["cases"].append(item)
        (output_dir / f"case_{index:03d}.json").write_text(json.dumps(item, indent=2))
        save()
        print(json.dumps({"case": index, "kind": kind, "status": item["status"],
                          "elapsed_seconds": report["elapsed_seconds"]}), flush=True)
        if fatal:
            break
        gc.collect()
    report["completed_cases"] = len(report["cases"])
    report["passed_cases"] = sum(c["status"] == "passed" for c in report["cases"])
    report["status"] = ("failed" if any(c["status"] != "passed" for c in report["cases"])
                        else "partial_budget" if len(report["cases"]) < len(jobs) else "passed")
    save()
    return report


def main(argv=None) -> int:
    parser = argparse.ArgumentParser(description=__doc__,
                                     formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--stage", choices=("smoke", "study"), default="smoke")
    parser.add_argument("--output-dir", type=Path, required=True)
    parser.add_argument("--time-budget-seconds", type=float, default=480)
    parser.add_argument("--include-flex", action="store_true")
    args = parser.parse_args(argv)
    if args.time_budget_seconds <= 0:
        parser.error("time budget must be positive")
    args.output_dir.mkdir(parents=True, exist_ok=True)
    import torch
    if not torch.cuda.is_available():
        raise RuntimeError("A CUDA GPU is required; this command provisions nothing")
    torch.backends.cuda.matmul.allow_tf32 = False    # the fp32 oracle must really be fp32
    torch.backends.cudnn.allow_tf32 = False
    report = {"stage": args.stage, "budget_seconds": args.time_budget_seconds,
              "environment": {"python": platform.python_version(), "torch": torch.__version__,
                              "cuda": torch.version.cuda, "gpu": torch.cuda.get_device_name()},
              "implementation": ("online-softmax forward saving the log-sum-exp; dQ owned by "
                                 "query tiles, dK/dV owned by key tiles over the transposed "
                                 "schedule; fp32 accumulation in tensor memory; no atomics"),
              "limitations": ["first derivatives only", "no dropout",
                              "one sequence length for Q, K and V",
                              "one document-label sequence shared by batch and heads"]}
    report = run_jobs(planned_jobs(args.stage, include_flex=args.include_flex), args.output_dir,
                      report, args.time_budget_seconds)
    print(json.dumps({"status": report["status"],
                      "output": str(args.output_dir / "summary.json")}), flush=True)
    return {"passed": 0, "partial_budget": 2}.get(report["status"], 1)


if __name__ == "__main__":
    raise SystemExit(main())
