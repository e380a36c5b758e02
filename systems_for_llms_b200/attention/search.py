"""Budgeted selection of an attention-kernel configuration for one workload.

The contract is the reference selector's (attention_lab/search.py:17-229): the evaluator
owns correctness checks and hardware timing; the search only decides which configuration
to try next, never invents a measurement, spends budget on failures too, and records
every observation so that a run can be replayed offline against the recorded table.

Every field of the space changes what the sm_100a kernels execute:

``pipeline``         which forward kernel runs - ``two_stream`` (two independent work
                     streams per CTA, P kept in tensor memory; head dimension 64),
                     ``two_stream_smem_p`` (same, P through shared memory) or
                     ``one_stream`` (one query tile per CTA, the only form for D = 128);
``implementation``   ``csr`` (tile list + sub-block bitmaps from memory) or ``interval``
                     (tile range computed in registers, no metadata);
``block_q, block_k`` granularity at which a CSR schedule is compiled - it decides which
                     128 x 128 tiles count as full and what their bitmaps hold (the
                     interval form has no schedule, so it appears once, at 128 x 128);
``use_full_blocks``  whether full tiles may skip the token-level predicate.

Two strategies over the same candidates and budget.  ``random`` samples without
replacement and is the baseline.  ``descent`` is a coordinate search, which fits a small
factorial space whose fields act almost independently: starting from an incumbent it
sweeps one field at a time through its untried values with the other fields fixed, adopts
whatever was faster, and after a pass over all fields without improvement restarts from
the untried candidate that differs from everything measured so far in the most fields.
"""

from __future__ import annotations

import json
import math
import random
from dataclasses import asdict, dataclass, fields
from typing import Callable, Iterable

IMPLEMENTATIONS = ("csr", "interval")
PIPELINES = ("two_stream", "two_stream_smem_p", "one_stream")
FIELD_ORDER = ("pipeline", "implementation", "use_full_blocks", "block_q", "block_k")


@dataclass(frozen=True)
class KernelConfig:
    block_q: int
    block_k: int
    implementation: str = "csr"
    use_full_blocks: bool = True
    pipeline: str = "two_stream"

    def __post_init__(self) -> None:
        for name in ("block_q", "block_k"):
            value = getattr(self, name)
            if type(value) is not int or value <= 0:
                raise ValueError(f"{name} must be a positive integer")
        if self.implementation not in IMPLEMENTATIONS:
            raise ValueError("implementation must be 'csr' or 'interval'")
        if type(self.use_full_blocks) is not bool:
            raise ValueError("use_full_blocks must be a bool")
        if self.pipeline not in PIPELINES:
            raise ValueError(f"pipeline must be one of {', '.join(PIPELINES)}")


def default_configs(head_dim: int = 64) -> tuple[KernelConfig, ...]:
    """The candidate set for a head dimension: 42 configurations at D = 64, 14 at D = 128."""
    pipelines = PIPELINES if head_dim == 64 else ("one_stream",)
    found = []
    for pipeline in pipelines:
        for full in (True, False):
            found.append(KernelConfig(128, 128, "interval", full, pipeline))
            for q in (64, 128):
                for k in (32, 64, 128):
                    found.append(KernelConfig(q, k, "csr", full, pipeline))
    return tuple(found)


def _is_number(value) -> bool:
    return isinstance(value, (int, float)) and not isinstance(value, bool) and math.isfinite(value)


@dataclass(frozen=True)
class CandidateResult:
    correct: bool
    latency_ms: float | None = None
    compile_ms: float | None = None
    error: str | None = None

    @property
    def eligible(self) -> bool:
        if self.correct is not True or self.error is not None:
            return False
        if not _is_number(self.latency_ms) or self.latency_ms <= 0:
            return False
        return self.compile_ms is None or (_is_number(self.compile_ms) and self.compile_ms >= 0)


@dataclass(frozen=True)
class Observation:
    evaluation: int
    config: KernelConfig
    result: CandidateResult
    origin: str                       # "random", "start", "sweep:<field>" or "restart"
    parent: KernelConfig | None = None   # the incumbent a sweep step was derived from


@dataclass(frozen=True)
class SearchResult:
    method: str
    seed: int
    requested_budget: int
    unique_configurations: int
    history: tuple[Observation, ...]

    @property
    def best(self) -> Observation | None:
        eligible = [o for o in self.history if o.result.eligible]
        return min(eligible, key=lambda o: o.result.latency_ms) if eligible else None

    def to_dict(self) -> dict:
        best = self.best
        return {"schema_version": 2, "method": self.method, "seed": self.seed,
                "requested_budget": self.requested_budget,
                "unique_configurations": self.unique_configurations,
                "evaluations": len(self.history),
                "eligible_evaluations": sum(o.result.eligible for o in self.history),
                "best": asdict(best) if best is not None else None,
                "history": [asdict(o) for o in self.history]}

    def to_json(self, *, indent: int | None = 2) -> str:
        return json.dumps(self.to_dict(), indent=indent, allow_nan=False)


def sanitize(value) -> CandidateResult:
    """Turn whatever an evaluator returned into a well-formed result."""
    if not isinstance(value, CandidateResult):
        return CandidateResult(False, error="invalid_result: expected CandidateResult")
    problems = [] if value.error is None else [str(value.error)]
    correct = value.correct
    if type(correct) is not bool:
        correct = False
        problems.append("invalid_correctness: expected bool")
    latency = value.latency_ms
    if latency is not None and (not _is_number(latency) or latency <= 0):
        problems.append(f"invalid_latency_ms: {latency!r}")
        latency = None
    if correct and latency is None:
        problems.append("missing_valid_latency")
    compile_ms = value.compile_ms
    if compile_ms is not None and (not _is_number(compile_ms) or compile_ms < 0):
        problems.append(f"invalid_compile_ms: {compile_ms!r}")
        compile_ms = None
    return CandidateResult(correct, None if latency is None else float(latency),
                           None if compile_ms is None else float(compile_ms),
                           "; ".join(problems) or None)


def differing_fields(a: KernelConfig, b: KernelConfig) -> int:
    return sum(getattr(a, f.name) != getattr(b, f.name) for f in fields(KernelConfig))


class _Run:
    """Bookkeeping shared by both strategies: budget, candidates left, the record."""

    def __init__(self, evaluate, candidates, budget):
        self.evaluate, self.budget = evaluate, budget
        self.remaining = list(candidates)
        self.history: list[Observation] = []

    @property
    def open(self) -> bool:
        return bool(self.remaining) and len(self.history) < self.budget

    def measure(self, config: KernelConfig, origin: str, parent=None) -> Observation:
        self.remaining.remove(config)
        try:
            result = sanitize(self.evaluate(config))
        except Exception as error:     # a failing candidate is evidence and spends budget
            result = CandidateResult(False, error=f"{type(error).__name__}: {error}")
        observation = Observation(len(self.history) + 1, config, result, origin, parent)
        self.history.append(observation)
        return observation


def _farthest(run: _Run, rng: random.Random) -> KernelConfig:
    """Untried candidate whose nearest measured configuration is as far away as possible."""
    measured = [o.config for o in run.history]
    if not measured:
        return rng.choice(run.remaining)
    order = list(run.remaining)
    rng.shuffle(order)                 # ties are broken by the seed, not by list position
    return max(order, key=lambda c: min(differing_fields(c, m) for m in measured))


def _descent(run: _Run, rng: random.Random, start: KernelConfig | None) -> None:
    first = True
    while run.open:
        seed_config = start if first and start in run.remaining else _farthest(run, rng)
        observation = run.measure(seed_config, "start" if first else "restart")
        first = False
        if not observation.result.eligible:
            continue                   # nothing to descend from: restart elsewhere
        incumbent, incumbent_ms = observation.config, observation.result.latency_ms
        improved = True
        while improved and run.open:
            improved = False
            for name in FIELD_ORDER:
                siblings = [c for c in run.remaining
                            if differing_fields(c, incumbent) == 1
                            and getattr(c, name) != getattr(incumbent, name)]
                rng.shuffle(siblings)
                best_step = None
                for candidate in siblings:
                    if not run.open:
                        break
                    step = run.measure(candidate, f"sweep:{name}", incumbent)
                    if step.result.eligible and step.result.latency_ms < incumbent_ms and (
                            best_step is None
                            or step.result.latency_ms < best_step.result.latency_ms):
                        best_step = step
                if best_step is not None:
                    incumbent, incumbent_ms = best_step.config, best_step.result.latency_ms
                    improved = True


def search(evaluate: Callable[[KernelConfig], CandidateResult],
           configs: Iterable[KernelConfig] | None = None, *, budget: int,
           method: str = "descent", seed: int = 0,
           start: KernelConfig | None = None) -> SearchResult:
    """Evaluate at most ``budget`` distinct configurations (failures included)."""
    if type(budget) is not int or budget < 0:
        raise ValueError("budget must be a non-negative integer")
    if method not in ("descent", "random"):
        raise ValueError("method must be 'descent' or 'random'")
    if type(seed) is not int:
        raise ValueError("seed must be an integer")
    if start is not None and not isinstance(start, KernelConfig):
        raise TypeError("start must be a KernelConfig")
    supplied = default_configs() if configs is None else tuple(configs)
    if any(not isinstance(c, KernelConfig) for c in supplied):
        raise TypeError("configs must contain KernelConfig values")
    candidates = list(dict.fromkeys(supplied))
    run = _Run(evaluate, candidates, budget)
    rng = random.Random(seed)
    if method == "random":
        while run.open:
            run.measure(rng.choice(run.remaining), "random")
    else:
        _descent(run, rng, start)
    return SearchResult(method, seed, budget, len(candidates), tuple(run.history))


def replay(history: Iterable[dict], *, budget: int, method: str, seed: int,
           configs: Iterable[KernelConfig] | None = None) -> SearchResult:
    """Re-run a search offline against recorded measurements (no GPU involved)."""
    table = {}
    for item in history:
        config = KernelConfig(**item["config"])
        table[config] = CandidateResult(**item["result"])

    def lookup(config: KernelConfig) -> CandidateResult:
        if config not in table:
            return CandidateResult(False, error="not measured in the recorded history")
        return table[config]

    return search(lookup, configs if configs is not None else tuple(table), budget=budget,
                  method=method, seed=seed)
