"""Budgeted search over a declared attention-kernel configuration space.

Role and rules of the reference's selector (attention_lab/search.py:17-229): the
evaluator owns correctness checks and hardware timing; the search only decides
which configuration to try next, never invents measurements, spends budget on
failures too, and records every observation so a run can be replayed offline.
Two strategies over the same candidate set and budget: uniform ``random``
sampling without replacement, and ``evolution`` - mutate exactly one field of a
measured, correct parent chosen from a small diversity-preserving parent set
(fastest first, then the candidates farthest from those already chosen), with a
restart probability for exploration.

The sm_100a kernel has one fixed warp layout, so the space is what actually
changes its work: the granularity at which the block schedule is compiled
(``block_q`` x ``block_k``, which decides how many tiles are partial), the
schedule form (``csr`` or ``interval``) and whether full tiles may skip the
token-level mask - 2 x 3 x 2 x 2 = 24 candidates.
"""

from __future__ import annotations

import json
import math
import random
from dataclasses import asdict, dataclass, fields
from typing import Callable, Iterable

IMPLEMENTATIONS = ("csr", "interval")


@dataclass(frozen=True)
class KernelConfig:
    block_q: int
    block_k: int
    implementation: str = "csr"
    use_full_blocks: bool = True

    def __post_init__(self) -> None:
        for name in ("block_q", "block_k"):
            value = getattr(self, name)
            if type(value) is not int or value <= 0:
                raise ValueError(f"{name} must be a positive integer")
        if self.implementation not in IMPLEMENTATIONS:
            raise ValueError("implementation must be 'csr' or 'interval'")
        if type(self.use_full_blocks) is not bool:
            raise ValueError("use_full_blocks must be a bool")


def default_configs() -> tuple[KernelConfig, ...]:
    return tuple(KernelConfig(q, k, impl, full) for q in (64, 128) for k in (32, 64, 128)
                 for impl in IMPLEMENTATIONS for full in (True, False))


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
    origin: str
    parent: KernelConfig | None = None


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
        return {"schema_version": 1, "method": self.method, "seed": self.seed,
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


def hamming(a: KernelConfig, b: KernelConfig) -> int:
    return sum(getattr(a, f.name) != getattr(b, f.name) for f in fields(KernelConfig))


def select_parents(history: list[Observation], size: int) -> list[KernelConfig]:
    """Fastest eligible configuration first, then maximise distance to the chosen set."""
    pool = sorted((o for o in history if o.result.eligible),
                  key=lambda o: (o.result.latency_ms, o.evaluation))
    if not pool:
        return []
    chosen = [pool.pop(0)]
    while pool and len(chosen) < size:
        def spread(o):
            return (min(hamming(o.config, c.config) for c in chosen), -o.result.latency_ms,
                    -o.evaluation)
        pick = max(pool, key=spread)
        pool.remove(pick)
        chosen.append(pick)
    return [o.config for o in chosen]


def search(evaluate: Callable[[KernelConfig], CandidateResult],
           configs: Iterable[KernelConfig] | None = None, *, budget: int,
           method: str = "evolution", seed: int = 0, population_size: int = 4,
           restart_probability: float = 0.2) -> SearchResult:
    """Evaluate at most ``budget`` distinct configurations (failures included)."""
    if type(budget) is not int or budget < 0:
        raise ValueError("budget must be a non-negative integer")
    if method not in ("evolution", "random"):
        raise ValueError("method must be 'evolution' or 'random'")
    if type(seed) is not int:
        raise ValueError("seed must be an integer")
    if type(population_size) is not int or population_size <= 0:
        raise ValueError("population_size must be a positive integer")
    if not _is_number(restart_probability) or not 0 <= restart_probability <= 1:
        raise ValueError("restart_probability must be between zero and one")
    supplied = default_configs() if configs is None else tuple(configs)
    if any(not isinstance(c, KernelConfig) for c in supplied):
        raise TypeError("configs must contain KernelConfig values")
    candidates = list(dict.fromkeys(supplied))
    remaining = list(candidates)
    rng = random.Random(seed)
    history: list[Observation] = []
    while remaining and len(history) < budget:
        config, parent, origin = None, None, "random" if method == "random" else "restart"
        if method == "evolution":
            parents = select_parents(history, population_size)
            if parents and rng.random() >= restart_probability:
                rng.shuffle(parents)
                for candidate_parent in parents:
                    neighbours = [c for c in remaining if hamming(c, candidate_parent) == 1]
                    if neighbours:
                        config, parent, origin = (rng.choice(neighbours), candidate_parent,
                                                  "mutation")
                        break
        if config is None:
            config = rng.choice(remaining)
        remaining.remove(config)
        try:
            result = sanitize(evaluate(config))
        except Exception as error:     # a failing candidate is evidence and spends budget
            result = CandidateResult(False, error=f"{type(error).__name__}: {error}")
        history.append(Observation(len(history) + 1, config, result, origin, parent))
    return SearchResult(method, seed, budget, len(candidates), tuple(history))


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
