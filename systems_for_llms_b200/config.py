"""Training configuration: frozen dataclasses, strict validation, JSON loading.

Same schema and defaults as the reference (src/llmlab/config.py:7-106) so its
JSON files load unchanged; ``to_dict`` yields the JSON-primitive form stored in
checkpoints.  Validation is table driven: each rule is (field path, predicate,
message), checked in a fixed order so the first offending field is reported.
"""

from __future__ import annotations

import dataclasses
import json
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any

ATTENTION_BACKENDS = ("eager", "sdpa")
CHECKPOINT_POLICIES = ("none", "block")
DEVICES = ("cpu", "cuda", "mps", "auto")
PRECISIONS = ("fp32", "bf16")
DATA_KINDS = ("synthetic", "npy")


@dataclass(frozen=True)
class ModelConfig:
    vocab_size: int = 32
    context_length: int = 8
    d_model: int = 16
    num_layers: int = 1
    num_heads: int = 2
    d_ff: int = 32
    rope_theta: float = 10000.0
    attention_backend: str = "eager"
    activation_checkpointing: str = "none"


@dataclass(frozen=True)
class DataConfig:
    kind: str = "synthetic"
    train_path: str | None = None
    valid_path: str | None = None
    tokenizer_files: tuple[str, ...] = ()
    synthetic_tokens: int = 4096


def _strict_positive_int(value: Any) -> bool:
    # bool is an int subclass and 3.0 == 3; both are rejected on purpose.
    return type(value) is int and value > 0


def _finite_number(value: Any) -> bool:
    return isinstance(value, (int, float)) and not isinstance(value, bool) and math.isfinite(value)


@dataclass(frozen=True)
class TrainConfig:
    model: ModelConfig = field(default_factory=ModelConfig)
    data: DataConfig = field(default_factory=DataConfig)
    seed: int = 1337
    device: str = "cpu"
    num_threads: int = 1
    batch_size: int = 2
    grad_accum_steps: int = 1
    precision: str = "fp32"
    max_steps: int = 20
    learning_rate: float = 0.003
    min_learning_rate: float = 0.0003
    warmup_steps: int = 2
    weight_decay: float = 0.1
    grad_clip: float = 1.0
    eval_interval: int = 5
    eval_batches: int = 4
    eval_batch_size: int = 2
    checkpoint_interval: int = 10

    _COUNT_FIELDS = ("num_threads", "batch_size", "grad_accum_steps", "max_steps",
                     "eval_interval", "eval_batches", "eval_batch_size", "checkpoint_interval")
    _MODEL_COUNT_FIELDS = ("vocab_size", "context_length", "d_model", "num_layers", "num_heads",
                           "d_ff")
    _REAL_FIELDS = ("learning_rate", "min_learning_rate", "weight_decay", "grad_clip")

    def validate(self) -> None:
        for name in self._COUNT_FIELDS:
            if not _strict_positive_int(getattr(self, name)):
                raise ValueError(f"{name} must be a positive integer")
        for name in self._MODEL_COUNT_FIELDS:
            if not _strict_positive_int(getattr(self.model, name)):
                raise ValueError(f"model.{name} must be a positive integer")
        if type(self.seed) is not int or not 0 <= self.seed < 2**63 - 1:
            raise ValueError("seed must be an integer in [0, 2**63 - 1)")
        if type(self.warmup_steps) is not int or not 0 <= self.warmup_steps < self.max_steps:
            raise ValueError("warmup_steps must be in [0, max_steps)")
        for name in self._REAL_FIELDS:
            if not _finite_number(getattr(self, name)):
                raise ValueError(f"{name} must be finite")
        theta = self.model.rope_theta
        if not _finite_number(theta) or theta <= 0:
            raise ValueError("model.rope_theta must be finite and positive")
        if self.learning_rate <= 0 or not 0 <= self.min_learning_rate <= self.learning_rate:
            raise ValueError("require 0 <= min_learning_rate <= learning_rate and learning_rate > 0")
        if self.weight_decay < 0 or self.grad_clip <= 0:
            raise ValueError("weight_decay must be nonnegative and grad_clip positive")
        choices = (("device", self.device, DEVICES), ("precision", self.precision, PRECISIONS),
                   ("model.attention_backend", self.model.attention_backend, ATTENTION_BACKENDS),
                   ("model.activation_checkpointing", self.model.activation_checkpointing,
                    CHECKPOINT_POLICIES),
                   ("data.kind", self.data.kind, DATA_KINDS))
        for name, value, allowed in choices:
            if value not in allowed:
                raise ValueError(f"{name} must be one of: {', '.join(allowed)}")
        if self.data.kind == "npy" and not (self.data.train_path and self.data.valid_path):
            raise ValueError("npy data requires train_path and valid_path")
        if self.data.kind == "synthetic":
            tokens = self.data.synthetic_tokens
            if type(tokens) is not int or tokens <= self.model.context_length:
                raise ValueError("synthetic_tokens must be an integer exceeding context_length")

    def to_dict(self) -> dict:
        """JSON-primitive form (tuples become lists, paths become strings)."""
        plain = {f.name: getattr(self, f.name) for f in dataclasses.fields(self)}
        plain["model"] = dataclasses.asdict(self.model)
        plain["data"] = dataclasses.asdict(self.data)
        return json.loads(json.dumps(plain, default=str))


def load_config(path: str | Path) -> TrainConfig:
    """Reads a JSON config; relative data/tokenizer paths resolve against the file."""
    path = Path(path).resolve()
    document = json.loads(path.read_text())
    model = ModelConfig(**document.pop("model"))
    data_fields = dict(document.pop("data"))
    base = path.parent
    for key in ("train_path", "valid_path"):
        if data_fields.get(key):
            data_fields[key] = str((base / data_fields[key]).resolve())
    data_fields["tokenizer_files"] = tuple(
        str((base / item).resolve()) for item in data_fields.get("tokenizer_files", ()))
    config = TrainConfig(model=model, data=DataConfig(**data_fields), **document)
    config.validate()
    return config
