"""Configuration validation and JSON loading (reference: src/llmlab/config.py)."""

import dataclasses
import json

import pytest

from systems_for_llms_b200.config import DataConfig, ModelConfig, TrainConfig, load_config


def make(**overrides):
    return dataclasses.replace(TrainConfig(model=ModelConfig(), data=DataConfig()), **overrides)


def test_defaults_validate():
    make().validate()


@pytest.mark.parametrize("field,value", [
    ("batch_size", 0), ("batch_size", True), ("batch_size", 2.0), ("max_steps", -1),
    ("seed", -1), ("seed", 2**63), ("warmup_steps", 20), ("learning_rate", float("nan")),
    ("learning_rate", 0.0), ("min_learning_rate", 1.0), ("weight_decay", -0.1),
    ("grad_clip", 0.0), ("device", "tpu"), ("precision", "fp16"),
])
def test_rejects_bad_top_level(field, value):
    with pytest.raises(ValueError):
        make(**{field: value}).validate()


@pytest.mark.parametrize("field,value", [
    ("d_model", 0), ("num_heads", 1.5), ("rope_theta", 0.0), ("rope_theta", float("inf")),
    ("attention_backend", "flash"), ("activation_checkpointing", "all"),
])
def test_rejects_bad_model(field, value):
    config = make(model=dataclasses.replace(ModelConfig(), **{field: value}))
    with pytest.raises(ValueError):
        config.validate()


def test_data_rules():
    with pytest.raises(ValueError):
        make(data=DataConfig(kind="npy")).validate()
    with pytest.raises(ValueError):
        make(data=DataConfig(kind="synthetic", synthetic_tokens=8)).validate()
    with pytest.raises(ValueError):
        make(data=DataConfig(kind="csv")).validate()


def test_to_dict_is_json_primitive():
    config = make(data=DataConfig(tokenizer_files=("a", "b")))
    plain = config.to_dict()
    assert plain["data"]["tokenizer_files"] == ["a", "b"]
    assert json.loads(json.dumps(plain)) == plain


def test_load_config_resolves_relative_paths(tmp_path):
    document = {"model": {"vocab_size": 64}, "data": {"kind": "npy", "train_path": "d/t.npy",
                                                     "valid_path": "d/v.npy",
                                                     "tokenizer_files": ["tok/vocab.pkl"]},
                "max_steps": 5, "warmup_steps": 1}
    path = tmp_path / "cfg" / "c.json"
    path.parent.mkdir()
    path.write_text(json.dumps(document))
    config = load_config(path)
    assert config.data.train_path == str((path.parent / "d/t.npy").resolve())
    assert config.data.tokenizer_files == (str((path.parent / "tok/vocab.pkl").resolve()),)
    assert config.model.vocab_size == 64 and config.max_steps == 5


def test_shipped_configs_load():
    from pathlib import Path
    root = Path(__file__).resolve().parents[1] / "configs"
    names = sorted(p.name for p in root.glob("*.json"))
    assert "smoke.json" in names and "scale-324m-s1024.json" in names
    for name in names:
        config = load_config(root / name)
        assert config.model.d_model % config.model.num_heads == 0
    big = load_config(root / "scale-324m-s1024.json")
    assert (big.model.num_layers, big.model.d_model, big.model.num_heads, big.model.d_ff,
            big.model.vocab_size) == (24, 1024, 16, 2752, 10000)
