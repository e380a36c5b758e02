"""Model numerics on the portable path (reference strategy: tests/test_model.py)."""

import dataclasses

import pytest
import torch
from torch.nn import functional as F

from systems_for_llms_b200.models import transformer as transformer_module
from systems_for_llms_b200.models.transformer import TransformerLM
from systems_for_llms_b200.training.loss import cross_entropy, perplexity

BASE = dict(vocab_size=37, context_length=12, d_model=32, num_layers=2, num_heads=4, d_ff=48,
            rope_theta=10000.0)


def build(seed=0, **overrides):
    torch.manual_seed(seed)
    return TransformerLM(**{**BASE, **overrides}, dtype=torch.float32)


def batch(seed=1, size=3, length=12):
    generator = torch.Generator().manual_seed(seed)
    tokens = torch.randint(0, BASE["vocab_size"], (size, length + 1), generator=generator)
    return tokens[:, :-1], tokens[:, 1:]


def grads(model, x, y):
    model.zero_grad(set_to_none=True)
    loss = cross_entropy(model(x).float(), y)
    loss.backward()
    return loss.detach(), {n: p.grad.clone() for n, p in model.named_parameters()}


def test_eager_and_sdpa_agree():
    eager, sdpa = build(attention_backend="eager"), build(attention_backend="sdpa")
    x, y = batch()
    loss_a, grads_a = grads(eager, x, y)
    loss_b, grads_b = grads(sdpa, x, y)
    torch.testing.assert_close(loss_a, loss_b, rtol=1e-5, atol=1e-6)
    for name in grads_a:
        torch.testing.assert_close(grads_a[name], grads_b[name], rtol=1e-4, atol=1e-6)


def test_checkpointing_preserves_init_and_gradients():
    plain, ckpt = build(), build(activation_checkpointing="block")
    for (na, pa), (nb, pb) in zip(plain.named_parameters(), ckpt.named_parameters()):
        assert na == nb and torch.equal(pa, pb)
    x, y = batch()
    loss_a, grads_a = grads(plain, x, y)
    loss_b, grads_b = grads(ckpt, x, y)
    torch.testing.assert_close(loss_a, loss_b, rtol=0, atol=0)
    for name in grads_a:
        torch.testing.assert_close(grads_a[name], grads_b[name], rtol=1e-6, atol=1e-8)


def test_recompute_only_when_training_with_grad(monkeypatch):
    calls = []
    real = transformer_module.checkpoint

    def spy(function, *args, **kwargs):
        calls.append(function)
        return real(function, *args, **kwargs)

    monkeypatch.setattr(transformer_module, "checkpoint", spy)
    model = build(activation_checkpointing="block")
    x, _ = batch()
    model.train()
    model(x)
    assert len(calls) == BASE["num_layers"]
    calls.clear()
    with torch.no_grad():
        model(x)
    model.eval()
    model(x)
    assert calls == []
    none = build(activation_checkpointing="none")
    none.train()
    none(x)
    assert calls == []


def test_causal_prefix_invariance():
    model = build().eval()
    x, _ = batch()
    with torch.no_grad():
        full = model(x)
        prefix = model(x[:, :7])
    torch.testing.assert_close(full[:, :7], prefix, rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("scale", [1.0, 1000.0])
def test_cross_entropy_matches_torch(scale):
    generator = torch.Generator().manual_seed(3)
    logits = torch.randn(4, 9, 37, generator=generator) * scale
    targets = torch.randint(0, 37, (4, 9), generator=generator)
    expected = F.cross_entropy(logits.reshape(-1, 37), targets.reshape(-1))
    torch.testing.assert_close(cross_entropy(logits, targets), expected, rtol=1e-5, atol=1e-5)
    torch.testing.assert_close(perplexity(logits, targets), expected.exp(), rtol=1e-4, atol=1e-4)


def test_state_dict_keys_match_reference_layout():
    model = build(num_layers=1)
    assert list(model.state_dict()) == [
        "token_embeddings.weight", "layers.0.attn_norm.weight", "layers.0.attn.q_proj.weight",
        "layers.0.attn.k_proj.weight", "layers.0.attn.v_proj.weight",
        "layers.0.attn.output_proj.weight", "layers.0.ffn_norm.weight", "layers.0.ffn.w1.weight",
        "layers.0.ffn.w2.weight", "layers.0.ffn.w3.weight", "ln_final.weight", "lm_head.weight"]


def test_loss_entry_point_equals_logits_path():
    model = build()
    x, y = batch()
    direct = cross_entropy(model(x).float(), y)
    torch.testing.assert_close(model.loss(x, y), direct, rtol=0, atol=0)
    torch.testing.assert_close(model.loss(x, y, 0.25), direct / 4, rtol=0, atol=0)


@pytest.mark.parametrize("overrides", [
    {"d_model": 0}, {"num_heads": 5}, {"activation_checkpointing": "layer"},
    {"attention_backend": "flash"}, {"vocab_size": 2.5}])
def test_invalid_model_arguments(overrides):
    with pytest.raises(ValueError):
        build(**overrides)


def test_sequence_length_bounds():
    model = build()
    with pytest.raises(ValueError):
        model(torch.zeros(1, 13, dtype=torch.long))
    with pytest.raises(ValueError):
        model(torch.zeros(1, 0, dtype=torch.long))


def test_rope_is_interleaved_pairs():
    from systems_for_llms_b200.models.attention import RotaryPositionalEmbedding
    rope = RotaryPositionalEmbedding(10000.0, 4, 16)
    x = torch.arange(8, dtype=torch.float32).reshape(1, 2, 4)
    out = rope(x, torch.tensor([0, 3]))
    torch.testing.assert_close(out[0, 0], x[0, 0])
    angle = torch.tensor(3.0)
    expected = x[0, 1, 0] * torch.cos(angle) - x[0, 1, 1] * torch.sin(angle)
    torch.testing.assert_close(out[0, 1, 0], expected)
    assert "rope.cos" not in dict(rope.state_dict())
