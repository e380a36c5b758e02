"""Fused sm_100a engine against the portable PyTorch path (needs a B200)."""

import dataclasses
import json

import pytest
import torch

pytestmark = pytest.mark.gpu

CFG = dict(vocab_size=1000, context_length=256, d_model=128, num_layers=2, num_heads=2, d_ff=344,
           rope_theta=10000.0, attention_backend="sdpa")


@pytest.fixture(scope="module")
def dev():
    from systems_for_llms_b200.ops import lib
    if not lib.available():
        pytest.skip("kernels need a compute-capability 10.x device")
    return torch.device("cuda")


def build(dev, **overrides):
    from systems_for_llms_b200.models.transformer import TransformerLM
    torch.manual_seed(0)
    return TransformerLM(**{**CFG, **overrides}, device=dev, dtype=torch.float32)


def relative(a, b):
    return ((a - b).norm() / (b.norm() + 1e-12)).item()


@pytest.mark.parametrize("ckpt", ["none", "block"])
def test_fused_matches_portable(dev, ckpt):
    from systems_for_llms_b200.ops.gemm import check_status
    from systems_for_llms_b200.optim import FusedAdamW
    fused, plain = build(dev, activation_checkpointing=ckpt), build(dev, activation_checkpointing=ckpt)
    plain.disable_fused()
    x = torch.randint(0, 1000, (3, 256), device=dev)
    y = torch.randint(0, 1000, (3, 256), device=dev)
    for _ in range(2):     # second pass exercises accumulation into the flat buffer
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss_f, loss_p = fused.loss(x, y, 0.5), plain.loss(x, y, 0.5)
        loss_f.backward()
        loss_p.backward()
    assert fused._fused is not None, "the fused engine must be the path that ran"
    torch.cuda.synchronize()
    check_status()
    assert loss_f.item() == pytest.approx(loss_p.item(), rel=2e-3)
    for (name, a), (_, b) in zip(fused.named_parameters(), plain.named_parameters()):
        assert relative(a.grad, b.grad) < 0.03, name
        assert a.grad.data_ptr() == fused._fused.grad_view(a).data_ptr()
    with torch.autocast("cuda", dtype=torch.bfloat16):
        logits_f, logits_p = fused(x), plain(x)
    assert logits_f.shape == logits_p.shape == (3, 256, 1000)
    assert relative(logits_f.float(), logits_p.float()) < 0.02
    opt_f = FusedAdamW(fused.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1,
                       engine=fused._fused)
    opt_p = torch.optim.AdamW(plain.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1)
    norm_f = opt_f.clip_and_step(0.5)
    norm_p = torch.nn.utils.clip_grad_norm_(plain.parameters(), 0.5)
    opt_p.step()
    assert norm_f.item() == pytest.approx(norm_p.item(), rel=5e-3)
    # optimizer state is exposed in torch.optim.AdamW's format
    state = opt_f.state_dict()["state"]
    assert set(state[0]) == {"step", "exp_avg", "exp_avg_sq"} and float(state[0]["step"]) == 1.0
    with torch.autocast("cuda", dtype=torch.bfloat16), torch.no_grad():
        after_f, after_p = fused.loss(x, y).item(), plain.loss(x, y).item()
    assert after_f == pytest.approx(after_p, rel=5e-3)
    check_status()


def test_gradient_arriving_at_the_loss_is_applied(dev):
    """The head skips its scaling pass when the incoming gradient is exactly one; any
    other factor (a caller scaling the loss) must still reach every parameter."""
    model = build(dev)
    x = torch.randint(0, 1000, (2, 256), device=dev)
    y = torch.randint(0, 1000, (2, 256), device=dev)
    grads = []
    for factor in (1.0, -2.5):
        model.zero_grad(set_to_none=True)
        with torch.autocast("cuda", dtype=torch.bfloat16):
            loss = model.loss(x, y, 1.0)
        (loss * factor).backward()
        grads.append([p.grad.clone() for p in model.parameters()])
    for unit, scaled in zip(*grads):
        assert relative(scaled, -2.5 * unit) < 0.02


def test_shadow_follows_external_parameter_changes(dev):
    model = build(dev)
    x = torch.randint(0, 1000, (2, 128), device=dev)
    y = torch.randint(0, 1000, (2, 128), device=dev)
    with torch.autocast("cuda", dtype=torch.bfloat16), torch.no_grad():
        first = model.loss(x, y).item()
        state = {k: v.clone() for k, v in model.state_dict().items()}
        for p in model.parameters():
            p.mul_(0.5)
        changed = model.loss(x, y).item()
        model.load_state_dict(state)
        restored = model.loss(x, y).item()
    assert changed != first and restored == first


def test_trainer_runs_bf16_on_gpu(dev, tmp_path):
    from systems_for_llms_b200 import train as trainer
    from systems_for_llms_b200.config import DataConfig, ModelConfig, TrainConfig
    config = TrainConfig(
        model=ModelConfig(**{k: v for k, v in CFG.items() if k != "rope_theta"}),
        data=DataConfig(kind="synthetic", synthetic_tokens=20000), device="cuda", precision="bf16",
        batch_size=2, grad_accum_steps=2, max_steps=6, warmup_steps=1, learning_rate=1e-3,
        min_learning_rate=1e-4, eval_interval=3, eval_batches=2, eval_batch_size=2,
        checkpoint_interval=3)
    summary = trainer.run(config, tmp_path / "run")
    assert summary["status"] == "completed"
    rows = [json.loads(line) for line in (tmp_path / "run" / "metrics.jsonl").read_text().splitlines()]
    losses = [r["loss"] for r in rows if r["event"] == "train"]
    assert losses[-1] < losses[0]
    checkpoint = torch.load(tmp_path / "run" / "checkpoint.pt", weights_only=True)
    assert all(v.dtype == torch.float32 for v in checkpoint["model"].values())
    # resume continues from the checkpoint with the fused optimizer state
    trainer.run(config, tmp_path / "a", stop_after=3)
    resumed = trainer.run(config, tmp_path / "b", resume=tmp_path / "a" / "checkpoint.pt")
    assert resumed["valid_loss"] == pytest.approx(summary["valid_loss"], rel=1e-3)


def test_library_is_loaded_from_the_source_tree(dev):
    from systems_for_llms_b200.ops import build
    maps = open("/proc/self/maps").read()
    assert str(build.LIB_PATH) in maps
