"""Out-of-bounds checks without a sanitizer: guard bands around kernel outputs, and the
bounds-checked debug build of the library (needs a B200)."""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def dev():
    from systems_for_llms_b200.ops import lib
    if not lib.available():
        pytest.skip("kernels need a compute-capability 10.x device")
    return torch.device("cuda")


def rnd(*shape, dev):
    return torch.randn(*shape, device=dev).bfloat16()


@pytest.mark.parametrize("M,N,K", [(1000, 520, 264), (128, 256, 64), (4096, 1000, 1024), (77, 8, 8)])
def test_gemm_outputs_stay_inside_their_rows(dev, M, N, K):
    """Ragged row and column tails, aligned (staged TMA epilogue) and unaligned (direct) pitches."""
    from systems_for_llms_b200.ops import gemm as G
    from systems_for_llms_b200.ops.canary import guarded
    from systems_for_llms_b200.ops.gemm import check_status
    x, w = rnd(M, K, dev=dev), rnd(N, K, dev=dev)
    out = guarded((M, N), torch.bfloat16, dev)
    G.linear_fwd(x, w, out.tensor)
    grad = guarded((N, K), torch.float32, dev)
    G.linear_wgrad(rnd(M, N, dev=dev), x, grad.tensor, False)
    dx = guarded((M, K), torch.bfloat16, dev)
    G.linear_dgrad(rnd(M, N, dev=dev), w, dx.tensor)
    torch.cuda.synchronize()
    check_status(dev)
    for name, g in (("forward", out), ("wgrad", grad), ("dgrad", dx)):
        assert g.intact(), f"{name} wrote outside its output"
        assert g.untouched() < g.nbytes // 50, f"{name} left part of its output unwritten"
    want = x.float() @ w.float().t()
    torch.testing.assert_close(out.tensor.float(), want, atol=0.05 * K ** 0.5, rtol=0.02)


@pytest.mark.parametrize("N,D", [(777, 64), (1000, 128), (129, 64)])
def test_attention_outputs_stay_inside_their_rows(dev, N, D):
    from systems_for_llms_b200.attention import flash
    from systems_for_llms_b200.attention.masks import MaskSpec
    from systems_for_llms_b200.ops.canary import guarded
    from systems_for_llms_b200.ops.gemm import check_status
    B, H = 2, 3
    q, k, v, upstream = (rnd(B, H, N, D, dev=dev) for _ in range(4))
    mask = flash.prepare_mask(q, None, MaskSpec(causal=True), None, "interval")
    out = guarded((B, H, N, D), torch.bfloat16, dev)
    lse = guarded((B, H, N), torch.float32, dev)
    flash.flash_fwd(q, k, v, out.tensor, lse.tensor, mask, D ** -0.5)
    grads = [guarded((B, H, N, D), torch.bfloat16, dev) for _ in range(3)]
    flash.flash_bwd(q, k, v, out.tensor, upstream, lse.tensor, *(g.tensor for g in grads), mask,
                    D ** -0.5)
    torch.cuda.synchronize()
    check_status(dev)
    for name, g in (("out", out), ("lse", lse), ("dq", grads[0]), ("dk", grads[1]),
                    ("dv", grads[2])):
        assert g.intact(), f"{name} was written out of bounds"
        assert g.untouched() < g.nbytes // 50, f"{name} has unwritten elements"
    assert torch.isfinite(out.tensor.float()).all()


def test_loss_gradient_and_embedding_gradient_stay_in_bounds(dev):
    from systems_for_llms_b200.ops import functional as K
    from systems_for_llms_b200.ops.canary import guarded
    from systems_for_llms_b200.ops.gemm import check_status
    rows, vocab = 300, 1000
    logits = rnd(rows, vocab, dev=dev)
    targets = torch.randint(0, vocab, (rows,), device=dev)
    dlogits = guarded((rows, vocab), torch.bfloat16, dev)
    K.cross_entropy_rows(logits, targets, vocab, dlogits.tensor, 1.0)
    table = guarded((50, 64), torch.float32, dev)
    ids = torch.randint(0, 50, (4, 40), device=dev)
    K.embedding_bwd(torch.randn(4, 40, 64, device=dev), ids, table.tensor, False)
    torch.cuda.synchronize()
    check_status(dev)
    assert dlogits.intact() and dlogits.untouched() < dlogits.nbytes // 50
    assert table.intact()


DEBUG_SCRIPT = r"""
import torch
from systems_for_llms_b200.models.transformer import TransformerLM
from systems_for_llms_b200.ops import lib
from systems_for_llms_b200.ops.gemm import check_status
from systems_for_llms_b200.optim import FusedAdamW
assert "debug" in lib.os.environ["SFL_LIBRARY"]
torch.manual_seed(0)
dev = torch.device("cuda")
model = TransformerLM(vocab_size=1000, context_length=200, d_model=128, num_layers=2, num_heads=2,
                      d_ff=344, rope_theta=10000.0, device=dev, dtype=torch.float32,
                      attention_backend="sdpa")
x = torch.randint(0, 1000, (3, 200), device=dev)
with torch.autocast("cuda", dtype=torch.bfloat16):
    loss = model.loss(x, x)
assert model._fused is not None
loss.backward()
FusedAdamW(model.parameters(), lr=1e-3, betas=(0.9, 0.95), weight_decay=0.1,
           engine=model._fused).clip_and_step(1.0)
torch.cuda.synchronize()
check_status(dev)          # a failed bounds predicate would have set the status word
assert torch.isfinite(loss).item()
print("debug build ok", loss.item())
"""


def test_bounds_checked_debug_build_runs_a_training_step_cleanly(dev, tmp_path):
    """-DSFL_DEBUG_BOUNDS compiles the store predicates in; a correct step must not trip
    any of them (ragged sequence length and a d_ff that is only a multiple of 8)."""
    from systems_for_llms_b200.ops import build
    library = build.build(defines=("SFL_DEBUG_BOUNDS",), output=tmp_path / "libsfl_debug.so")
    env = dict(os.environ, PYTHONPATH=str(ROOT), SFL_LIBRARY=str(library))
    result = subprocess.run([sys.executable, "-c", DEBUG_SCRIPT], cwd=ROOT, env=env,
                            capture_output=True, text=True, timeout=600)
    assert result.returncode == 0, result.stderr[-3000:]
    assert "debug build ok" in result.stdout
