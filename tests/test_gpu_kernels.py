"""sm_100a kernels against plain PyTorch fp32 references (needs a B200)."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from systems_for_llms_b200.ops import lib
    if not lib.available():
        pytest.skip("kernels need a compute-capability 10.x device")
    lib.lib()   # a missing or stale library must fail loudly here, not fall back
    return torch.device("cuda")


def rnd(dev, *shape, scale=1.0, seed=0):
    generator = torch.Generator(device=dev).manual_seed(seed)
    return (torch.randn(*shape, device=dev, generator=generator) * scale).to(torch.bfloat16)


def rel(a, b):
    a, b = a.float(), b.float()
    return ((a - b).abs().max() / (b.abs().max() + 1e-9)).item()


def check(dev):
    from systems_for_llms_b200.ops.gemm import check_status
    torch.cuda.synchronize()
    check_status()


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (256, 512, 256), (300, 200, 136),
                                   (4096, 3072, 1024), (1000, 10000, 512)])
def test_gemm_forward(dev, M, N, K):
    from systems_for_llms_b200.ops import gemm as G
    x, w = rnd(dev, M, K, seed=1), rnd(dev, N, K, seed=2)
    out = G.linear_fwd(x, w)
    check(dev)
    assert rel(out, x.float() @ w.float().t()) < 1e-2


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (300, 200, 136), (2048, 1024, 2752)])
def test_gemm_dgrad_and_wgrad(dev, M, N, K):
    from systems_for_llms_b200.ops import gemm as G
    dy, w, x = rnd(dev, M, N, seed=1), rnd(dev, N, K, seed=2), rnd(dev, M, K, seed=3)
    assert rel(G.linear_dgrad(dy, w), dy.float() @ w.float()) < 1e-2
    grad = torch.randn(N, K, device=dev)
    start = grad.clone()
    G.linear_wgrad(dy, x, grad, True)
    check(dev)
    expect = dy.float().t() @ x.float()
    assert rel(grad, start + expect) < 1e-4
    G.linear_wgrad(dy, x, grad, False)
    check(dev)
    assert rel(grad, expect) < 1e-4


def test_wgrad_grouped_matches_separate_products(dev):
    from systems_for_llms_b200.ops import gemm as G
    shapes = [(1024, 3072, 1024), (1024, 1024, 1024), (1024, 704, 520), (300, 200, 136)]
    problems, expected = [], []
    for index, (tokens, rows, cols) in enumerate(shapes):
        dy, x = rnd(dev, tokens, rows, seed=10 + index), rnd(dev, tokens, cols, seed=20 + index)
        grad = torch.randn(rows, cols, device=dev)
        accumulate = index % 2 == 0
        product = dy.float().t() @ x.float()
        expected.append(grad.clone() + product if accumulate else product)
        problems.append((dy, x, grad, accumulate))
    G.wgrad_grouped(problems)
    check(dev)
    for (_, _, grad, _), want in zip(problems, expected):
        assert rel(grad, want) < 1e-4
    # a product TMA cannot address (odd pitch) is computed on its own
    dy, x = rnd(dev, 64, 24, seed=1), rnd(dev, 64, 40, seed=2)
    odd = torch.zeros(24, 41, device=dev)[:, :40]
    G.wgrad_grouped([(dy, x, odd, False), problems[1]])
    check(dev)
    assert rel(odd, dy.float().t() @ x.float()) < 1e-4
    # two launches of the same group are bit-identical (no atomics across tiles)
    first = [g.clone() for _, _, g, _ in problems]
    for (_, _, grad, _), start in zip(problems, first):
        grad.copy_(start)
    G.wgrad_grouped([(dy_, x_, g_, True) for dy_, x_, g_, _ in problems])
    once = [g.clone() for _, _, g, _ in problems]
    for (_, _, grad, _), start in zip(problems, first):
        grad.copy_(start)
    G.wgrad_grouped([(dy_, x_, g_, True) for dy_, x_, g_, _ in problems])
    check(dev)
    assert all(torch.equal(a, g) for a, (_, _, g, _) in zip(once, problems))


def test_gemm_epilogues(dev):
    from systems_for_llms_b200.ops import gemm as G
    M, K, F = 512, 256, 344
    x = rnd(dev, M, K, seed=1)
    w = rnd(dev, 1024, K, scale=0.05, seed=2)
    resid = torch.randn(M, 1024, device=dev)
    out = G.linear_fwd_resid(x, w, resid)
    # the product is rounded to bf16 before the add; a flipped rounding moves one bf16 ulp
    assert rel(out, resid + (x.float() @ w.float().t()).bfloat16().float()) < 5e-3
    # rotary epilogue
    B, T, H, D = 2, 256, 2, 64
    wq = rnd(dev, 3 * H * D, K, scale=0.05, seed=3)
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2, device=dev).float() / D))
    angles = torch.arange(T, device=dev).float()[:, None] * inv[None]
    cos, sin = (f(angles).bfloat16().float().contiguous() for f in (torch.cos, torch.sin))
    got = G.linear_fwd_rope(x, wq, cos, sin, T, 2 * H * D, D).view(B, T, 3, H, D)
    y = (x.float() @ wq.float().t()).bfloat16().float().view(B, T, 3, H, D)
    want = y.clone()
    for part in range(2):
        even, odd = y[:, :, part, :, 0::2], y[:, :, part, :, 1::2]
        c, s = cos[None, :, None, :], sin[None, :, None, :]
        want[:, :, part, :, 0::2] = even * c - odd * s
        want[:, :, part, :, 1::2] = even * s + odd * c
    assert rel(got, want) < 1e-2
    # SwiGLU forward and backward
    w13 = rnd(dev, 2 * F, K, scale=0.05, seed=4)
    g, a13 = G.swiglu_fwd(x, w13, F)
    a = (x.float() @ w13.float().t()).bfloat16().float()
    assert rel(a13, a) < 1e-2
    assert rel(g, torch.nn.functional.silu(a[:, :F]) * a[:, F:]) < 1e-2
    dy, w2 = rnd(dev, M, K, seed=5), rnd(dev, K, F, scale=0.05, seed=6)
    d13 = G.swiglu_bwd(dy, w2, a13)
    check(dev)
    a1 = a13[:, :F].float().requires_grad_(True)
    a3 = a13[:, F:].float().requires_grad_(True)
    (torch.nn.functional.silu(a1) * a3).backward((dy.float() @ w2.float()).bfloat16().float())
    assert rel(d13, torch.cat([a1.grad, a3.grad], 1)) < 1e-2


@pytest.mark.parametrize("rows,dim", [(4096, 1024), (37, 16), (5, 50), (300, 384)])
def test_rmsnorm_forward_backward(dev, rows, dim):
    from systems_for_llms_b200.ops import functional as K
    x, w = torch.randn(rows, dim, device=dev), torch.randn(dim, device=dev)
    y, rstd = K.rmsnorm(x, w, 1e-5)
    xr, wr = x.clone().requires_grad_(True), w.clone().requires_grad_(True)
    ref = xr / torch.sqrt((xr * xr).mean(-1, keepdim=True) + 1e-5) * wr
    assert rel(y, ref.detach().bfloat16()) < 1e-2
    dy = torch.randn(rows, dim, device=dev).bfloat16()
    dres = torch.randn(rows, dim, device=dev)
    ref.backward(dy.float())
    dw = torch.ones(dim, device=dev)
    dx, dxb = K.rmsnorm_bwd(dy, x, w, rstd, dres, dw, True, want_bf16=True)
    check(dev)
    assert rel(dx, xr.grad + dres) < 1e-5
    assert rel(dxb, (xr.grad + dres).bfloat16()) < 1e-2
    assert rel(dw, wr.grad + 1) < 1e-4


@pytest.mark.parametrize("rows,vocab", [(512, 10000), (16, 32), (7, 1000), (5, 1003), (3, 20000)])
def test_cross_entropy(dev, rows, vocab):
    from systems_for_llms_b200.ops import functional as K
    ld = -(-vocab // 8) * 8
    logits = (torch.randn(rows, ld, device=dev) * 3).bfloat16()
    targets = torch.randint(0, vocab, (rows,), device=dev)
    dl = torch.empty_like(logits)
    losses = K.cross_entropy_rows(logits, targets, vocab, dl, 0.5)
    check(dev)
    wide = logits[:, :vocab].float().requires_grad_(True)
    ref = torch.nn.functional.cross_entropy(wide, targets, reduction="none")
    (ref.sum() * 0.5).backward()
    assert rel(losses, ref.detach()) < 1e-5
    assert rel(dl[:, :vocab], wide.grad.bfloat16()) < 1e-2


def test_adamw_and_norm(dev):
    from systems_for_llms_b200.ops import functional as K
    n = 1_000_003
    g = torch.randn(n, device=dev)
    p = torch.randn(n, device=dev)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    shadow = torch.empty(n, dtype=torch.bfloat16, device=dev)
    stats = K.grad_norm_and_coef(g, 1.0)
    norm = torch.linalg.vector_norm(g)
    assert abs(stats[0].item() - norm.item()) / norm.item() < 1e-6
    ref = torch.nn.Parameter(p.clone())
    opt = torch.optim.AdamW([ref], lr=3e-4, betas=(0.9, 0.95), weight_decay=0.1)
    for step in (1, 2, 3):
        ref.grad = g * stats[1]
        opt.step()
        K.adamw_step(p, g, m, v, shadow, step=step, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8,
                     weight_decay=0.1, coef=stats[1:2], ok_flag=stats[2:3])
    check(dev)
    assert (p - ref.detach()).abs().max().item() < 2e-6
    assert torch.equal(shadow, p.bfloat16())
    # a non-finite norm suppresses the update
    before = p.clone()
    bad = K.grad_norm_and_coef(torch.full((8,), float("nan"), device=dev), 1.0)
    K.adamw_step(p, g, m, v, shadow, step=4, lr=3e-4, beta1=0.9, beta2=0.95, eps=1e-8,
                 weight_decay=0.1, coef=bad[1:2], ok_flag=bad[2:3])
    check(dev)
    assert torch.equal(p, before) and bad[2].item() == 0.0


@pytest.mark.parametrize("rows,dim,vocab,skew", [(4096, 1024, 10000, False), (777, 96, 50, True),
                                                 (2048, 130, 1000, True)])
def test_embedding_backward_is_a_deterministic_scatter_add(dev, rows, dim, vocab, skew):
    """Against an fp64 index_add; bitwise repeatable; accumulate and overwrite modes;
    ``skew`` makes a few ids very frequent (long chains) and leaves many rows unused."""
    from systems_for_llms_b200.ops import functional as K
    torch.manual_seed(rows + dim)
    ids = torch.randint(0, vocab, (rows,), device=dev)
    if skew:
        ids[torch.rand(rows, device=dev) < 0.5] = 3
    dx = torch.randn(rows, dim, device=dev)
    expected = torch.zeros(vocab, dim, device=dev, dtype=torch.float64).index_add_(0, ids, dx.double())
    grad = torch.full((vocab, dim), 7.0, device=dev)          # overwrite must clear stale values
    assert K.embedding_bwd(dx, ids, grad, False)
    first = grad.clone()
    torch.testing.assert_close(grad.double(), expected, rtol=1e-5, atol=1e-3)
    grad.fill_(-1.0)
    assert K.embedding_bwd(dx, ids, grad, False)
    assert torch.equal(grad, first)                            # same order of additions every time
    assert K.embedding_bwd(dx, ids.view(1, rows), grad, True)  # second microbatch accumulates
    torch.testing.assert_close(grad.double(), 2 * expected, rtol=1e-5, atol=2e-3)
    too_many = torch.zeros(K.EMBEDDING_BWD_MAX_ROWS + 1, dtype=torch.int64, device=dev)
    assert not K.embedding_bwd(torch.zeros(too_many.numel(), 8, device=dev), too_many,
                               torch.zeros(4, 8, device=dev), False)


@pytest.mark.parametrize("d_model,heads,d_ff,ranks", [(512, 8, 1408, 4), (512, 8, 1408, 8),
                                                      (1024, 16, 2752, 8)])
def test_gemm_tensor_parallel_shard_shapes(dev, d_model, heads, d_ff, ranks):
    """The products of one tensor-parallel rank: narrow outputs (two heads, or one), a
    feed-forward slice that is only a multiple of 8 (344, 176) as output width and as
    reduction length (TMA zero-fills the ragged last 64-deep step)."""
    from systems_for_llms_b200.ops import gemm as G
    M, aw, ff = 1024, d_model // ranks, d_ff // ranks
    dk = d_model // heads
    x = rnd(dev, M, d_model, seed=1)
    wqkv = rnd(dev, 3 * aw, d_model, scale=0.05, seed=2)
    wo = rnd(dev, d_model, aw, scale=0.05, seed=3)
    w13 = rnd(dev, 2 * ff, d_model, scale=0.05, seed=4)
    w2 = rnd(dev, d_model, ff, scale=0.05, seed=5)
    attn = rnd(dev, M, aw, seed=6)
    resid = torch.randn(M, d_model, device=dev)
    T = 256
    inv = 1.0 / (10000.0 ** (torch.arange(0, dk, 2, device=dev).float() / dk))
    angles = torch.arange(T, device=dev).float()[:, None] * inv[None]
    cos, sin = (f(angles).bfloat16().float().contiguous() for f in (torch.cos, torch.sin))
    # q|k|v projection with rotary epilogue: the v columns are the plain product
    qkv = G.linear_fwd_rope(x, wqkv, cos, sin, T, 2 * aw, dk)
    plain = (x.float() @ wqkv.float().t())
    assert rel(qkv[:, 2 * aw:], plain[:, 2 * aw:]) < 1e-2
    # row-parallel products (reduction over the local width) as partial sums
    assert rel(G.linear_fwd(attn, wo), attn.float() @ wo.float().t()) < 1e-2
    assert rel(G.linear_fwd_resid(attn, wo, resid),
               resid + (attn.float() @ wo.float().t()).bfloat16().float()) < 5e-3
    g, a13 = G.swiglu_fwd(x, w13, ff)
    a = (x.float() @ w13.float().t()).bfloat16().float()
    want_g = torch.nn.functional.silu(a[:, :ff]) * a[:, ff:]
    assert rel(a13, a) < 1e-2 and rel(g, want_g) < 2e-2
    assert rel(G.linear_fwd(g, w2), g.float() @ w2.float().t()) < 1e-2
    # backward: activation derivative, input gradients, weight gradients
    dy = rnd(dev, M, d_model, seed=7)
    d13 = G.swiglu_bwd(dy, w2, a13)
    dg = (dy.float() @ w2.float()).bfloat16().float()
    a1, a3 = a13[:, :ff].float(), a13[:, ff:].float()
    sig = torch.sigmoid(a1)
    want = torch.cat([dg * a3 * (sig + a1 * sig * (1 - sig)), dg * a1 * sig], dim=1)
    assert rel(d13, want) < 2e-2
    assert rel(G.linear_dgrad(d13, w13), d13.float() @ w13.float()) < 1e-2
    dqkv = rnd(dev, M, 3 * aw, seed=8)
    assert rel(G.linear_dgrad(dqkv, wqkv), dqkv.float() @ wqkv.float()) < 1e-2
    problems, wants = [], []
    for dy_, x_ in ((dy, g), (d13, x), (dy, attn), (dqkv, x)):
        grad = torch.zeros(dy_.shape[1], x_.shape[1], device=dev)
        problems.append((dy_, x_, grad, False))
        wants.append(dy_.float().t() @ x_.float())
    G.wgrad_grouped(problems)
    check(dev)
    for (_, _, grad, _), want in zip(problems, wants):
        assert rel(grad, want) < 1e-3
