"""Split-KV GQA decode against an fp32 token-level reference (needs a B200).

Coverage mirrors the reference's smoke matrix (attention_lab/cuda_decode/
study.py:73-124): dtypes x head dims x GQA ratios x lengths x splits, 128 splits
with a custom scale, a non-default stream, and CUDA-graph replay after an
in-place length change.  Tolerances: bf16 0.02, fp16 0.004.
"""

import itertools

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dev():
    from systems_for_llms_b200.ops import lib
    if not lib.available():
        pytest.skip("kernels need a compute-capability 10.x device")
    return torch.device("cuda")


def reference(q, k, v, lengths, scale):
    B, Hq, D = q.shape
    Hkv = k.shape[1]
    groups = Hq // Hkv
    out = torch.zeros(B, Hq, D, device=q.device)
    for b in range(B):
        n = int(lengths[b])
        if n == 0:
            continue
        for h in range(Hq):
            keys = k[b, h // groups, :n].float()
            values = v[b, h // groups, :n].float()
            weights = torch.softmax(keys @ q[b, h].float() * scale, 0)
            out[b, h] = weights @ values
    return out


MATRIX = list(itertools.product([torch.bfloat16, torch.float16], [64, 128], [1, 2, 4, 8]))


@pytest.mark.parametrize("dtype,D,groups", MATRIX)
def test_decode_matrix(dev, dtype, D, groups):
    from systems_for_llms_b200.attention.decode import decode
    generator = torch.Generator(device=dev).manual_seed(D + groups)
    B, Hkv, N = 3, 2, 520
    q = torch.randn(B, Hkv * groups, D, device=dev, generator=generator).to(dtype)
    k = torch.randn(B, Hkv, N, D, device=dev, generator=generator).to(dtype)
    v = torch.randn(B, Hkv, N, D, device=dev, generator=generator).to(dtype)
    tol = 0.02 if dtype == torch.bfloat16 else 0.004
    for lengths in ([1, 31, 32], [33, 127, 513], [0, 520, 64]):
        lens = torch.tensor(lengths, dtype=torch.int32, device=dev)
        want = reference(q, k, v, lengths, D ** -0.5)
        for splits, variant in itertools.product([1, 3, 8], ["token", "tile", "mma"]):
            got = decode(q, k, v, lens, splits=splits, variant=variant)
            torch.testing.assert_close(got.float(), want, atol=tol, rtol=tol,
                                       msg=f"{lengths} {splits} {variant}")


def test_many_splits_custom_scale_and_stream(dev):
    from systems_for_llms_b200.attention.decode import prepare
    q = torch.randn(2, 32, 128, device=dev).bfloat16()
    k = torch.randn(2, 4, 4096, 128, device=dev).bfloat16()
    v = torch.randn(2, 4, 4096, 128, device=dev).bfloat16()
    lens = torch.tensor([4096, 1000], dtype=torch.int32, device=dev)
    for variant in ("tile", "mma"):
        op = prepare(q, k, v, lens, splits=128, scale=0.05, variant=variant)
        assert op.scratch_bytes == 2 * 32 * 128 * 4 * 2 + 2 * 32 * 128 * 128 * 4
        stream = torch.cuda.Stream()
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            got = op().clone()
        stream.synchronize()
        torch.testing.assert_close(got.float(), reference(q, k, v, lens.tolist(), 0.05),
                                   atol=0.02, rtol=0.02, msg=variant)


@pytest.mark.parametrize("variant", ["tile", "mma"])
def test_cuda_graph_replay_after_length_change(dev, variant):
    from systems_for_llms_b200.attention.decode import prepare
    q = torch.randn(1, 8, 64, device=dev).half()
    k = torch.randn(1, 2, 2048, 64, device=dev).half()
    v = torch.randn(1, 2, 2048, 64, device=dev).half()
    lens = torch.tensor([2048], dtype=torch.int32, device=dev)
    op = prepare(q, k, v, lens, splits=16, variant=variant)
    op()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        op()
    for n in (2048, 700, 1):
        lens.fill_(n)
        graph.replay()
        torch.cuda.synchronize()
        torch.testing.assert_close(op.output.float(), reference(q, k, v, [n], 64 ** -0.5),
                                   atol=0.004, rtol=0.004)


def test_validation(dev):
    from systems_for_llms_b200.attention.decode import decode, prepare
    q = torch.randn(1, 8, 64, device=dev).half()
    k = torch.randn(1, 2, 128, 64, device=dev).half()
    with pytest.raises(ValueError):
        decode(q.cpu(), k.cpu(), k.cpu())
    with pytest.raises(ValueError):
        decode(q, k, k, splits=0)
    with pytest.raises(ValueError):
        decode(q, k, k, variant="block")
    with pytest.raises(TypeError):
        decode(q.float(), k.float(), k.float())
    with pytest.raises(ValueError):
        decode(q, k, k, torch.tensor([129], dtype=torch.int32, device=dev))
    with pytest.raises(ValueError):
        decode(q[:, :6], k, k)      # 6 / 2 = 3 is not a supported group size
    with pytest.raises(ValueError):
        prepare(q, k, k, scale=float("nan"))
