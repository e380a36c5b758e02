"""The allocation-free decode entry point, called through its exported C symbol.

``sfl_decode_static`` exists for callers that cannot allocate device memory at
the point where they decode (graph capture, latency-critical serving loops,
plug-ins without an allocator of their own, plain C programs): its split-KV
scratch is a fixed array inside the library.  The test loads the shared object
with ctypes - no Python wrapper in between - runs it twice in a row on different
inputs (the second call sees the first call's leftovers in the shared scratch)
and compares each result with the regular entry point that uses caller-provided
scratch.  It also checks that an oversized request is refused with a message.

The file name sorts last so that a run that stops at the first failure has
already exercised everything else.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def library():
    from systems_for_llms_b200.ops import build, lib
    if not lib.available():
        pytest.skip("kernels need a compute-capability 10.x device")
    build.build()
    handle = ctypes.CDLL(str(build.LIB_PATH))
    handle.sfl_decode_static.restype = ctypes.c_int
    handle.sfl_decode_static.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 6 + [
        ctypes.c_float, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    handle.sfl_decode_static_error.restype = ctypes.c_char_p
    handle.sfl_decode_static_capacity_slots.restype = ctypes.c_long
    return handle


def call_static(handle, q, k, v, lengths, splits, variant):
    out = torch.empty_like(q)
    B, Hq, D = q.shape
    Hkv, N = k.shape[1:3]
    code = handle.sfl_decode_static(
        q.data_ptr(), k.data_ptr(), v.data_ptr(), lengths.data_ptr(), out.data_ptr(), B, Hq, Hkv,
        N, D, splits, D ** -0.5, int(variant == "tile"), int(q.dtype == torch.float16),
        torch.cuda.current_stream().cuda_stream)
    return code, out


def test_static_scratch_matches_regular_entry_point_twice(library):
    from systems_for_llms_b200.attention.decode import decode
    device = torch.device("cuda")
    generator = torch.Generator(device=device).manual_seed(11)
    cases = [(torch.bfloat16, 2, 32, 4, 3000, 128, 32, "tile", [3000, 1234]),
             (torch.float16, 3, 8, 2, 700, 64, 5, "token", [700, 1, 0])]
    for dtype, B, Hq, Hkv, N, D, splits, variant, lens in cases:   # two calls in a row
        q = torch.randn(B, Hq, D, device=device, generator=generator).to(dtype)
        k = torch.randn(B, Hkv, N, D, device=device, generator=generator).to(dtype)
        v = torch.randn(B, Hkv, N, D, device=device, generator=generator).to(dtype)
        lengths = torch.tensor(lens, dtype=torch.int32, device=device)
        code, got = call_static(library, q, k, v, lengths, splits, variant)
        assert code == 0, library.sfl_decode_static_error()
        want = decode(q, k, v, lengths, splits=splits, variant=variant)
        torch.cuda.synchronize()
        tol = 0.02 if dtype == torch.bfloat16 else 0.004
        torch.testing.assert_close(got.float(), want.float(), atol=tol, rtol=tol)


def test_oversized_request_is_refused(library):
    device = torch.device("cuda")
    capacity = library.sfl_decode_static_capacity_slots()
    B, Hq, Hkv, N, D, splits = 8, 32, 4, 256, 64, 128        # 8 * 32 * 128 slots
    assert B * Hq * splits > capacity
    q = torch.zeros(B, Hq, D, device=device, dtype=torch.bfloat16)
    k = torch.zeros(B, Hkv, N, D, device=device, dtype=torch.bfloat16)
    lengths = torch.full((B,), N, dtype=torch.int32, device=device)
    code, _ = call_static(library, q, k, k, lengths, splits, "tile")
    assert code != 0
    assert b"capacity" in library.sfl_decode_static_error()


def test_bad_group_ratio_and_null_pointers_are_refused_before_anything_is_queued(library):
    """A plain C caller gets a message naming the problem instead of a faulting kernel or a
    misleading launch failure: both are rejected before the stream sees any work."""
    device = torch.device("cuda")
    stream = torch.cuda.current_stream().cuda_stream
    B, Hq, Hkv, N, D = 1, 6, 2, 64, 64                       # three query heads per KV head
    q = torch.zeros(B, Hq, D, device=device, dtype=torch.bfloat16)
    k = torch.zeros(B, Hkv, N, D, device=device, dtype=torch.bfloat16)
    lengths = torch.full((B,), N, dtype=torch.int32, device=device)
    code, _ = call_static(library, q, k, k, lengths, 2, "tile")
    assert code == -2
    assert b"1, 2, 4 or 8" in library.sfl_decode_static_error()
    out = torch.empty_like(q)
    code = library.sfl_decode_static(q.data_ptr(), None, k.data_ptr(), lengths.data_ptr(),
                                     out.data_ptr(), B, 4, Hkv, N, D, 2, D ** -0.5, 1, 0, stream)
    assert code == -2
    assert b"must not be null" in library.sfl_decode_static_error()
    torch.cuda.synchronize()
