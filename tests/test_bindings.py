"""The ctypes mirrors of the library's C structures must match the compiled layout."""

import ctypes

import pytest

from systems_for_llms_b200.ops import build as builder


@pytest.fixture(scope="module")
def library():
    from systems_for_llms_b200.ops import lib
    try:
        builder.build()
        return lib.lib()
    except Exception as error:      # no CUDA toolkit on this machine
        pytest.skip(f"kernel library unavailable: {error}")


def test_struct_sizes_match_the_compiled_library(library):
    from systems_for_llms_b200.attention.flash import AttnMask, AttnTensor
    from systems_for_llms_b200.ops.lib import BlockArgs, GemmEpilogue, WgradProblem
    from systems_for_llms_b200.parallel.comm import CommStruct, TpFuseStruct
    handle = library._handle
    handle.sfl_struct_sizes.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.c_int]
    handle.sfl_struct_sizes.restype = ctypes.c_int
    sizes = (ctypes.c_int * 8)()
    count = handle.sfl_struct_sizes(sizes, 8)
    mirrors = [GemmEpilogue, WgradProblem, AttnTensor, AttnMask, CommStruct, BlockArgs, TpFuseStruct]
    assert count == len(mirrors)
    assert [ctypes.sizeof(m) for m in mirrors] == list(sizes)[:count]


def test_block_runner_rejects_bad_shapes_without_a_gpu(library):
    from systems_for_llms_b200.ops.lib import BlockArgs
    args = BlockArgs()
    assert library.sfl_block_saved_bytes(ctypes.byref(args)) == -1       # all zero
    args.batch, args.seq_len, args.d_model, args.heads, args.head_dim, args.d_ff = 4, 1024, 1024, 16, 64, 2752
    saved = library.sfl_block_saved_bytes(ctypes.byref(args))
    scratch = library.sfl_block_scratch_bytes(ctypes.byref(args))
    tokens = 4 * 1024
    # h1, qkv, attn, h2, a13, g in bf16; x_mid in fp32; statistics
    expected = tokens * 2 * (1024 + 3072 + 1024 + 1024 + 2 * 2752 + 2752) + tokens * 1024 * 4
    statistics = 4 * 16 * 1024 * 4 + 2 * tokens * 4        # log-sum-exp, two 1/rms vectors
    assert expected + statistics <= saved <= expected + statistics + 16 * 256
    assert scratch > tokens * 2 * (2 * 2752 + 3 * 1024)
    args.head_dim = 48                                                     # unsupported width
    assert library.sfl_block_saved_bytes(ctypes.byref(args)) == -1
    assert library.sfl_block_forward(ctypes.byref(args), None) == -2     # refused before any launch


def test_fused_tensor_parallel_gemm_validates_before_launching(library):
    from systems_for_llms_b200.parallel.comm import TpFuseStruct
    assert library.sfl_gemm_tp_stage_bytes(4096, 1024, 2) == 2 * 32 * 4 * 128 * 256 * 2
    assert library.sfl_gemm_tp_tile_flag_bytes(4096, 1024) == 32 * 4 * 8 * 8 * 4
    assert library.sfl_gemm_tp_stage_bytes(1000, 512, 8) == 8 * 8 * 2 * 128 * 256 * 2   # ragged rows
    table = TpFuseStruct()
    call = library._handle.sfl_gemm_tp_reduce
    call.restype = ctypes.c_int
    call.argtypes = None
    args = lambda n, world: (ctypes.c_void_p(256), ctypes.c_long(64), ctypes.c_void_p(512),
                             ctypes.c_long(64), 0, 128, n, 64, ctypes.byref(table),
                             ctypes.c_long(0), 1, None, ctypes.c_long(0), 0, 1, 1, None, None)
    table.rank, table.world = 0, 1
    assert call(*args(256, 1)) == -2          # a group of one has nothing to reduce
    table.world = 2
    assert call(*args(200, 2)) == -2          # N must be whole 256-column tiles
    assert call(*args(256, 2)) == -2          # pointer tables not filled in


def test_new_elementwise_entry_points_validate_before_launching(library):
    handle = library._handle
    bwd = handle.sfl_embedding_bwd
    bwd.restype = ctypes.c_int
    bwd.argtypes = None
    p = ctypes.c_void_p(256)
    # rows <= 0, and more rows than fit in shared memory, are refused without a launch
    assert bwd(p, p, p, 0, 8, 10, 0, p, p, None) == -2
    assert bwd(p, p, p, 60000, 8, 10, 0, p, p, None) == -2
    assert bwd(p, p, None, 16, 8, 10, 0, p, p, None) == -2
    scale = handle.sfl_scale_bf16_unless_one
    scale.restype = ctypes.c_int
    scale.argtypes = None
    assert scale(None, ctypes.c_long(8), p, None) == -2
    assert scale(p, ctypes.c_long(0), p, None) == 0            # nothing to do


def test_fused_tensor_parallel_staging_arithmetic_stays_in_bounds(library):
    """The kernel's strip and flag addressing, restated on the host, for the largest
    indices of several shapes: every 4 KB block and every flag word must lie inside
    the buffers whose sizes the library reports."""
    BM, BN, WARPS, PEERS, BLOCK = 128, 256, 8, 8, 4096
    for M, N, world in [(4096, 1024, 2), (4096, 1024, 8), (1000, 512, 2), (130, 256, 3),
                        (16384, 2048, 4)]:
        m_tiles, n_tiles = -(-M // BM), N // BN
        tiles = m_tiles * n_tiles
        stage = library.sfl_gemm_tp_stage_bytes(M, N, world)
        flags = library.sfl_gemm_tp_tile_flag_bytes(M, N)
        tile_elems = BM * BN
        worst_block = worst_flag = 0
        for rank in (0, world - 1):
            for tile in (0, tiles - 1):
                for quarter in range(4):
                    strip = quarter * 32
                    base = ((rank * tiles + tile) * tile_elems + strip * BN) * 2
                    for chunk in range(BN // 64):
                        worst_block = max(worst_block, base + chunk * BLOCK + BLOCK)
                for warp in range(WARPS):
                    worst_flag = max(worst_flag, ((tile * PEERS + rank) * WARPS + warp) * 4 + 4)
        assert worst_block <= stage, (M, N, world)
        assert worst_flag <= flags, (M, N, world)
        # strips of one tile tile the 64 KB exactly: 4 quarters x 4 chunks x 4 KB
        assert 4 * (BN // 64) * BLOCK == tile_elems * 2
