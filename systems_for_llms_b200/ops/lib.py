"""ctypes access to the sm_100a kernel library.

``lib()`` returns the loaded ``libsfl_b200.so`` with argument types declared.
On a machine with a CUDA device the library is required: a missing or stale
build raises instead of silently falling back to eager PyTorch, so a GPU run
can never pass on the wrong code path.
"""

from __future__ import annotations

import ctypes
import os
from ctypes import POINTER, Structure, c_char_p, c_float, c_int, c_long, c_uint, c_void_p
from functools import lru_cache

import torch

from . import build as _build


class GemmEpilogue(Structure):
    """Mirror of ``SflGemmEpilogue`` in csrc/sfl.h."""

    _fields_ = [
        ("kind", c_int), ("beta", c_int),
        ("out", c_void_p), ("ldo", c_long),
        ("out2", c_void_p), ("ldo2", c_long),
        ("aux", c_void_p), ("ldaux", c_long),
        ("rope_cos", c_void_p), ("rope_sin", c_void_p),
        ("rope_T", c_int), ("rope_cols", c_int), ("head_dim", c_int),
        ("dual_offset", c_int), ("dual_rows", c_int),
        ("status", c_void_p),
    ]


class WgradProblem(Structure):
    """Mirror of ``SflWgradProblem`` in csrc/sfl.h."""

    _fields_ = [
        ("dy", c_void_p), ("ld_dy", c_long), ("x", c_void_p), ("ld_x", c_long),
        ("grad", c_void_p), ("ld_grad", c_long),
        ("rows", c_int), ("cols", c_int), ("tokens", c_int), ("accumulate", c_int),
    ]


class BlockArgs(Structure):
    """Mirror of ``SflBlockArgs`` in csrc/sfl.h."""

    _fields_ = [
        ("batch", c_int), ("seq_len", c_int), ("d_model", c_int), ("heads", c_int),
        ("head_dim", c_int), ("d_ff", c_int),
        ("eps1", c_float), ("eps2", c_float), ("attn_scale", c_float),
        ("wqkv", c_void_p), ("wo", c_void_p), ("w13", c_void_p), ("w2", c_void_p),
        ("norm1", c_void_p), ("norm2", c_void_p), ("rope_cos", c_void_p), ("rope_sin", c_void_p),
        ("mask", c_void_p), ("x", c_void_p), ("x_out", c_void_p), ("saved", c_void_p),
        ("d_out", c_void_p), ("d_out_bf16", c_void_p), ("dx", c_void_p), ("dx_bf16", c_void_p),
        ("scratch", c_void_p),
        ("g_wqkv", c_void_p), ("g_wo", c_void_p), ("g_w13", c_void_p), ("g_w2", c_void_p),
        ("g_norm1", c_void_p), ("g_norm2", c_void_p),
        ("acc_wqkv", c_int), ("acc_wo", c_int), ("acc_w13", c_int), ("acc_w2", c_int),
        ("acc_norm1", c_int), ("acc_norm2", c_int),
        ("status", c_void_p),
        ("tp_pool", c_void_p), ("tp_small", c_void_p), ("tp_off_mid", c_long),
        ("tp_off_out", c_long), ("tp_slot", c_int * 2), ("tp_epoch", c_uint * 2),
        ("tp_tile_epoch", c_uint * 2),
    ]


EPI_BF16, EPI_F32, EPI_RESID, EPI_ROPE, EPI_SWIGLU, EPI_SWIGLU_BWD = range(6)

_P = c_void_p
_SIGNATURES = {
    "sfl_gemm_bf16": [_P, c_long, c_int, _P, c_long, c_int, c_int, c_int, c_int,
                      POINTER(GemmEpilogue), c_int, c_int, _P],
    "sfl_gemm_wgrad_grouped": [POINTER(WgradProblem), c_int, _P, _P],
    "sfl_block_forward": [POINTER(BlockArgs), _P],
    "sfl_block_backward": [POINTER(BlockArgs), _P],
    "sfl_block_saved_bytes": [POINTER(BlockArgs)],
    "sfl_block_scratch_bytes": [POINTER(BlockArgs)],
    "sfl_rmsnorm_fwd": [_P, _P, _P, _P, c_int, c_int, c_float, _P],
    "sfl_rmsnorm_bwd_blocks": [c_int],
    "sfl_rmsnorm_bwd": [_P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, _P],
    "sfl_rmsnorm_dw_reduce": [_P, c_int, _P, c_int, c_int, _P],
    "sfl_cross_entropy": [_P, c_long, _P, _P, _P, c_float, c_int, c_int, _P],
    "sfl_sqnorm_blocks": [c_long],
    "sfl_sqnorm_partial": [_P, c_long, _P, _P],
    "sfl_norm_finalize": [_P, c_int, c_float, c_float, _P, _P],
    "sfl_adamw": [_P, _P, _P, _P, _P, c_long, c_float, c_float, c_float, c_float, c_float,
                  c_float, c_float, _P, c_float, _P, _P],
    "sfl_cast_f32_to_bf16": [_P, _P, c_long, _P],
    "sfl_scale_f32": [_P, c_long, _P, c_float, _P],
    "sfl_scale_bf16_unless_one": [_P, c_long, _P, _P],
    "sfl_embedding_fwd": [_P, _P, _P, c_int, c_int, c_int, _P],
    "sfl_embedding_bwd": [_P, _P, _P, c_int, c_int, c_int, c_int, _P, _P, _P],
}
_OPTIONAL: dict[str, list] = {}


def register_signature(name: str, argtypes: list) -> None:
    """Lets other modules (attention, comm) declare their entry points."""
    _OPTIONAL[name] = argtypes
    lib.cache_clear()


# Kernels launched per call of each entry point (default 1, 0 for host-only calls).
_KERNELS_PER_CALL = {"sfl_attn_bwd": 2, "sfl_embedding_bwd": 2, "sfl_block_forward": 7, "sfl_block_backward": 11,
                     "sfl_block_saved_bytes": 0, "sfl_block_scratch_bytes": 0, "sfl_rmsnorm_bwd_blocks": 0, "sfl_sqnorm_blocks": 0,
                     "sfl_ipc_alloc": 0, "sfl_ipc_free": 0, "sfl_ipc_get_handle": 0,
                     "sfl_ipc_open_handle": 0, "sfl_ipc_close_handle": 0,
                     "sfl_comm_set_spin_limit": 0, "sfl_comm_flag_bytes": 0, "sfl_comm_slots": 0,
                     "sfl_comm_max_ctas": 0, "sfl_gemm_tp_stage_bytes": 0,
                     "sfl_gemm_tp_tile_flag_bytes": 0}
_launches = [0]


def launch_count() -> int:
    """Number of this library's kernels launched by the current process so far."""
    return _launches[0]


class _Library:
    """The loaded shared object with typed entry points that count their launches."""

    def __init__(self, handle: ctypes.CDLL):
        self._handle = handle

    def _bind(self, name: str, argtypes: list):
        function = getattr(self._handle, name)
        function.argtypes = argtypes
        function.restype = c_long if name.endswith("_bytes") else c_int
        weight = _KERNELS_PER_CALL.get(name, 1)
        counter = _launches

        def call(*args):
            counter[0] += weight
            return function(*args)

        setattr(self, name, call if weight else function)

    def __getattr__(self, name):   # entry points without a declared signature
        return getattr(self._handle, name)


@lru_cache(maxsize=1)
def lib() -> "_Library":
    """The kernel library.  ``SFL_LIBRARY=/path/lib.so`` loads an instrumented variant built
    with ``ops.build.build(defines=..., output=...)`` (bounds-checked stores, phase timers)
    instead of the in-tree optimised build."""
    override = os.environ.get("SFL_LIBRARY")
    if override:
        handle = ctypes.CDLL(override)
    else:
        if not _build.LIB_PATH.exists() or not _build.is_current():
            _build.build()
        handle = ctypes.CDLL(str(_build.LIB_PATH))
    library = _Library(handle)
    for name, argtypes in {**_SIGNATURES, **_OPTIONAL}.items():
        library._bind(name, argtypes)
    handle.sfl_version.restype = c_char_p
    handle.sfl_version.argtypes = []
    handle.sfl_comm_flag_bytes.restype = c_long
    return library


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = torch.cuda.current_device
if _raw_stream is None:     # very old builds: fall back to the object API
    def _raw_stream(index):  # noqa: F811
        return torch.cuda.current_stream(index).cuda_stream


def available() -> bool:
    """True when kernels can run: a CUDA device of compute capability 10.x."""
    if not torch.cuda.is_available():
        return False
    major, _ = torch.cuda.get_device_capability()
    return major == 10


def stream_ptr() -> int:
    """Raw handle of the calling thread's current CUDA stream.

    ``torch.cuda.current_stream()`` builds a Python ``Stream`` object per call
    (several microseconds, paid once per kernel launch); the raw query is the
    same lookup without the object.
    """
    return _raw_stream(_current_device())


def ptr(tensor: torch.Tensor | None) -> int | None:
    return None if tensor is None else tensor.data_ptr()


def check(code: int, what: str) -> None:
    if code != 0:
        raise RuntimeError(f"{what} failed with code {code}")
