"""Single-token attention over a contiguous KV cache (split-KV, GQA).

Interface of the reference binding (attention_lab/cuda_decode/kernel.py:27-118):
``prepare(q, k, v, lengths=None, *, splits=1, scale=None, variant="token")``
validates, allocates scratch and output once and returns a ``PreparedDecode``
whose call launches on the current stream without allocating - so it can be
captured in a CUDA graph, and ``lengths`` may be edited in place between calls;
``decode(...)`` is the one-shot form.  The kernels merge the splits inside the same
launch.  Three variants: ``"token"`` and ``"tile"`` are the reference's two softmax
schedules on the CUDA cores (csrc/decode.cu); ``"mma"`` computes the scores of a GQA
group and the weighted value sum as tcgen05 matrix products fed by TMA
(csrc/attention.cu, ``decode_mma2_kernel``: cached tokens are the rows of the score
tile, the head group its 16 columns) - the one that keeps up with HBM when several
query heads share a KV head.
"""

from __future__ import annotations

import math
from ctypes import c_float, c_int, c_void_p
from dataclasses import dataclass

import torch

from ..ops import lib as _lib

_P = c_void_p
_lib.register_signature("sfl_decode", [_P, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int,
                                       c_int, c_int, c_int, c_float, c_int, c_int, _P])
_lib.register_signature("sfl_decode_mma", [_P, _P, _P, _P, _P, _P, _P, _P, _P, c_int, c_int, c_int,
                                           c_int, c_int, c_int, c_float, c_int, _P, _P])
VARIANTS = ("token", "tile", "mma")


def _validate(q, k, v, lengths, splits):
    if type(splits) is not int or not 1 <= splits <= 128:
        raise ValueError("splits must be an integer in [1, 128]")
    if q.ndim != 3 or k.ndim != 4 or v.shape != k.shape:
        raise ValueError("expected q[B,Hq,D], k/v[B,Hkv,N,D]")
    batch, query_heads, dim = q.shape
    if min(q.shape) <= 0 or k.shape[0] != batch or k.shape[3] != dim:
        raise ValueError("Q/K/V batch and head dimensions must match and be nonempty")
    kv_heads, capacity = k.shape[1:3]
    if kv_heads <= 0 or capacity <= 0 or query_heads % kv_heads:
        raise ValueError("query heads must be divisible by positive KV heads")
    if dim not in (64, 128) or query_heads // kv_heads not in (1, 2, 4, 8):
        raise ValueError("supported head dimensions are 64/128 and GQA ratios 1/2/4/8")
    if q.dtype not in (torch.float16, torch.bfloat16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("Q/K/V must have the same FP16 or BF16 dtype")
    if not q.is_cuda or any(t.device != q.device for t in (k, v, lengths)):
        raise ValueError("all tensors must be on the same CUDA device")
    if any(not t.is_contiguous() for t in (q, k, v, lengths)):
        raise ValueError("all tensors must be contiguous")
    if lengths.dtype != torch.int32 or lengths.shape != (batch,):
        raise ValueError("lengths must be an int32 tensor of shape [B]")
    low, high = torch.aminmax(lengths)
    if low.item() < 0 or high.item() > capacity:
        raise ValueError("each length must be in [0, cache capacity]")
    return batch, query_heads, kv_heads, capacity, dim


@dataclass
class PreparedDecode:
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    lengths: torch.Tensor
    partial_max: torch.Tensor
    partial_sum: torch.Tensor
    partial_output: torch.Tensor
    counters: torch.Tensor
    output: torch.Tensor
    splits: int
    scale: float
    variant: str
    status: torch.Tensor | None = None

    def __call__(self) -> torch.Tensor:
        B, Hq, D = self.q.shape
        Hkv, N = self.k.shape[1:3]
        if self.variant == "mma":
            code = _lib.lib().sfl_decode_mma(
                self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.lengths.data_ptr(),
                self.partial_max.data_ptr(), self.partial_sum.data_ptr(),
                self.partial_output.data_ptr(), self.counters.data_ptr(), self.output.data_ptr(),
                B, Hq, Hkv, N, D, self.splits, self.scale, int(self.q.dtype == torch.float16),
                self.status.data_ptr(), _lib.stream_ptr())
            _lib.check(code, "sfl_decode_mma")
            return self.output
        code = _lib.lib().sfl_decode(
            self.q.data_ptr(), self.k.data_ptr(), self.v.data_ptr(), self.lengths.data_ptr(),
            self.partial_max.data_ptr(), self.partial_sum.data_ptr(),
            self.partial_output.data_ptr(), self.counters.data_ptr(), self.output.data_ptr(),
            B, Hq, Hkv, N, D, self.splits, self.scale, int(self.variant == "tile"),
            int(self.q.dtype == torch.float16), _lib.stream_ptr())
        _lib.check(code, "sfl_decode")
        return self.output

    @property
    def scratch_bytes(self) -> int:
        return sum(t.numel() * t.element_size()
                   for t in (self.partial_max, self.partial_sum, self.partial_output))


def prepare(q, k, v, lengths=None, *, splits=1, scale=None, variant="token") -> PreparedDecode:
    """Validate and allocate outside of capture; returns a reusable operation.

    The single query is the newest position, so every valid cache entry is
    visible.  Zero-length rows yield zeros.  Concurrent use needs separate
    prepared operations because scratch and output are owned by the object.
    """
    if variant not in VARIANTS:
        raise ValueError("variant must be one of " + ", ".join(VARIANTS))
    for tensor in (q, k, v):
        if not isinstance(tensor, torch.Tensor) or not tensor.is_cuda:
            raise ValueError("all tensors must be on the same CUDA device")
    if lengths is None:
        if q.ndim != 3 or k.ndim != 4:
            raise ValueError("expected q[B,Hq,D], k/v[B,Hkv,N,D]")
        lengths = torch.full((q.shape[0],), k.shape[2], device=q.device, dtype=torch.int32)
    batch, heads, kv_heads, _, dim = _validate(q, k, v, lengths, splits)
    if scale is None:
        scale = dim ** -0.5
    if not math.isfinite(scale) or scale <= 0:
        raise ValueError("scale must be finite and positive")
    maximum = torch.empty(batch, heads, splits, device=q.device, dtype=torch.float32)
    normalizer = torch.empty_like(maximum)
    numerator = torch.empty(batch, heads, splits, dim, device=q.device, dtype=torch.float32)
    counters = torch.zeros(batch, kv_heads, device=q.device, dtype=torch.int32)
    from ..ops.gemm import status_word
    return PreparedDecode(q, k, v, lengths, maximum, normalizer, numerator, counters,
                          torch.empty_like(q), splits, float(scale), variant,
                          status_word(q.device))


def decode(q, k, v, lengths=None, *, splits=1, scale=None, variant="token") -> torch.Tensor:
    """One-shot decode on the current stream."""
    return prepare(q, k, v, lengths, splits=splits, scale=scale, variant=variant)()
