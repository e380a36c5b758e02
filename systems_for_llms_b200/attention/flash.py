"""Block-sparse flash attention on sm_100a: forward API and low-level launchers.

Public surface mirrors the reference's forward-only entry point
(attention_lab/triton_attention.py:326-438): ``attention(q, k, v, schedule, spec,
...)`` over contiguous ``[B, H, N, D]`` fp16/bf16 tensors with a compiled CSR
schedule or the metadata-free interval form, optional LSE output, and
``interval_regions`` as the host mirror of the interval arithmetic.  The kernels
themselves (csrc/attention.cu) are tcgen05/TMA kernels and accept arbitrary
batch/head/token strides, which the training model uses to read q, k and v
straight out of the fused projection output without a layout change.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_long, c_void_p
from dataclasses import dataclass

import torch

from ..ops import lib as _lib
from ..ops.gemm import status_word
from .masks import (KERNEL_TILE, BlockSchedule, KernelSchedule, MaskSpec, compile_mask,
                    to_kernel_schedule, validate_schedule)


class AttnTensor(Structure):
    _fields_ = [("ptr", c_void_p), ("stride_b", c_long), ("stride_h", c_long),
                ("stride_t", c_long)]


class AttnMask(Structure):
    _fields_ = [("mode", c_int), ("causal", c_int), ("window_left", c_int),
                ("window_right", c_int), ("doc", c_void_p),
                ("row_ptr", c_void_p), ("col_idx", c_void_p), ("full", c_void_p),
                ("bitmap", c_void_p),
                ("t_row_ptr", c_void_p), ("t_col_idx", c_void_p), ("t_full", c_void_p),
                ("t_bitmap", c_void_p)]


_A = POINTER(AttnTensor)
_lib.register_signature("sfl_attn_fwd", [_A, _A, _A, _A, c_void_p, c_int, c_int, c_int, c_int,
                                         c_float, POINTER(AttnMask), c_int, c_void_p, c_void_p])
_lib.register_signature("sfl_attn_fwd_pipeline",
                        [_A, _A, _A, _A, c_void_p, c_int, c_int, c_int, c_int, c_float,
                         POINTER(AttnMask), c_int, c_int, c_void_p, c_void_p])
PIPELINES = {None: 0, "default": 0, "one_stream": 1, "two_stream": 2, "two_stream_smem_p": 3}
_lib.register_signature("sfl_attn_bwd", [_A, _A, _A, _A, _A, c_void_p, c_void_p, _A, _A, _A,
                                         c_int, c_int, c_int, c_int, c_float, POINTER(AttnMask),
                                         c_int, c_void_p, c_void_p, c_void_p, c_void_p])
_lib.register_signature("sfl_rope_bwd", [c_void_p, c_long, c_void_p, c_void_p, c_long, c_int,
                                         c_int, c_int, c_void_p])


def interval_regions(length, spec, block_q, block_k, query_block):
    """Retained and full key-tile ranges ``(begin, full_begin, full_end, end)``
    of one query tile for a window-only spec; the kernels derive the same bounds
    in registers (reference mirror: attention_lab/triton_attention.py:11-36)."""
    if not isinstance(spec, MaskSpec) or spec.same_document:
        raise ValueError("interval schedules require a MaskSpec without document constraints")
    for name, value in (("length", length), ("block_q", block_q), ("block_k", block_k)):
        if type(value) is not int or value < 1:
            raise ValueError(f"{name} must be a positive integer")
    tiles = -(-length // block_q)
    if type(query_block) is not int or not 0 <= query_block < tiles:
        raise ValueError("query_block is out of bounds")
    q_lo = query_block * block_q
    q_hi = min(q_lo + block_q, length) - 1
    left, right = spec.window_left, spec.effective_right
    k_lo = 0 if left is None else max(0, q_lo - left)
    k_hi = length - 1 if right is None else min(length - 1, q_hi + right)
    begin, end = k_lo // block_k, k_hi // block_k + 1
    first_full = 0 if left is None else max(0, q_hi - left)
    full_begin = min(end, max(begin, -(-first_full // block_k)))
    if right is None or q_lo + right >= length - 1:
        full_end = end
    else:
        full_end = (q_lo + right + 1) // block_k
    full_end = max(full_begin, min(end, full_end))
    return begin, full_begin, full_end, end


@dataclass
class DeviceMask:
    """A mask uploaded to one device, ready to hand to the kernels."""

    struct: AttnMask
    tensors: tuple
    length: int
    mode: str


_mask_cache: dict = {}


def _window(value: int | None) -> int:
    return -1 if value is None else int(value)


def device_mask(device, length: int, spec: MaskSpec, *, mode: str = "interval",
                kernel_schedule: KernelSchedule | None = None,
                document_ids=None, cache_key=None) -> DeviceMask:
    """Uploads (and caches) the schedule arrays and document labels."""
    device = torch.device(device)
    key = None
    if cache_key is not None:
        key = (str(device), length, spec, mode, cache_key)
        hit = _mask_cache.get(key)
        if hit is not None:
            return hit
    struct = AttnMask()
    struct.mode = 1 if mode == "interval" else 0
    struct.causal = int(spec.causal)
    struct.window_left = _window(spec.window_left)
    struct.window_right = _window(spec.effective_right)
    keep = []
    if spec.same_document:
        if isinstance(document_ids, torch.Tensor):
            docs = document_ids.to(device=device, dtype=torch.int32).contiguous()
        else:
            docs = torch.tensor(list(document_ids), dtype=torch.int32, device=device)
        if docs.numel() != length:
            raise ValueError("document_ids must have exactly length elements")
        keep.append(docs)
        struct.doc = docs.data_ptr()
    if mode != "interval":
        if kernel_schedule is None:
            raise ValueError("a CSR mask needs a kernel schedule")
        ks = kernel_schedule

        def up(values, dtype):
            t = torch.tensor(values if len(values) else [0], dtype=dtype, device=device)
            keep.append(t)
            return t.data_ptr()

        def up_bits(values):
            # 64-bit patterns as signed int64
            signed = [v - (1 << 64) if v >= (1 << 63) else v for v in values]
            return up(signed, torch.int64)

        struct.row_ptr = up(ks.row_ptr, torch.int32)
        struct.col_idx = up(ks.col_idx, torch.int32)
        struct.full = up([int(f) for f in ks.full], torch.uint8)
        struct.t_row_ptr = up(ks.t_row_ptr, torch.int32)
        struct.t_col_idx = up(ks.t_col_idx, torch.int32)
        struct.t_full = up([int(f) for f in ks.t_full], torch.uint8)
        if ks.bitmap is not None:
            struct.bitmap = up_bits(ks.bitmap)
            struct.t_bitmap = up_bits(ks.t_bitmap)
    result = DeviceMask(struct, tuple(keep), length, mode)
    if key is not None:
        if len(_mask_cache) > 64:
            _mask_cache.clear()
        _mask_cache[key] = result
    return result


def causal_mask(device, length: int) -> DeviceMask:
    """Dense causal attention in interval form (what the training model uses)."""
    return device_mask(device, length, MaskSpec(causal=True), mode="interval", cache_key="causal")


def _view(t: torch.Tensor) -> AttnTensor:
    """``t`` is indexed [B, H, N, D] with D contiguous (any other strides)."""
    if t.dim() != 4 or t.stride(3) != 1:
        raise ValueError("attention tensors are [B, H, N, D] views with contiguous D")
    return AttnTensor(t.data_ptr(), t.stride(0), t.stride(1), t.stride(2))


def flash_fwd(q, k, v, out, lse, mask: DeviceMask, scale: float, pipeline: str | None = None) -> None:
    """Launch the forward kernel on [B, H, N, D] views (strided views allowed).

    ``pipeline`` picks the kernel variant (``PIPELINES``): ``two_stream`` (two independent
    work streams per CTA, P in tensor memory; the default at head dimension 64),
    ``two_stream_smem_p`` (P through shared memory) or ``one_stream`` (one query tile per
    CTA; what head dimension 128 always runs)."""
    if pipeline not in PIPELINES:
        raise ValueError(f"pipeline must be one of {sorted(k for k in PIPELINES if k)}")
    B, H, N, D = q.shape
    fp16 = int(q.dtype == torch.float16)
    status = status_word(q.device)
    code = _lib.lib().sfl_attn_fwd_pipeline(
        ctypes.byref(_view(q)), ctypes.byref(_view(k)), ctypes.byref(_view(v)),
        ctypes.byref(_view(out)), None if lse is None else lse.data_ptr(), B, H, N, D,
        float(scale), ctypes.byref(mask.struct), fp16, PIPELINES[pipeline], status.data_ptr(),
        _lib.stream_ptr())
    _lib.check(code, "sfl_attn_fwd")


def flash_bwd(q, k, v, out, d_out, lse, dq, dk, dv, mask: DeviceMask, scale: float,
              rope: tuple[torch.Tensor, torch.Tensor] | None = None) -> None:
    """Launch the dQ kernel (which also computes delta) and the dK/dV kernel.

    All tensors are [B, H, N, D] views.  ``rope = (cos, sin)``, fp32 ``[>=N, D/2]``
    tables of the interleaved-pair rotary embedding that produced q and k, makes
    the kernels return dq and dk as gradients of the un-rotated projections.
    """
    B, H, N, D = q.shape
    cos_ptr = sin_ptr = None
    if rope is not None:
        cos, sin = rope
        for table in (cos, sin):
            if (table.dtype != torch.float32 or table.dim() != 2 or table.shape[0] < N
                    or table.shape[1] != D // 2 or not table.is_contiguous()):
                raise ValueError("rotary tables are contiguous fp32 [>=N, D/2]")
        cos_ptr, sin_ptr = cos.data_ptr(), sin.data_ptr()
    fp16 = int(q.dtype == torch.float16)
    delta = torch.empty(B, H, N, dtype=torch.float32, device=q.device)
    status = status_word(q.device)
    code = _lib.lib().sfl_attn_bwd(
        ctypes.byref(_view(q)), ctypes.byref(_view(k)), ctypes.byref(_view(v)),
        ctypes.byref(_view(out)), ctypes.byref(_view(d_out)), lse.data_ptr(), delta.data_ptr(),
        ctypes.byref(_view(dq)), ctypes.byref(_view(dk)), ctypes.byref(_view(dv)), B, H, N, D,
        float(scale), ctypes.byref(mask.struct), fp16, status.data_ptr(), cos_ptr, sin_ptr,
        _lib.stream_ptr())
    _lib.check(code, "sfl_attn_bwd")


def rope_bwd_(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq_len: int, cols: int,
              head_dim: int) -> None:
    """In-place inverse rotation of the first ``cols`` columns of bf16 ``x[rows, ld]``."""
    code = _lib.lib().sfl_rope_bwd(x.data_ptr(), x.stride(0), cos.data_ptr(), sin.data_ptr(),
                                   x.shape[0], cols, seq_len, head_dim, _lib.stream_ptr())
    _lib.check(code, "sfl_rope_bwd")


def _check_inputs(q, k, v, *, allow_grad: bool) -> None:
    for name, t in (("q", q), ("k", k), ("v", v)):
        if not isinstance(t, torch.Tensor) or t.dim() != 4:
            raise ValueError(f"{name} must be a [B, H, N, D] tensor")
        if not t.is_cuda:
            raise ValueError("attention kernels need CUDA tensors")
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous")
        if not allow_grad and t.requires_grad:
            raise ValueError("the forward-only API does not accept tensors that require grad")
    if q.shape != k.shape or q.shape != v.shape:
        raise ValueError("q, k and v must have the same shape")
    if q.dtype not in (torch.float16, torch.bfloat16) or k.dtype != q.dtype or v.dtype != q.dtype:
        raise TypeError("q, k and v must share an fp16 or bf16 dtype")
    if q.shape[-1] not in (64, 128):
        raise ValueError("head dimension must be 64 or 128")


def prepare_mask(q, schedule: BlockSchedule | None, spec: MaskSpec, document_ids,
                 implementation: str, use_full_blocks: bool = True) -> DeviceMask:
    """Validates the schedule against the inputs and uploads the kernel form."""
    N = q.shape[2]
    if implementation not in ("csr", "interval"):
        raise ValueError("implementation must be 'csr' or 'interval'")
    if not isinstance(spec, MaskSpec):
        raise TypeError("spec must be a MaskSpec")
    if implementation == "interval":
        if spec.same_document:
            raise ValueError("the interval implementation does not support document masks")
        if schedule is not None:
            validate_schedule(schedule)
            if schedule.length != N:
                raise ValueError("schedule length does not match the sequence length")
        return device_mask(q.device, N, spec, mode="interval",
                           cache_key=("interval", use_full_blocks))
    if schedule is None:
        schedule = compile_mask(N, spec, KERNEL_TILE, KERNEL_TILE, _doc_list(document_ids))
    validate_schedule(schedule)
    if schedule.length != N:
        raise ValueError("schedule length does not match the sequence length")
    ks = to_kernel_schedule(schedule)
    if not use_full_blocks:
        ks.full = [False] * len(ks.full)
        ks.t_full = [False] * len(ks.t_full)
    docs = _doc_list(document_ids) if spec.same_document else None
    key = (schedule.block_q, schedule.block_k, tuple(schedule.row_ptr), tuple(schedule.col_idx),
           tuple(schedule.full_blocks), use_full_blocks, None if docs is None else tuple(docs))
    return device_mask(q.device, N, spec, mode="csr", kernel_schedule=ks, document_ids=docs,
                       cache_key=key)


def _doc_list(document_ids):
    if document_ids is None:
        return None
    if isinstance(document_ids, torch.Tensor):
        return [int(x) for x in document_ids.tolist()]
    return list(document_ids)


def attention(q, k, v, schedule, spec, *, document_ids=None, implementation="csr",
              use_full_blocks=True, return_lse=False, scale=None, num_warps=4, num_stages=2,
              launch_metadata=None, pipeline=None):
    """Forward-only block-sparse attention.

    ``pipeline`` selects the forward kernel variant (see ``flash_fwd``); it is the knob the
    configuration search turns on this hardware.  ``num_warps`` / ``num_stages`` are
    accepted for signature compatibility with the reference's tunable Triton kernel and
    validated, but the sm_100a kernels have fixed warp-specialised layouts.
    ``launch_metadata`` (a dict) receives the static resource figures of the variant used.
    """
    _check_inputs(q, k, v, allow_grad=False)
    if num_warps not in (1, 2, 4, 8) or num_stages not in (1, 2, 3, 4):
        raise ValueError("num_warps must be in {1,2,4,8} and num_stages in {1,2,3,4}")
    mask = prepare_mask(q, schedule, spec, document_ids, implementation, use_full_blocks)
    B, H, N, D = q.shape
    out = torch.empty_like(q)
    lse = torch.empty(B, H, N, dtype=torch.float32, device=q.device) if return_lse else None
    flash_fwd(q, k, v, out, lse, mask, D ** -0.5 if scale is None else scale, pipeline)
    if launch_metadata is not None:
        two = D == 64 and pipeline != "one_stream"
        launch_metadata.update({
            "kernel_name": f"attn_fwd2_kernel<{D}>" if two else f"attn_fwd_kernel<{D}>",
            "pipeline": ("one_stream" if not two else pipeline or "two_stream"),
            "threads": 384 if two else 192, "tile": KERNEL_TILE, "tensor_memory_columns": 512,
            "source": "static configuration of the sm_100a kernel; not a profiler measurement",
        })
    return (out, lse) if return_lse else out
