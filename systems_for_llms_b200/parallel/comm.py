"""Symmetric peer memory and the fused collectives built on it.

Control plane: ``torch.distributed`` (NCCL on GPUs, gloo on CPU) for rendezvous,
barriers, object exchange and the baseline collectives - as in the reference,
which uses nothing else (distributed/llmdist/train.py:234-236).

Data plane on B200: every rank allocates identical buffers with ``cudaMalloc``,
exchanges CUDA IPC handles once through the process group and maps its peers'
buffers, after which the kernels in csrc/comm.cu move data with loads and stores
on peer pointers over NVLink / NVSwitch and synchronise through flag words.  This
module owns those buffers (``SymmetricBuffer``), the per-process communicator
(``PeerComm``) and thin launchers for the kernels.
"""

from __future__ import annotations

import ctypes
from ctypes import POINTER, Structure, c_float, c_int, c_long, c_size_t, c_uint, c_void_p

import torch
import torch.distributed as dist

from ..ops import lib as _lib
from ..ops.gemm import status_word

MAX_PEERS = 8


class CommStruct(Structure):
    """Mirror of ``SflComm`` (csrc/sfl.h)."""

    _fields_ = [("rank", c_int), ("world", c_int), ("data", c_void_p * MAX_PEERS),
                ("data2", c_void_p * MAX_PEERS), ("flags", c_void_p * MAX_PEERS)]


class TpFuseStruct(Structure):
    """Mirror of ``SflTpFuse`` (csrc/sfl.h)."""

    _fields_ = [("rank", c_int), ("world", c_int), ("stage", c_void_p * MAX_PEERS),
                ("out", c_void_p * MAX_PEERS), ("tile_flags", c_void_p * MAX_PEERS),
                ("flags", c_void_p * MAX_PEERS)]


_C = POINTER(CommStruct)
_P = c_void_p
for _name, _args in {
    "sfl_ipc_alloc": [POINTER(c_void_p), c_size_t],
    "sfl_ipc_free": [_P],
    "sfl_ipc_get_handle": [_P, _P],
    "sfl_ipc_open_handle": [_P, POINTER(c_void_p)],
    "sfl_ipc_close_handle": [_P],
    "sfl_comm_set_spin_limit": [c_uint],
    "sfl_allreduce_f32": [_C, c_long, c_long, c_float, c_int, c_uint, c_int, c_int, _P, _P],
    "sfl_reduce_scatter_f32": [_C, c_long, c_long, c_float, _P, c_int, c_uint, c_int, c_int, _P, _P],
    "sfl_comm_norm_finalize": [_C, _P, c_int, c_int, c_float, _P, _P, _P],
    "sfl_adamw_allgather": [_C, c_long, c_long, _P, _P, _P, c_float, c_float, c_float, c_float,
                            c_float, c_float, c_float, _P, _P, c_int, c_uint, c_int, _P, _P],
    "sfl_adamw_allgather_ranges": [_C, _P, c_int, _P, _P, _P, c_float, c_float, c_float, c_float,
                                   c_float, c_float, c_float, _P, _P, c_int, c_uint, c_int, _P, _P],
    "sfl_allgather_bytes": [_C, c_long, c_long, c_int, c_uint, c_int, _P, _P],
    "sfl_allgather_into": [_C, c_long, c_long, _P, c_int, c_uint, c_int, _P, _P],
    "sfl_reduce_rows_resid": [_C, c_long, c_long, _P, c_long, c_int, c_int, c_uint, c_int, _P, _P],
    "sfl_reduce_rows_bf16": [_C, c_long, c_long, c_long, c_int, c_int, c_uint, c_int, _P, _P],
    "sfl_allreduce_rows_f32": [_C, c_long, c_long, c_long, c_int, c_uint, c_int, _P, _P],
    "sfl_gemm_tp_stage_bytes": [c_int, c_int, c_int],
    "sfl_gemm_tp_tile_flag_bytes": [c_int, c_int],
    "sfl_gemm_tp_reduce": [_P, c_long, _P, c_long, c_int, c_int, c_int, c_int,
                           POINTER(TpFuseStruct), c_long, c_int, _P, c_long, c_int, c_uint,
                           c_uint, _P, _P],
}.items():
    _lib.register_signature(_name, _args)


class _DevicePointer:
    """Lets ``torch.as_tensor`` wrap raw device memory without copying."""

    def __init__(self, address: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1",
                                         "data": (address, False), "version": 2}


def wrap_device_memory(address: int, nbytes: int, device: torch.device) -> torch.Tensor:
    return torch.as_tensor(_DevicePointer(address, nbytes), device=device)


_symmetric_bytes = {"live": 0, "peak": 0}


def symmetric_memory_bytes() -> dict:
    """Bytes of this process's own symmetric buffers: ``live`` now and the ``peak`` since
    the last ``reset_symmetric_peak``.  They come from ``cudaMalloc`` directly, so
    ``torch.cuda.max_memory_allocated`` does not see them; a true peak figure of a
    multi-GPU run is the allocator's peak plus this peak."""
    return dict(_symmetric_bytes)


def reset_symmetric_peak() -> None:
    _symmetric_bytes["peak"] = _symmetric_bytes["live"]


class SymmetricBuffer:
    """``nbytes`` of device memory on every rank of ``group``, mapped on all peers.

    ``local`` is this rank's memory as a uint8 tensor; ``peer_ptrs[r]`` is the
    address at which rank ``r``'s copy is visible here.  Collective: every rank
    must construct buffers in the same order.
    """

    def __init__(self, nbytes: int, device: torch.device, group=None):
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        if self.world > MAX_PEERS:
            raise ValueError("peer-memory collectives support at most 8 ranks")
        self.nbytes = -(-nbytes // 256) * 256
        self.device = torch.device(device)
        handle = _lib.lib()
        with torch.cuda.device(self.device):
            base = c_void_p()
            _lib.check(handle.sfl_ipc_alloc(ctypes.byref(base), self.nbytes), "sfl_ipc_alloc")
            self._base = base.value
            _symmetric_bytes["live"] += self.nbytes
            _symmetric_bytes["peak"] = max(_symmetric_bytes["peak"], _symmetric_bytes["live"])
            self.peer_ptrs = [None] * self.world
            self.peer_ptrs[self.rank] = self._base
            self._opened = []
            if self.world > 1:
                token = ctypes.create_string_buffer(64)
                _lib.check(handle.sfl_ipc_get_handle(self._base, token), "sfl_ipc_get_handle")
                tokens = [None] * self.world
                dist.all_gather_object(tokens, bytes(token.raw), group=group)
                for peer, raw in enumerate(tokens):
                    if peer == self.rank:
                        continue
                    mapped = c_void_p()
                    _lib.check(handle.sfl_ipc_open_handle(raw, ctypes.byref(mapped)),
                               "sfl_ipc_open_handle")
                    self.peer_ptrs[peer] = mapped.value
                    self._opened.append(mapped.value)
        self.local = wrap_device_memory(self._base, self.nbytes, self.device)

    def view(self, dtype: torch.dtype, numel: int, byte_offset: int = 0) -> torch.Tensor:
        size = numel * torch.empty((), dtype=dtype).element_size()
        return self.local[byte_offset:byte_offset + size].view(dtype)

    def close(self) -> None:
        """Unmap peers and free the local memory (call on every rank, after a barrier)."""
        handle = _lib.lib()
        for address in self._opened:
            handle.sfl_ipc_close_handle(address)
        self._opened = []
        if self._base is not None:
            self.local = None
            handle.sfl_ipc_free(self._base)
            self._base = None
            _symmetric_bytes["live"] -= self.nbytes


class PeerComm:
    """Flag buffer, slot/epoch bookkeeping and kernel launchers for one group."""

    def __init__(self, device: torch.device, group=None, ctas: int = 32):
        self.device = torch.device(device)
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        handle = _lib.lib()
        self.flags = SymmetricBuffer(handle.sfl_comm_flag_bytes(), device, group)
        self.slots = handle.sfl_comm_slots()
        self.ctas = min(ctas, handle.sfl_comm_max_ctas())
        # The optimizer pass runs after backward with the GPU to itself: its kernels
        # (AdamW arithmetic on 34 bytes per element plus the parameter push) take the
        # whole machine instead of the few CTAs that collectives overlapped with
        # backward are limited to.
        self.update_ctas = handle.sfl_comm_max_ctas()
        self._epochs = [0] * self.slots
        self.status = status_word(self.device)
        self._structs: dict = {}

    def struct(self, primary: SymmetricBuffer, secondary: SymmetricBuffer | None = None):
        key = (id(primary), id(secondary))
        cached = self._structs.get(key)
        if cached is None:
            cached = CommStruct()
            cached.rank, cached.world = self.rank, self.world
            for peer in range(self.world):
                cached.data[peer] = primary.peer_ptrs[peer]
                cached.flags[peer] = self.flags.peer_ptrs[peer]
                if secondary is not None:
                    cached.data2[peer] = secondary.peer_ptrs[peer]
            self._structs[key] = cached
        return cached

    def next_epoch(self, slot: int) -> int:
        self._epochs[slot] += 1
        return self._epochs[slot]

    def set_spin_limit(self, iterations: int) -> None:
        with torch.cuda.device(self.device):
            _lib.check(_lib.lib().sfl_comm_set_spin_limit(iterations), "sfl_comm_set_spin_limit")

    # ------------------------------------------------------------ launchers --
    def allreduce(self, buffer: SymmetricBuffer, offset: int, count: int, scale: float,
                  slot: int, accumulate_partial: bool = False, ctas: int | None = None) -> None:
        """In-place ``scale * sum`` over ranks of fp32 ``buffer[offset:offset+count]``.
        ``ctas`` overrides the group's grid size (a reduction with nothing left to overlap
        with may take the whole GPU); a slot must keep one grid size within a step."""
        code = _lib.lib().sfl_allreduce_f32(
            ctypes.byref(self.struct(buffer)), offset, count, scale, slot, self.next_epoch(slot),
            int(accumulate_partial), ctas or self.ctas, self.status.data_ptr(), _lib.stream_ptr())
        _lib.check(code, "sfl_allreduce_f32")

    def reduce_scatter(self, buffer: SymmetricBuffer, offset: int, count: int, scale: float,
                       out: torch.Tensor | None, slot: int,
                       accumulate_partial: bool = False, accumulate_out: bool = False,
                       ctas: int | None = None) -> None:
        """Rank r keeps ``scale * sum`` of slice r (compact in ``out``); with
        ``accumulate_out`` the result is added to what ``out`` already holds."""
        flags = int(accumulate_partial) | (int(accumulate_out) << 1)
        code = _lib.lib().sfl_reduce_scatter_f32(
            ctypes.byref(self.struct(buffer)), offset, count, scale, _lib.ptr(out), slot,
            self.next_epoch(slot), flags, ctas or self.ctas, self.status.data_ptr(),
            _lib.stream_ptr())
        _lib.check(code, "sfl_reduce_scatter_f32")

    def norm_finalize(self, buffer: SymmetricBuffer, slots: torch.Tensor, max_norm: float,
                      extra_sq: torch.Tensor | None = None) -> torch.Tensor:
        """``[norm, clip coefficient, finite]`` from the partials left by reductions."""
        out = torch.empty(3, dtype=torch.float32, device=self.device)
        code = _lib.lib().sfl_comm_norm_finalize(
            ctypes.byref(self.struct(buffer)), slots.data_ptr(), slots.numel(), self.ctas,
            float(max_norm), _lib.ptr(extra_sq), out.data_ptr(), _lib.stream_ptr())
        _lib.check(code, "sfl_comm_norm_finalize")
        return out

    def adamw_allgather(self, params: SymmetricBuffer, shadows: SymmetricBuffer, offset: int,
                        count: int, grad: torch.Tensor, exp_avg: torch.Tensor,
                        exp_avg_sq: torch.Tensor, *, step: int, lr: float, beta1: float,
                        beta2: float, eps: float, weight_decay: float, coef: torch.Tensor | None,
                        ok: torch.Tensor | None, slot: int) -> None:
        code = _lib.lib().sfl_adamw_allgather(
            ctypes.byref(self.struct(params, shadows)), offset, count, grad.data_ptr(),
            exp_avg.data_ptr(), exp_avg_sq.data_ptr(), lr, beta1, beta2, eps, weight_decay,
            1.0 - beta1 ** step, 1.0 - beta2 ** step, _lib.ptr(coef), _lib.ptr(ok), slot,
            self.next_epoch(slot), self.update_ctas, self.status.data_ptr(), _lib.stream_ptr())
        _lib.check(code, "sfl_adamw_allgather")

    def adamw_allgather_ranges(self, params: SymmetricBuffer, shadows: SymmetricBuffer,
                               ranges: torch.Tensor, grad: torch.Tensor, exp_avg: torch.Tensor,
                               exp_avg_sq: torch.Tensor, *, step: int, lr: float, beta1: float,
                               beta2: float, eps: float, weight_decay: float,
                               coef: torch.Tensor | None, ok: torch.Tensor | None,
                               slot: int) -> None:
        """Sharded AdamW + parameter all-gather for every bucket range in one launch.

        ``ranges`` is an int64 device tensor ``[n, 3]`` of (element offset, element
        count, offset of this rank's slice inside ``grad`` / ``exp_avg`` /
        ``exp_avg_sq``).
        """
        if ranges.dtype != torch.int64 or ranges.dim() != 2 or ranges.shape[1] != 3 \
                or not ranges.is_contiguous():
            raise ValueError("ranges must be a contiguous int64 [n, 3] tensor")
        code = _lib.lib().sfl_adamw_allgather_ranges(
            ctypes.byref(self.struct(params, shadows)), ranges.data_ptr(), ranges.shape[0],
            grad.data_ptr(), exp_avg.data_ptr(), exp_avg_sq.data_ptr(), lr, beta1, beta2, eps,
            weight_decay, 1.0 - beta1 ** step, 1.0 - beta2 ** step, _lib.ptr(coef), _lib.ptr(ok),
            slot, self.next_epoch(slot), self.update_ctas, self.status.data_ptr(),
            _lib.stream_ptr())
        _lib.check(code, "sfl_adamw_allgather_ranges")

    def allgather_bytes(self, buffer: SymmetricBuffer, offset_bytes: int, chunk_bytes: int,
                        slot: int) -> None:
        code = _lib.lib().sfl_allgather_bytes(
            ctypes.byref(self.struct(buffer)), offset_bytes, chunk_bytes, slot,
            self.next_epoch(slot), self.ctas, self.status.data_ptr(), _lib.stream_ptr())
        _lib.check(code, "sfl_allgather_bytes")

    def allgather_into(self, source: SymmetricBuffer, src_offset_bytes: int, chunk_bytes: int,
                       dst: torch.Tensor, slot: int) -> None:
        """``dst`` (local) receives chunk r from every peer r's ``source`` buffer."""
        code = _lib.lib().sfl_allgather_into(
            ctypes.byref(self.struct(source)), src_offset_bytes, chunk_bytes, dst.data_ptr(),
            slot, self.next_epoch(slot), self.ctas, self.status.data_ptr(), _lib.stream_ptr())
        _lib.check(code, "sfl_allgather_into")

    def reduce_rows_resid(self, partial: SymmetricBuffer, out: SymmetricBuffer, in_off: int,
                          out_off: int, resid: torch.Tensor | None, rows: int, cols: int,
                          slot: int) -> None:
        code = _lib.lib().sfl_reduce_rows_resid(
            ctypes.byref(self.struct(partial, out)), in_off, out_off, _lib.ptr(resid), rows, cols,
            slot, self.next_epoch(slot), self.ctas, self.status.data_ptr(), _lib.stream_ptr())
        _lib.check(code, "sfl_reduce_rows_resid")

    def reduce_rows_bf16(self, partial: SymmetricBuffer, out: SymmetricBuffer, in_off: int,
                         out_off: int, rows: int, cols: int, slot: int) -> None:
        code = _lib.lib().sfl_reduce_rows_bf16(
            ctypes.byref(self.struct(partial, out)), in_off, out_off, rows, cols, slot,
            self.next_epoch(slot), self.ctas, self.status.data_ptr(), _lib.stream_ptr())
        _lib.check(code, "sfl_reduce_rows_bf16")

    def allreduce_rows_f32(self, partial: SymmetricBuffer, out: SymmetricBuffer, in_off: int,
                           out_off: int, count: int, slot: int) -> None:
        code = _lib.lib().sfl_allreduce_rows_f32(
            ctypes.byref(self.struct(partial, out)), in_off, out_off, count, slot,
            self.next_epoch(slot), self.ctas, self.status.data_ptr(), _lib.stream_ptr())
        _lib.check(code, "sfl_allreduce_rows_f32")

    def tp_struct(self, stage: SymmetricBuffer, out: SymmetricBuffer,
                  tile_flags: SymmetricBuffer) -> TpFuseStruct:
        key = ("tp", id(stage), id(out), id(tile_flags))
        cached = self._structs.get(key)
        if cached is None:
            cached = TpFuseStruct()
            cached.rank, cached.world = self.rank, self.world
            for peer in range(self.world):
                cached.stage[peer] = stage.peer_ptrs[peer]
                cached.out[peer] = out.peer_ptrs[peer]
                cached.tile_flags[peer] = tile_flags.peer_ptrs[peer]
                cached.flags[peer] = self.flags.peer_ptrs[peer]
            self._structs[key] = cached
        return cached

    def gemm_tp_reduce(self, a: torch.Tensor, b: torch.Tensor, b_mn: bool, n: int,
                       stage: SymmetricBuffer, tile_flags: SymmetricBuffer, out: SymmetricBuffer,
                       out_off: int, resid: torch.Tensor | None, slot: int,
                       tile_epoch: int) -> None:
        """One kernel: ``a @ b`` on this rank's K-slice, summed over ranks, finished
        (``resid + sum`` in fp32, or the bf16 sum when ``resid`` is None) and written
        into ``out`` at ``out_off`` bytes on every rank.  ``b`` is ``[n, K]``, or
        ``[K, n]`` with ``b_mn``."""
        m, k = a.shape
        code = _lib.lib().sfl_gemm_tp_reduce(
            a.data_ptr(), a.stride(0), b.data_ptr(), b.stride(0), int(b_mn), m, n, k,
            ctypes.byref(self.tp_struct(stage, out, tile_flags)), out_off, int(resid is None),
            _lib.ptr(resid), resid.stride(0) if resid is not None else 0, slot,
            self.next_epoch(slot), tile_epoch, self.status.data_ptr(), _lib.stream_ptr())
        _lib.check(code, "sfl_gemm_tp_reduce")

    def close(self) -> None:
        self.flags.close()


def peer_memory_available(device: torch.device) -> bool:
    """True on a B200 with the kernel library present (one process per GPU)."""
    return torch.device(device).type == "cuda" and _lib.available()
