"""Tensor parallelism over attention heads and feed-forward units.

Semantics follow the reference (distributed/llmdist/tensor_parallel.py:25-207):
every rank sees the whole batch; q/k/v and w1/w3 are split by output rows
(heads, hidden units), output_proj and w2 by input columns; embeddings, norms
and the vocabulary head are replicated; ``parallelize_model`` rewrites an
already initialised model in place from slices of identical weights without
touching the RNG; ``clip_grad_norm_tp`` counts sharded gradients on every rank
and replicated ones once; ``reconstruct_state_dict`` rebuilds full tensors.

Data paths:

* portable (any device): the two conjugate autograd functions below call
  ``torch.distributed.all_reduce``;
* B200 fused (see ``TensorParallelEngine``): the row-parallel GEMMs write bf16
  partial sums into symmetric memory and one kernel per reduction sums the
  peers' partials over NVLink, adds the fp32 residual and stores the result into
  every rank's buffer (``reduce_rows_resid``), so the all-reduce, the dtype
  promotion and the residual add are a single pass.
"""

from __future__ import annotations

import ctypes
import math
import os

import torch
import torch.distributed as dist
from torch import nn
from torch.nn import functional as F

from ..models.attention import scaled_dot_product_attention
from ..models.layers import silu


def _world(group) -> tuple[int, int]:
    if not dist.is_available() or not dist.is_initialized():
        raise RuntimeError("Tensor parallelism requires an initialized process group")
    return dist.get_world_size(group), dist.get_rank(group)


class _CopyToParallel(torch.autograd.Function):
    """Identity forward; sums the per-shard input gradients in backward."""

    @staticmethod
    def forward(ctx, value, group):
        ctx.group = group
        return value

    @staticmethod
    def backward(ctx, gradient):
        total = gradient.contiguous().clone()
        if dist.get_world_size(ctx.group) > 1:
            dist.all_reduce(total, group=ctx.group)
        return total, None


class _ReduceFromParallel(torch.autograd.Function):
    """Sums partial outputs in forward; identity backward (the loss is replicated)."""

    @staticmethod
    def forward(ctx, value, group):
        total = value.contiguous().clone()
        if dist.get_world_size(group) > 1:
            dist.all_reduce(total, group=group)
        return total

    @staticmethod
    def backward(ctx, gradient):
        return gradient, None


class _ShardLinear(nn.Module):
    """One rank's slice of a bias-free linear layer."""

    def __init__(self, original, dimension: int, rank: int, world_size: int):
        super().__init__()
        width = original.weight.shape[dimension] // world_size
        piece = original.weight.detach().narrow(dimension, rank * width, width).clone().contiguous()
        self.weight = nn.Parameter(piece, requires_grad=original.weight.requires_grad)
        self.weight._tp_shard_dim = dimension
        self.weight._tp_full_shape = tuple(original.weight.shape)
        self.out_features, self.in_features = piece.shape

    def forward(self, value):
        return F.linear(value, self.weight)


class _ParallelAttention(nn.Module):
    def __init__(self, original, group):
        super().__init__()
        world_size, rank = _world(group)
        self.group = group
        self.d_model, self.d_k = original.d_model, original.d_k
        self.num_heads = original.num_heads // world_size
        self.max_seq_len = original.max_seq_len
        self.attention_backend = original.attention_backend
        self.q_proj = _ShardLinear(original.q_proj, 0, rank, world_size)
        self.k_proj = _ShardLinear(original.k_proj, 0, rank, world_size)
        self.v_proj = _ShardLinear(original.v_proj, 0, rank, world_size)
        self.output_proj = _ShardLinear(original.output_proj, 1, rank, world_size)
        self.rope = original.rope

    def forward(self, value, token_positions=None):
        if value.ndim < 2 or value.shape[-1] != self.d_model:
            raise ValueError("Attention input must end in (sequence_length, d_model)")
        length = value.shape[-2]
        if length <= 0 or (self.max_seq_len is not None and length > self.max_seq_len):
            raise ValueError("Sequence length outside the configured context")
        if token_positions is None:
            token_positions = torch.arange(length, device=value.device)
        # One copy node shared by q, k and v: their input gradients are summed
        # locally first and cross the wire once.
        shared = _CopyToParallel.apply(value, self.group)

        def split(projected):
            return projected.unflatten(-1, (self.num_heads, self.d_k)).transpose(-3, -2)

        query, key, content = (split(proj(shared)) for proj in
                               (self.q_proj, self.k_proj, self.v_proj))
        if self.rope is not None:
            query = self.rope(query, token_positions)
            key = self.rope(key, token_positions)
        if self.attention_backend == "sdpa":
            attended = F.scaled_dot_product_attention(query, key, content, is_causal=True,
                                                      dropout_p=0.0)
        else:
            causal = torch.ones(length, length, device=value.device, dtype=torch.bool).tril()
            attended = scaled_dot_product_attention(query, key, content, mask=causal)
        merged = attended.transpose(-3, -2).flatten(-2)
        return _ReduceFromParallel.apply(self.output_proj(merged), self.group)


class _ParallelSwiGLU(nn.Module):
    def __init__(self, original, group):
        super().__init__()
        world_size, rank = _world(group)
        self.group = group
        self.d_model, self.d_ff = original.d_model, original.d_ff // world_size
        self.w1 = _ShardLinear(original.w1, 0, rank, world_size)
        self.w2 = _ShardLinear(original.w2, 1, rank, world_size)
        self.w3 = _ShardLinear(original.w3, 0, rank, world_size)

    def forward(self, value):
        shared = _CopyToParallel.apply(value, self.group)
        partial = self.w2(silu(self.w1(shared)) * self.w3(shared))
        return _ReduceFromParallel.apply(partial, self.group)


def parallelize_model(model, group=None):
    """Shard attention and feed-forward matrices in place.

    Every rank must hold the same full model.  All layers are validated before
    any is changed, and no random numbers are drawn.  Build the optimizer after.
    """
    world_size, _ = _world(group)
    if getattr(model, "_tp_parallelized", False):
        raise ValueError("Model is already tensor parallel")
    for layer in model.layers:
        if layer.attn.num_heads % world_size or layer.ffn.d_ff % world_size:
            raise ValueError(
                "Attention head count and feed-forward width must divide TP world size")
    for layer in model.layers:
        layer.attn = _ParallelAttention(layer.attn, group)
        layer.ffn = _ParallelSwiGLU(layer.ffn, group)
    model._tp_parallelized, model._tp_group = True, group
    model._fused = None
    return model


@torch.no_grad()
def clip_grad_norm_tp(model, max_norm, error_if_nonfinite=True):
    """Clip by the norm of the logical full-model gradient."""
    if not getattr(model, "_tp_parallelized", False):
        raise ValueError("Expected a tensor-parallel model")
    if not math.isfinite(max_norm) or max_norm < 0:
        raise ValueError("max_norm must be finite and nonnegative")
    _, rank = _world(model._tp_group)
    parameters = list(model.parameters())
    gradients = [p.grad for p in parameters if p.grad is not None]
    wide = any(g.dtype == torch.float64 for g in gradients)
    dtype = torch.float64 if wide else torch.float32
    squares = [torch.linalg.vector_norm(p.grad.detach(), 2, dtype=dtype).square()
               for p in parameters
               if p.grad is not None and (hasattr(p, "_tp_shard_dim") or rank == 0)]
    total = (torch.stack(squares).sum() if squares
             else torch.zeros((), device=parameters[0].device, dtype=dtype))
    dist.all_reduce(total, group=model._tp_group)
    norm = total.sqrt()
    if error_if_nonfinite and not torch.isfinite(norm):
        raise RuntimeError("Non-finite tensor-parallel gradient norm")
    coefficient = (max_norm / (norm + 1e-6)).clamp(max=1.0)
    for gradient in gradients:
        gradient.mul_(coefficient.to(device=gradient.device, dtype=gradient.dtype))
    return norm


def describe_sharding(model) -> dict:
    world_size, rank = _world(model._tp_group)
    sharded = sum(p.numel() for p in model.parameters() if hasattr(p, "_tp_shard_dim"))
    replicated = sum(p.numel() for p in model.parameters() if not hasattr(p, "_tp_shard_dim"))
    return {"world_size": world_size, "rank": rank,
            "local_sharded_parameters": sharded, "local_replicated_parameters": replicated,
            "logical_parameter_count": sharded * world_size + replicated,
            "replicated_components": ["token_embeddings", "RMSNorm", "lm_head"],
            "shard_dimensions": {name: getattr(p, "_tp_shard_dim", None)
                                 for name, p in model.named_parameters()}}


@torch.no_grad()
def reconstruct_state_dict(model) -> dict:
    """Full tensors on every rank (collective; meant for audits and final saves)."""
    world_size, _ = _world(model._tp_group)
    named = dict(model.named_parameters())
    full = {}
    for name, tensor in model.state_dict().items():
        dimension = getattr(named.get(name), "_tp_shard_dim", None)
        if dimension is None:
            full[name] = tensor.detach().clone()
            continue
        pieces = [torch.empty_like(tensor) for _ in range(world_size)]
        dist.all_gather(pieces, tensor.contiguous(), group=model._tp_group)
        full[name] = torch.cat(pieces, dim=dimension)
    return full


class TensorParallelComm:
    """Peer-memory buffers and reductions for the fused tensor-parallel engine.

    ``partial(M, d)`` is where a row-parallel GEMM writes its bf16 partial sums;
    ``reduce_residual`` sums the peers' partials, adds the fp32 residual and
    returns the fp32 result, which lives in a per-(layer, position) slot of a
    symmetric pool so it can serve as the saved activation without a copy;
    ``reduce_bf16`` does the same without a residual for input gradients.
    A peer may write into this rank's buffers only after this rank has entered
    the same collective (ready barrier), which is after it finished every use of
    the previous contents in stream order.
    """

    def __init__(self, device, group, num_layers: int):
        from . import comm as pm
        self.pm = pm
        self.device, self.group, self.num_layers = device, group, num_layers
        self.comm = pm.PeerComm(device, group, ctas=96)
        self.rows = self.cols = 0
        self.partial_buf = self.pool = self.small = self.stage = self.tile_flags = None
        self._calls = 0
        self._tile_epoch = 0
        # SFL_TP_UNFUSED=1 keeps the GEMM and its reduction as two kernels (A/B runs)
        self.fuse_gemm = os.environ.get("SFL_TP_UNFUSED", "0") != "1"
        # SFL_TP_FUSE_WIDE=0 keeps groups of more than two ranks on the two-kernel path
        self.fuse_wide = os.environ.get("SFL_TP_FUSE_WIDE", "1") != "0"

    def _ensure(self, rows: int, cols: int) -> None:
        if rows <= self.rows and cols == self.cols:
            return
        for buffer in (self.partial_buf, self.pool, self.small, self.stage, self.tile_flags):
            if buffer is not None:
                buffer.close()
        pm = self.pm
        self.comm._structs.clear()      # cached pointer tables name the old buffers
        self.rows, self.cols = rows, cols
        from ..ops import lib as _kernel_lib
        handle = _kernel_lib.lib()
        world = self.comm.world
        self.stage = pm.SymmetricBuffer(max(256, handle.sfl_gemm_tp_stage_bytes(rows, cols, world)),
                                        self.device, self.group)
        self.tile_flags = pm.SymmetricBuffer(
            max(256, handle.sfl_gemm_tp_tile_flag_bytes(rows, cols)), self.device, self.group)
        self.partial_buf = pm.SymmetricBuffer(rows * cols * 2, self.device, self.group)
        self.pool = pm.SymmetricBuffer(2 * self.num_layers * rows * cols * 4, self.device,
                                       self.group)
        self.small = pm.SymmetricBuffer(rows * cols * 2, self.device, self.group)

    def partial(self, rows: int, cols: int) -> torch.Tensor:
        self._ensure(rows, cols)
        return self.partial_buf.view(torch.bfloat16, rows * cols).view(rows, cols)

    def _slot(self) -> int:
        self._calls += 1
        return self._calls % 32

    def reduce_residual(self, partial: torch.Tensor, resid: torch.Tensor, position: int):
        rows, cols = partial.shape
        offset = position * self.rows * self.cols * 4
        self.comm.reduce_rows_resid(self.partial_buf, self.pool, 0, offset, resid, rows, cols,
                                    self._slot())
        return self.pool.view(torch.float32, rows * cols, offset).view(rows, cols)

    def can_fuse(self, cols: int) -> bool:
        """The one-kernel GEMM + all-reduce needs whole 256-column tiles.

        With two ranks every rank finishes every row; larger groups use owned tiles, whose
        waits rely on every rank running the same grid with all CTAs resident (parity with
        one GPU is tested at 4 and 8 ranks; 105.1 against 107.0 ms per step for the
        two-kernel path at 8 ranks).  ``SFL_TP_FUSE_WIDE=0`` keeps groups of more than two on
        the two-kernel path (GEMM, then ``reduce_rows``).
        """
        if not (self.fuse_gemm and self.comm.world > 1 and cols % 256 == 0):
            return False
        return self.comm.world == 2 or self.fuse_wide

    def _next_tile_epoch(self) -> int:
        self._tile_epoch += 1
        return self._tile_epoch

    def gemm_reduce_residual(self, a: torch.Tensor, weight: torch.Tensor, resid: torch.Tensor,
                             position: int) -> torch.Tensor:
        """``resid + sum over ranks of a @ weight.T`` (row-parallel forward) in one kernel:
        tiles go to their owner rank as they finish and the finished rows come back
        to every rank's pool slot while later tiles are still in the tensor cores."""
        rows, cols = a.shape[0], weight.shape[0]
        self._ensure(rows, cols)
        offset = position * self.rows * self.cols * 4
        self.comm.gemm_tp_reduce(a, weight, False, cols, self.stage, self.tile_flags, self.pool,
                                 offset, resid, self._slot(), self._next_tile_epoch())
        return self.pool.view(torch.float32, rows * cols, offset).view(rows, cols)

    def gemm_reduce_bf16(self, dy: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
        """bf16 ``sum over ranks of dy @ weight`` (column-parallel input gradient)."""
        rows, cols = dy.shape[0], weight.shape[1]
        self._ensure(rows, cols)
        self.comm.gemm_tp_reduce(dy, weight, True, cols, self.stage, self.tile_flags, self.small,
                                 0, None, self._slot(), self._next_tile_epoch())
        return self.small.view(torch.bfloat16, rows * cols).view(rows, cols)

    def fill_block_args(self, args, index: int, rows: int, cols: int) -> torch.Tensor:
        """Tensor-parallel part of a native block call (csrc/block.cu): pointer tables,
        pool offsets of the layer's two results, and barrier slots / epochs for the
        call's two fused products.  Returns the view where ``x_out`` will appear."""
        self._ensure(rows, cols)
        comm = self.comm
        pool = comm.tp_struct(self.stage, self.pool, self.tile_flags)
        small = comm.tp_struct(self.stage, self.small, self.tile_flags)
        args.tp_pool, args.tp_small = ctypes.addressof(pool), ctypes.addressof(small)
        slot_bytes = self.rows * self.cols * 4
        args.tp_off_mid, args.tp_off_out = 2 * index * slot_bytes, (2 * index + 1) * slot_bytes
        for i in range(2):
            slot = self._slot()
            args.tp_slot[i] = slot
            args.tp_epoch[i] = comm.next_epoch(slot)
            args.tp_tile_epoch[i] = self._next_tile_epoch()
        return self.pool.view(torch.float32, rows * cols, args.tp_off_out).view(rows, cols)

    def reduce_bf16(self, partial: torch.Tensor) -> torch.Tensor:
        rows, cols = partial.shape
        self.comm.reduce_rows_bf16(self.partial_buf, self.small, 0, 0, rows, cols, self._slot())
        return self.small.view(torch.bfloat16, rows * cols).view(rows, cols)

    def close(self) -> None:
        for buffer in (self.partial_buf, self.pool, self.small, self.stage, self.tile_flags):
            if buffer is not None:
                buffer.close()
        self.comm.close()


def enable_fused(model, config_autocast) -> object | None:
    """Attach peer-memory reductions to a parallelised model's fused engine."""
    with config_autocast:
        engine = model.fused_engine()
    if engine is None:
        return None
    if engine.tp is None:
        engine.tp = TensorParallelComm(engine.device, model._tp_group, len(model.layers))
    return engine


@torch.no_grad()
def fused_grad_stats(model, engine, max_norm: float) -> torch.Tensor:
    """Device vector ``[norm, clip coefficient, finite]`` of the logical full gradient.

    Every rank sums the squares of its whole flat gradient; replicated parameters
    were counted ``world`` times, so ``world - 1`` copies of their squared norm
    are subtracted.
    """
    world, _ = _world(model._tp_group)
    flat = engine.flat_grad[:engine.total]
    local = torch.linalg.vector_norm(flat, 2, dtype=torch.float32).square()
    replicated = [p.grad for p in model.parameters()
                  if p.grad is not None and not hasattr(p, "_tp_shard_dim")]
    shared = torch.stack(torch._foreach_norm(replicated)).square().sum()
    dist.all_reduce(local, group=model._tp_group)
    norm = (local - (world - 1) * shared).clamp_min(0).sqrt()
    coefficient = (max_norm / (norm + 1e-6)).clamp(max=1.0)
    return torch.stack([norm, coefficient, torch.isfinite(norm).float()])
