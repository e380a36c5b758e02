"""Fully sharded data parallelism on the fused sm_100a engine (B200).

The reference wraps every block with PyTorch FSDP2 and lets NCCL all-gather fp32
shards before each block's forward and backward and reduce-scatter fp32
gradients after it (distributed/llmdist/train.py:258-262).  Here the same
ZeRO-3 schedule runs on the engine's flat layout and our peer-memory kernels:

* The flat parameter space is cut into ranges - embeddings, one per block, head.
  Rank r owns slice r of every range: fp32 master weights, AdamW moments and the
  gradient slice (1/world of the model each), plus a bf16 shadow slice kept in
  symmetric memory.  Only the RMSNorm weights (0.02 % of the model) stay
  replicated; their gradients are all-reduced once per step.
* Before a block runs, ``allgather_into`` pulls the peers' bf16 shadow slices of
  that block over NVLink into one of two local staging buffers on a side stream,
  one block ahead of compute (backward walks the other way).  What crosses the
  wire is bf16 - half the bytes of the reference's fp32 gathers - and the GEMMs
  read the staging buffer directly.
* Weight-gradient GEMMs write fp32 into one of two block-sized symmetric staging
  buffers; when the block's backward is done a ``reduce_scatter`` kernel sums the
  peers' staging buffers slice-wise straight into the owner's gradient slice
  (scaled by 1/world, accumulated over microbatches), overlapped with the next
  block's backward.
* The optimizer step is local: global norm from the slices (+ one scalar
  all-reduce), fused AdamW on the owned slices writing the new bf16 shadow, then
  the root tensors (fp32 embeddings, bf16 head) are re-gathered for the next step.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn

from ..models import fused
from ..ops import functional as K
from . import comm as pm


class FusedShardedTransformer(nn.Module):
    def __init__(self, model, engine, group=None, comm_ctas: int = 48):
        super().__init__()
        self.model = model
        self.engine = engine
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        device = engine.device
        W = self.world
        total = engine.total
        # ---- ranges: embeddings | blocks | head --------------------------------
        first = engine.layer_ranges[0][0]
        self.ranges = [(0, first), *engine.layer_ranges, (engine.head_offset, total)]
        for begin, end in self.ranges:
            if (end - begin) % (8 * W):
                raise ValueError("flat ranges must divide into 16-byte aligned slices")
        self.chunks = [(end - begin) // W for begin, end in self.ranges]
        self.shard_offsets = [0]
        for chunk in self.chunks:
            self.shard_offsets.append(self.shard_offsets[-1] + chunk)
        shard_numel = self.shard_offsets[-1]
        self.comm = pm.PeerComm(device, group, ctas=comm_ctas)
        # ---- owned slices ---------------------------------------------------------
        self.master_buf = pm.SymmetricBuffer(shard_numel * 4, device, group)
        self.shadow_buf = pm.SymmetricBuffer(shard_numel * 2, device, group)
        master = self.master_buf.view(torch.float32, shard_numel)
        self.shadow_shard = self.shadow_buf.view(torch.bfloat16, shard_numel)
        flat = engine.flat_param
        for j, (begin, _) in enumerate(self.ranges):
            lo = begin + self.rank * self.chunks[j]
            master[self.shard_offsets[j]:self.shard_offsets[j + 1]].copy_(
                flat[lo:lo + self.chunks[j]])
        K.cast_bf16(master, self.shadow_shard)
        self.shard = nn.Parameter(master)
        self.grad_shard = torch.zeros(shard_numel, dtype=torch.float32, device=device)
        self.exp_avg = torch.zeros_like(self.grad_shard)
        self.exp_avg_sq = torch.zeros_like(self.grad_shard)
        # ---- replicated norm weights ---------------------------------------------
        self.norm_params = [p for p in engine.params if p.dim() == 1]
        norm_numel = sum(p.numel() for p in self.norm_params)
        quantum = 4 * W * 64
        padded = -(-norm_numel // quantum) * quantum
        self.norm_numel = padded
        # One more quantum behind the norm gradients carries this rank's squared shard
        # norm through the same peer all-reduce, so the global gradient norm needs no
        # collective of its own (element `padded` of the buffer).
        self.norm_flat = torch.zeros(padded, dtype=torch.float32, device=device)
        self.norm_grad_buf = pm.SymmetricBuffer((padded + quantum) * 4, device, group)
        self.norm_grad_all = self.norm_grad_buf.view(torch.float32, padded + quantum)
        self.norm_grad = self.norm_grad_all[:padded]
        self.norm_exp_avg = torch.zeros_like(self.norm_flat)
        self.norm_exp_avg_sq = torch.zeros_like(self.norm_flat)
        self.norm_offsets = {}
        cursor = 0
        for p in self.norm_params:
            self.norm_flat[cursor:cursor + p.numel()].copy_(p.data)
            self.norm_offsets[id(p)] = cursor
            cursor += p.numel()
        # ---- staging ------------------------------------------------------------
        block_len = max(end - begin for begin, end in self.ranges)
        self.weight_stage = [torch.empty(block_len, dtype=torch.bfloat16, device=device)
                             for _ in range(2)]
        self.grad_stage_buf = [pm.SymmetricBuffer(block_len * 4, device, group) for _ in range(2)]
        self.grad_stage = [b.view(torch.float32, block_len) for b in self.grad_stage_buf]
        emb_len = self.ranges[0][1] - self.ranges[0][0]
        head_len = self.ranges[-1][1] - self.ranges[-1][0]
        self.emb_full = torch.empty(emb_len, dtype=torch.float32, device=device)
        self.head_full = torch.empty(head_len, dtype=torch.bfloat16, device=device)
        self.stream = torch.cuda.Stream(device=device)
        self.resident = [None, None]       # range index held by each weight staging buffer
        self.gather_done = [None, None]    # events
        self.stage_free = [None, None]     # events: reduce-scatter finished reading
        self.first_microbatch = True
        self.step_count = 0
        self._slot = 0
        self._last_prepared = None
        # ---- release the replicated copies and re-route the engine --------------------
        placeholder = torch.zeros(1, dtype=torch.float32, device=device)
        self.matrix_range = {}
        for p in engine.params:
            if p.dim() == 1:
                offset = self.norm_offsets[id(p)]
                p.data = self.norm_flat[offset:offset + p.numel()]
                p.grad = None
            else:
                self.matrix_range[id(p)] = self._range_of(engine.offsets[id(p)])
                p.data = placeholder.expand(p.shape)
                p.grad = None
        engine.flat_param = None
        engine.flat_shadow = None
        engine.flat_grad = None
        engine.shadow = self._shadow
        engine.grad_view = self._grad_view
        engine.claim = self._claim
        engine.prepare_block = self._prepare_block
        engine.embedding_table = self._embedding_table
        engine.sync_shadow = lambda: None
        engine.on_block_backward = self._on_backward_progress
        model._fused = engine
        self._gather_root()

    # -------------------------------------------------------------- bookkeeping --
    def _range_of(self, offset: int) -> int:
        for j, (begin, end) in enumerate(self.ranges):
            if begin <= offset < end:
                return j
        raise ValueError("offset outside the flat layout")

    def _next_slot(self) -> int:
        self._slot = (self._slot + 1) % 48
        return self._slot

    def named_parameters(self, prefix: str = "", recurse: bool = True,
                         remove_duplicate: bool = True):
        """Trainable tensors of this rank: the owned slice and the replicated norms."""
        yield (prefix + ("." if prefix else "") + "shard", self.shard)
        for name, p in self.model.named_parameters():
            if p.dim() == 1:
                yield (prefix + ("." if prefix else "") + "model." + name, p)

    def parameters(self, recurse: bool = True):
        for _, p in self.named_parameters():
            yield p

    # ------------------------------------------------------------------ gathers --
    def _gather_range(self, j: int, dst: torch.Tensor, source: pm.SymmetricBuffer,
                      element_size: int) -> None:
        chunk = self.chunks[j]
        self.comm.allgather_into(source, self.shard_offsets[j] * element_size, chunk * element_size,
                                 dst, self._next_slot())

    def _gather_root(self) -> None:
        """fp32 embeddings and bf16 head for the coming step (after an update)."""
        self._gather_range(0, self.emb_full, self.master_buf, 4)
        self._gather_range(len(self.ranges) - 1, self.head_full, self.shadow_buf, 2)
        self.resident = [None, None]
        self._last_prepared = None

    def _start_gather(self, j: int) -> None:
        slot = j % 2
        if self.resident[slot] == j:
            return
        current = torch.cuda.current_stream()
        self.stream.wait_stream(current)      # the buffer's previous reader is behind us
        with torch.cuda.stream(self.stream):
            self._gather_range(j, self.weight_stage[slot], self.shadow_buf, 2)
            event = torch.cuda.Event()
            event.record(self.stream)
        self.resident[slot] = j
        self.gather_done[slot] = event

    def _prepare_block(self, index: int, backward: bool) -> None:
        """Make block ``index``'s weights resident and prefetch its successor
        (predecessor when walking backward) on the side stream."""
        j = index + 1                          # range index of the block
        key = (j, backward)
        if self._last_prepared == key or (self._last_prepared == (j, True) and not backward):
            return                             # same block again (recompute inside backward)
        self._last_prepared = key
        slot = j % 2
        self._start_gather(j)
        if self.gather_done[slot] is not None:
            torch.cuda.current_stream().wait_event(self.gather_done[slot])
            self.gather_done[slot] = None
        neighbour = j - 1 if backward else j + 1
        if 1 <= neighbour <= len(self.ranges) - 2:
            self._start_gather(neighbour)

    # ------------------------------------------------------------ engine lookups --
    def _embedding_table(self) -> torch.Tensor:
        weight = self.model.token_embeddings.weight
        return self.emb_full.view(weight.shape)

    def _shadow(self, p: torch.Tensor, rows: int | None = None) -> torch.Tensor:
        j = self.matrix_range[id(p)]
        rows = p.shape[0] if rows is None else rows
        rel = self.engine.offsets[id(p)] - self.ranges[j][0]
        source = self.head_full if j == len(self.ranges) - 1 else self.weight_stage[j % 2]
        return source[rel:rel + rows * p.shape[1]].view(rows, p.shape[1])

    def _grad_view(self, p: torch.Tensor, rows: int | None = None) -> torch.Tensor:
        if p.dim() == 1:
            offset = self.norm_offsets[id(p)]
            return self.norm_grad[offset:offset + p.numel()]
        j = self.matrix_range[id(p)]
        rows = p.shape[0] if rows is None else rows
        rel = self.engine.offsets[id(p)] - self.ranges[j][0]
        self._claim_stage(j)
        return self.grad_stage[j % 2][rel:rel + rows * p.shape[1]].view(rows, p.shape[1])

    def _claim_stage(self, j: int) -> None:
        """Before the first write of range ``j``'s gradients, wait until the
        reduce-scatter that last read this staging buffer (on every rank) is done."""
        slot = j % 2
        event = self.stage_free[slot]
        if event is not None:
            torch.cuda.current_stream().wait_event(event)
            self.stage_free[slot] = None

    def _claim(self, *params: torch.Tensor) -> bool:
        if params[0].dim() != 1:
            return False                       # staging buffers are always overwritten
        fresh = all(p.grad is None for p in params)
        for p in params:
            view = self._grad_view(p)
            if p.grad is None:
                p.grad = view
        return not fresh

    def _on_backward_progress(self, offset: int) -> None:
        """Backward finished the range that starts at ``offset``: reduce-scatter it."""
        j = self._range_of(offset) if offset > 0 else 0
        begin, end = self.ranges[j]
        slot = j % 2
        self.stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(self.stream):
            out = self.grad_shard[self.shard_offsets[j]:self.shard_offsets[j + 1]]
            self.comm.reduce_scatter(self.grad_stage_buf[slot], 0, end - begin, 1.0 / self.world,
                                     out, self._next_slot(),
                                     accumulate_out=not self.first_microbatch)
            event = torch.cuda.Event()
            event.record(self.stream)
        self.stage_free[slot] = event

    # ------------------------------------------------------------------ training --
    def forward(self, input_ids):
        return self.model(input_ids)

    def loss(self, input_ids, targets, scale: float = 1.0):
        return self.model.loss(input_ids, targets, scale)

    def set_requires_gradient_sync(self, flag: bool) -> None:
        """Kept for interface parity; gradients are reduce-scattered after every
        microbatch and accumulated in the owned slice, which needs no full-size
        gradient buffer."""

    def zero_grad(self) -> None:
        for p in self.norm_params:
            p.grad = None
        self.first_microbatch = True

    def end_microbatch(self) -> None:
        self.first_microbatch = False

    @torch.no_grad()
    def clip_and_step(self, max_norm: float, *, lr: float, betas, eps: float,
                      weight_decay: float) -> torch.Tensor:
        current = torch.cuda.current_stream()
        current.wait_stream(self.stream)
        # Squared norm of the owned gradient slices (deterministic partial sums), times the
        # world size because the all-reduce below averages; then ONE peer all-reduce covers
        # the replicated norm-weight gradients and that scalar.
        local = K.grad_norm_and_coef(self.grad_shard, float("inf"))
        self.norm_grad_all[self.norm_numel] = local[0] * local[0] * self.world
        self.comm.allreduce(self.norm_grad_buf, 0, self.norm_grad_all.numel(), 1.0 / self.world,
                            self._next_slot())
        stats = K.grad_norm_and_coef(self.norm_grad, max_norm,
                                     extra_partials=self.norm_grad_all[self.norm_numel:
                                                                       self.norm_numel + 1])
        norm, coef, ok = stats[0], stats[1:2], stats[2:3]
        self.step_count += 1
        common = dict(step=self.step_count, lr=lr, beta1=betas[0], beta2=betas[1], eps=eps,
                      weight_decay=weight_decay, coef=coef, ok_flag=ok)
        K.adamw_step(self.shard.data, self.grad_shard, self.exp_avg, self.exp_avg_sq,
                     self.shadow_shard, **common)
        K.adamw_step(self.norm_flat, self.norm_grad, self.norm_exp_avg, self.norm_exp_avg_sq,
                     None, **common)
        self._gather_root()
        return norm

    def optimizer_state_bytes(self) -> int:
        tensors = (self.exp_avg, self.exp_avg_sq, self.norm_exp_avg, self.norm_exp_avg_sq)
        return sum(t.numel() * t.element_size() for t in tensors) + 4

    @torch.no_grad()
    def full_state_dict(self) -> dict[str, torch.Tensor]:
        """Every parameter as a full fp32 tensor (collective)."""
        engine = self.engine
        flat = torch.empty(engine.total, dtype=torch.float32, device=engine.device)
        for j, (begin, end) in enumerate(self.ranges):
            self._gather_range(j, flat[begin:end], self.master_buf, 4)
        state = {}
        for name, p in self.model.named_parameters():
            if p.dim() == 1:
                state[name] = p.detach().clone()
            else:
                begin = engine.offsets[id(p)]
                state[name] = flat[begin:begin + p.numel()].view(p.shape).clone()
        return state

    def close(self) -> None:
        torch.cuda.synchronize(self.engine.device)
        for buffer in (self.master_buf, self.shadow_buf, self.norm_grad_buf, *self.grad_stage_buf):
            buffer.close()
        self.comm.close()


class ShardedStepper:
    """Optimizer-shaped handle for the runner: learning-rate writes, ``zero_grad``
    and ``state_dict`` for the owned slices."""

    def __init__(self, sharded: FusedShardedTransformer, lr: float, betas, weight_decay: float,
                 eps: float = 1e-8):
        self.sharded = sharded
        self.param_groups = [{"params": list(sharded.parameters()), "lr": lr, "betas": betas,
                              "weight_decay": weight_decay, "eps": eps}]

    @property
    def state(self) -> dict:
        s = self.sharded
        return {"shard": {"exp_avg": s.exp_avg, "exp_avg_sq": s.exp_avg_sq},
                "norms": {"exp_avg": s.norm_exp_avg, "exp_avg_sq": s.norm_exp_avg_sq}}

    def zero_grad(self, set_to_none: bool = True) -> None:
        self.sharded.zero_grad()

    def clip_and_step(self, max_norm: float) -> torch.Tensor:
        group = self.param_groups[0]
        return self.sharded.clip_and_step(max_norm, lr=group["lr"], betas=group["betas"],
                                          eps=group["eps"], weight_decay=group["weight_decay"])

    def layout_sha256(self) -> str:
        """Identity of the sharding: the flat ranges, the slice of each that this world size
        gives a rank, and the replicated norm layout."""
        import hashlib
        import json
        s = self.sharded
        body = {"ranges": [list(r) for r in s.ranges], "chunks": list(s.chunks),
                "world_size": s.world, "norm_numel": int(s.norm_flat.numel())}
        return hashlib.sha256(json.dumps(body, sort_keys=True).encode()).hexdigest()

    def state_dict(self) -> dict:
        s = self.sharded
        return {"format_version": 1, "layout": "flat slices per range",
                "sharding": {"rank": s.rank, "world_size": s.world,
                             "layout_sha256": self.layout_sha256()},
                "rank": s.rank, "world_size": s.world, "step": s.step_count,
                "exp_avg": s.exp_avg, "exp_avg_sq": s.exp_avg_sq,
                "norm_exp_avg": s.norm_exp_avg, "norm_exp_avg_sq": s.norm_exp_avg_sq,
                "param_groups": [{k: v for k, v in group.items() if k != "params"}
                                 for group in self.param_groups]}

    def load_state_dict(self, state_dict: dict) -> None:
        """Restores this rank's moments and step count; refuses a shard written by another
        rank, for another world size or another parameter layout (the guard of the
        reference's sharded optimizer, distributed/llmdist/optim_shard.py:142-152)."""
        meta = state_dict.get("sharding", {})
        s = self.sharded
        if (state_dict.get("format_version") != 1 or meta.get("rank") != s.rank
                or meta.get("world_size") != s.world
                or meta.get("layout_sha256") != self.layout_sha256()):
            raise ValueError(
                "Optimizer shard does not match this rank, world size or parameter layout")
        for name in ("exp_avg", "exp_avg_sq", "norm_exp_avg", "norm_exp_avg_sq"):
            target = getattr(s, name)
            source = state_dict[name]
            if tuple(source.shape) != tuple(target.shape):
                raise ValueError(f"optimizer shard tensor {name} has the wrong shape")
            target.copy_(source)
        s.step_count = int(state_dict["step"])
        for group, saved in zip(self.param_groups, state_dict.get("param_groups", [])):
            group.update({k: v for k, v in saved.items() if k != "params"})
