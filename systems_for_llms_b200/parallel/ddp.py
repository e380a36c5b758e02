"""Data-parallel gradient reduction: bucketed, overlapped with backward.

``BucketedDDP`` plays the role the reference gives to
``torch.nn.parallel.DistributedDataParallel`` (distributed/llmdist/train.py:263-265,
142-143): replicated parameters, gradients averaged over ranks in buckets of
``bucket_cap_mb`` as backward produces them, ``no_sync()`` to skip the reduction
on all but the last microbatch.  Two data paths share that interface:

* **peer-memory path** (B200, fused model): the model's flat gradient buffer is
  placed in symmetric memory; as each block's backward finishes, the buckets that
  became final are reduced on a side stream by the ``allreduce_f32`` kernel
  (reduce-scatter + all-gather over NVLink in one launch, with the 1/world
  scale and the gradient-norm partials fused in).  In ``mode="scatter"`` the
  owner keeps its reduced slice and no write-back happens (sharded optimizer).
* **collective path** (anything else, including gloo on CPU): per-parameter
  hooks fill flat bucket tensors and launch asynchronous
  ``torch.distributed.all_reduce`` calls.

``finish()`` must be called after the last backward of a step; it joins the
reductions and, on the peer-memory path, returns the device vector
``[grad norm, clip coefficient, finite flag]``.
"""

from __future__ import annotations

from contextlib import contextmanager

import torch
import torch.distributed as dist
from torch import nn

from . import comm as pm


class BucketedDDP(nn.Module):
    def __init__(self, module: nn.Module, bucket_cap_mb: float = 25.0, process_group=None,
                 mode: str = "allreduce", comm_ctas: int = 32):
        super().__init__()
        if mode not in ("allreduce", "scatter"):
            raise ValueError("mode must be 'allreduce' or 'scatter'")
        if bucket_cap_mb <= 0:
            raise ValueError("bucket_cap_mb must be positive")
        self.module = module
        self.group = process_group
        self.mode = mode
        self.world = dist.get_world_size(process_group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(process_group) if dist.is_initialized() else 0
        self.bucket_bytes = int(bucket_cap_mb * 1024 * 1024)
        self.comm_ctas = comm_ctas
        self._sync = True
        self._peer = None          # peer-memory state, built lazily
        self._buckets = None       # collective-path buckets
        self._hooks = []
        self._pending = []
        self._install_hooks()

    # ----------------------------------------------------------- delegation --
    def forward(self, *args, **kwargs):
        self._begin_microbatch()
        return self.module(*args, **kwargs)

    def loss(self, *args, **kwargs):
        self._begin_microbatch()
        return self.module.loss(*args, **kwargs)

    def _begin_microbatch(self) -> None:
        """With a reduction after every microbatch, the previous one must have landed
        in ``.grad`` before this microbatch's backward accumulates on top of it."""
        if self.world == 1:
            return
        if self._peer_active():
            state = self._peer
            if state["next"] > 0:
                torch.cuda.current_stream().wait_stream(state["stream"])
                state["next"] = 0
                state["used_slots"] = set()
        elif any(bucket["launched"] for bucket in self._buckets):
            self._finish_collective()

    @contextmanager
    def no_sync(self):
        previous, self._sync = self._sync, False
        try:
            yield
        finally:
            self._sync = previous

    # ----------------------------------------------------- collective path --
    def _install_hooks(self) -> None:
        params = [p for p in self.module.parameters() if p.requires_grad]
        buckets, current, size = [], [], 0
        for p in reversed(params):       # backward produces gradients roughly in this order
            nbytes = p.numel() * p.element_size()
            if current and size + nbytes > self.bucket_bytes:
                buckets.append(current)
                current, size = [], 0
            current.append(p)
            size += nbytes
        if current:
            buckets.append(current)
        self._buckets = [{"params": group, "ready": 0, "flat": None, "work": None,
                          "launched": False} for group in buckets]
        index = {id(p): b for b, group in enumerate(buckets) for p in group}
        for p in params:
            self._hooks.append(p.register_post_accumulate_grad_hook(
                lambda param, b=index[id(p)]: self._on_grad(b)))

    def _on_grad(self, bucket_index: int) -> None:
        if not self._sync or self.world == 1 or self._peer_active():
            return
        bucket = self._buckets[bucket_index]
        bucket["ready"] += 1
        if bucket["ready"] == len(bucket["params"]):
            self._launch(bucket)

    def _launch(self, bucket) -> None:
        params = bucket["params"]
        grads = [p.grad if p.grad is not None else torch.zeros_like(p) for p in params]
        flat = torch.cat([g.reshape(-1) for g in grads])
        bucket["flat"] = flat
        bucket["work"] = dist.all_reduce(flat, group=self.group, async_op=True)
        bucket["launched"] = True

    def _finish_collective(self) -> None:
        for bucket in self._buckets:
            if not bucket["launched"]:
                self._launch(bucket)       # parameters that received no gradient this step
        for bucket in self._buckets:
            bucket["work"].wait()
            flat = bucket["flat"].div_(self.world)
            cursor = 0
            for p in bucket["params"]:
                piece = flat[cursor:cursor + p.numel()].view_as(p)
                if p.grad is None:
                    p.grad = piece.clone()
                else:
                    p.grad.copy_(piece)
                cursor += p.numel()
            bucket.update(ready=0, flat=None, work=None, launched=False)

    # ----------------------------------------------------- peer-memory path --
    def _peer_active(self) -> bool:
        return self._peer is not None

    def enable_peer_memory(self, engine) -> None:
        """Move the fused engine's gradients into symmetric memory and cut buckets."""
        if self._peer is not None or self.world == 1:
            return
        device = engine.device
        comm = pm.PeerComm(device, self.group, ctas=self.comm_ctas)
        total = engine.total
        grads = pm.SymmetricBuffer(total * 4, device, self.group)
        engine.relocate(flat_grad=grads.view(torch.float32, total))
        align = 4 * self.world * 64
        bucket_elems = max(align, (self.bucket_bytes // 4) // align * align)
        ranges = []
        end = total
        while end > 0:                    # cut from the end: backward finishes the tail first
            begin = max(0, end - bucket_elems)
            ranges.append((begin, end))
            end = begin
        slots = comm.slots - 8            # the last slots are kept for other collectives
        self._peer = {
            "engine": engine, "comm": comm, "grads": grads, "ranges": ranges, "next": 0,
            "stream": torch.cuda.Stream(device=device), "slot_count": slots,
            "slot_ids": torch.arange(min(slots, len(ranges)), dtype=torch.int32, device=device),
            "used_slots": set(), "bucket_elems": bucket_elems,
        }
        if self.mode == "scatter":
            per_rank = sum(self._slice_len(b, e) for b, e in ranges)
            self._peer["shard"] = torch.zeros(per_rank, dtype=torch.float32, device=device)
            offsets, cursor = [], 0
            for b, e in ranges:
                offsets.append(cursor)
                cursor += self._slice_len(b, e)
            self._peer["shard_offsets"] = offsets
        engine.on_block_backward = self._on_progress

    def _slice_len(self, begin: int, end: int) -> int:
        vecs = (end - begin) // 4
        per = -(-vecs // self.world)
        return per * 4

    def _on_progress(self, ready_from: int) -> None:
        """Called by the engine during backward: every gradient at flat offset
        ``ready_from`` or beyond is final."""
        if self._sync:
            self._reduce_ready(ready_from)

    def _reduce_ready(self, ready_from: int) -> None:
        state = self._peer
        comm, grads = state["comm"], state["grads"]
        launch = []
        while state["next"] < len(state["ranges"]) and state["ranges"][state["next"]][0] >= ready_from:
            launch.append(state["next"])
            state["next"] += 1
        if not launch:
            return
        stream = state["stream"]
        stream.wait_stream(torch.cuda.current_stream())
        scale = 1.0 / self.world
        # Buckets that only become final with the last gradient of the backward pass have
        # nothing left to hide behind: they take the whole GPU instead of the few CTAs that
        # reductions overlapped with backward are limited to.  A bucket index always gets
        # the same treatment, so each slot keeps one grid size.
        tail = ready_from == 0 and len(state["ranges"]) <= state["slot_count"]
        ctas = comm.update_ctas if tail else None
        with torch.cuda.stream(stream):
            for index in launch:
                begin, end = state["ranges"][index]
                slot = index % state["slot_count"]
                accumulate = slot in state["used_slots"]
                state["used_slots"].add(slot)
                if self.mode == "scatter":
                    offset = state["shard_offsets"][index]
                    out = state["shard"][offset:offset + self._slice_len(begin, end)]
                    comm.reduce_scatter(grads, begin, end - begin, scale, out, slot, accumulate,
                                        ctas=ctas)
                else:
                    comm.allreduce(grads, begin, end - begin, scale, slot, accumulate, ctas=ctas)

    def _finish_peer(self, max_norm: float) -> torch.Tensor:
        state = self._peer
        self._reduce_ready(0)             # anything the callbacks did not cover
        torch.cuda.current_stream().wait_stream(state["stream"])
        stats = state["comm"].norm_finalize(state["grads"], state["slot_ids"], max_norm)
        state["next"] = 0
        state["used_slots"] = set()
        return stats

    # ---------------------------------------------------------------- finish --
    def finish(self, max_norm: float = float("inf")):
        """Join this step's reductions.  Peer-memory path: returns the device vector
        ``[norm, clip coefficient, finite]`` of the averaged gradient; collective
        path: returns ``None`` (gradients are averaged in ``.grad``)."""
        if self.world == 1:
            return None
        if self._peer_active():
            return self._finish_peer(max_norm)
        self._finish_collective()
        return None

    def close(self) -> None:
        for hook in self._hooks:
            hook.remove()
        self._hooks = []
        if self._peer is not None:
            self._peer["engine"].on_block_backward = None
            self._peer["comm"].close()
            self._peer["grads"].close()
            self._peer = None
