"""AdamW with optimizer state sharded across data-parallel ranks (ZeRO stage 1).

Parameters and gradients stay replicated; every optimizer-state element has one
owner.  Two layouts behind one class:

* **whole-parameter ownership** (any device, gloo or NCCL) - the reference's
  scheme (distributed/llmdist/optim_shard.py:27-152): parameters are assigned to
  ranks greedily, largest first; each rank runs a real ``torch.optim.AdamW`` on
  the parameters it owns and the owners broadcast the results.  Same public
  surface: ``param_groups``, ``state``, ``zero_grad``, ``step``,
  ``local_state_bytes``, ``ownership_metadata``, ``state_dict`` /
  ``load_state_dict`` with rank / world / layout guards.
* **flat-slice ownership** (B200, fused model wrapped in ``BucketedDDP(mode=
  "scatter")``) - rank r owns slice r of every gradient bucket.  ``step`` is one
  kernel: AdamW on the owned fp32 master / moment slices using the gradient
  slices that the reduce-scatter left behind, then the updated fp32 parameters
  and bf16 shadow are stored straight into every peer's memory.  This replaces
  the all-reduce + local AdamW + 219 broadcasts of the reference with
  reduce-scatter -> fused update -> all-gather.
"""

from __future__ import annotations

import hashlib
import json
from collections.abc import Iterable

import torch
import torch.distributed as dist


def _tensor_bytes(value) -> int:
    if isinstance(value, torch.Tensor):
        return value.numel() * value.element_size()
    if isinstance(value, dict):
        return sum(_tensor_bytes(item) for item in value.values())
    if isinstance(value, (list, tuple)):
        return sum(_tensor_bytes(item) for item in value)
    return 0


def assign_owners(sizes: list[int], world_size: int) -> tuple[list[int], list[int]]:
    """Greedy longest-processing-time assignment: biggest tensor to the lightest rank,
    ties broken by lower parameter index, then lower rank.  Returns (owners, load)."""
    load = [0] * world_size
    owners = [0] * len(sizes)
    for index in sorted(range(len(sizes)), key=lambda i: (-sizes[i], i)):
        rank = min(range(world_size), key=lambda r: (load[r], r))
        owners[index] = rank
        load[rank] += sizes[index]
    return owners, load


class ShardedAdamW:
    def __init__(self, params: Iterable, lr: float = 1e-3, betas=(0.9, 0.95),
                 weight_decay: float = 0.1, process_group=None, **kwargs):
        supplied = list(params)
        if not supplied:
            raise ValueError("ShardedAdamW requires at least one parameter")
        if isinstance(supplied[0], dict):
            if not all(isinstance(group, dict) for group in supplied):
                raise TypeError("Do not mix parameters and parameter groups")
            groups = [dict(group, params=list(group["params"])) for group in supplied]
        else:
            groups = [{"params": supplied}]
        self._parameters = [p for group in groups for p in group["params"]]
        if not self._parameters:
            raise ValueError("ShardedAdamW requires at least one parameter")
        if any(not isinstance(p, torch.Tensor) for p in self._parameters):
            raise TypeError("Optimizer parameters must be tensors")
        if len({id(p) for p in self._parameters}) != len(self._parameters):
            raise ValueError("Duplicate parameters cannot have separate optimizer owners")
        if process_group is not None and not dist.is_initialized():
            raise ValueError("A process group requires initialized distributed training")
        self.process_group = process_group
        initialized = dist.is_initialized()
        self.rank = dist.get_rank(process_group) if initialized else 0
        self.world_size = dist.get_world_size(process_group) if initialized else 1
        self._owners, self._owner_numel = assign_owners(
            [p.numel() for p in self._parameters], self.world_size)
        defaults = {"lr": lr, "betas": betas, "weight_decay": weight_decay, **kwargs}
        descriptor = {
            "parameters": [{"shape": list(p.shape), "dtype": str(p.dtype),
                            "requires_grad": p.requires_grad} for p in self._parameters],
            "group_sizes": [len(group["params"]) for group in groups],
            "group_options": [{k: v for k, v in group.items() if k != "params"}
                              for group in groups],
            "defaults": defaults, "owners": self._owners,
        }
        self._layout_hash = hashlib.sha256(
            json.dumps(descriptor, sort_keys=True, default=str).encode()).hexdigest()
        if self.world_size > 1:
            hashes = [None] * self.world_size
            dist.all_gather_object(hashes, self._layout_hash, group=process_group)
            if len(set(hashes)) != 1:
                raise ValueError("Optimizer parameter layout or settings differ across ranks")
        cursor = 0
        local_groups = []
        for group in groups:
            mine = dict(group, params=[])
            for p in group["params"]:
                if self._owners[cursor] == self.rank:
                    mine["params"].append(p)
                cursor += 1
            local_groups.append(mine)
        # Groups may be empty: a rank that owns nothing still takes learning-rate writes.
        self._optimizer = torch.optim.AdamW(local_groups, **defaults)
        self._flat = None   # flat-slice state, see attach_flat()

    # -------------------------------------------------------- common surface --
    @property
    def param_groups(self):
        return self._optimizer.param_groups

    @property
    def state(self):
        return self._optimizer.state

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self._parameters:
            if p.grad is None:
                continue
            if set_to_none:
                p.grad = None
            else:
                # Gradients may be views into a communication buffer: keep the alias.
                if p.grad.grad_fn is not None:
                    p.grad = p.grad.detach()
                with torch.no_grad():
                    p.grad.zero_()

    def step(self, closure=None):
        if self._flat is not None:
            raise RuntimeError("flat-slice mode updates through step_flat()")
        loss = self._optimizer.step(closure)
        if self.world_size > 1:
            with torch.no_grad():
                for p, owner in zip(self._parameters, self._owners, strict=True):
                    source = (owner if self.process_group is None
                              else dist.get_global_rank(self.process_group, owner))
                    dist.broadcast(p, src=source, group=self.process_group)
        return loss

    def local_state_bytes(self) -> int:
        """Bytes of optimizer state held by this rank (moments and step counters)."""
        if self._flat is not None:
            return _tensor_bytes([self._flat["exp_avg"], self._flat["exp_avg_sq"]]) + 4
        return _tensor_bytes(self._optimizer.state)

    def ownership_metadata(self) -> dict:
        flat = self._flat is not None
        return {
            "algorithm": ("flat slices of gradient buckets; fused update and all-gather" if flat
                          else "greedy whole-parameter optimizer-state sharding"),
            "rank": self.rank, "world_size": self.world_size,
            "owners": list(self._owners), "parameter_numel_per_rank": list(self._owner_numel),
            "owned_parameter_indices": [i for i, o in enumerate(self._owners) if o == self.rank],
            "layout_sha256": self._layout_hash,
            "local_optimizer_state_bytes": self.local_state_bytes(),
            "parameter_scope": "replicated",
            "gradient_scope": ("reduce-scattered into owner slices" if flat
                               else "replicated; caller synchronizes"),
            "state_scope": "AdamW moments and step counters exist only on the owning rank",
            "communication": ("parameters stored into peer memory by the update kernel" if flat
                              else "synchronous parameter broadcasts after the optimizer step"),
        }

    def state_dict(self) -> dict:
        payload = {"format_version": 1, "sharding": self.ownership_metadata()}
        if self._flat is not None:
            payload["optimizer"] = {"flat": True, "step": self._flat["step"],
                                    "exp_avg": self._flat["exp_avg"],
                                    "exp_avg_sq": self._flat["exp_avg_sq"],
                                    "param_groups": [{k: v for k, v in g.items() if k != "params"}
                                                     for g in self.param_groups]}
        else:
            payload["optimizer"] = self._optimizer.state_dict()
        return payload

    def load_state_dict(self, state_dict: dict) -> None:
        meta = state_dict["sharding"]
        if (state_dict.get("format_version") != 1 or meta["rank"] != self.rank
                or meta["world_size"] != self.world_size
                or meta["layout_sha256"] != self._layout_hash):
            raise ValueError(
                "Optimizer shard does not match this rank, world size or parameter layout")
        inner = state_dict["optimizer"]
        if inner.get("flat"):
            if self._flat is None:
                raise ValueError("flat optimizer shard needs attach_flat() first")
            self._flat["exp_avg"].copy_(inner["exp_avg"])
            self._flat["exp_avg_sq"].copy_(inner["exp_avg_sq"])
            self._flat["step"] = int(inner["step"])
        else:
            self._optimizer.load_state_dict(inner)

    # ------------------------------------------------------ flat-slice mode --
    def attach_flat(self, ddp, engine) -> None:
        """Switch to flat-slice ownership on top of ``BucketedDDP(mode="scatter")``.

        Parameters and the bf16 shadow move into symmetric memory so owners can
        store updated values directly into their peers' copies.
        """
        from . import comm as pm
        state = ddp._peer
        if state is None or ddp.mode != "scatter":
            raise ValueError("flat mode needs a BucketedDDP in scatter mode with peer memory")
        if len(self.param_groups) != 1:
            raise ValueError("flat mode supports a single parameter group")
        device = engine.device
        total = engine.total
        params = pm.SymmetricBuffer(total * 4, device, ddp.group)
        shadows = pm.SymmetricBuffer(total * 2, device, ddp.group)
        engine.relocate(flat_param=params.view(torch.float32, total))
        old_shadow = engine.flat_shadow
        engine.flat_shadow = shadows.view(torch.bfloat16, total)
        engine.flat_shadow.copy_(old_shadow)
        engine._versions = None
        shard = state["shard"]
        self._flat = {"ddp": ddp, "engine": engine, "params": params, "shadows": shadows,
                      "exp_avg": torch.zeros_like(shard), "exp_avg_sq": torch.zeros_like(shard),
                      "step": 0}

    @torch.no_grad()
    def step_flat(self, stats: torch.Tensor) -> None:
        """``stats`` is the ``[norm, coef, finite]`` vector returned by ``ddp.finish``."""
        flat = self._flat
        ddp, engine = flat["ddp"], flat["engine"]
        state = ddp._peer
        comm = state["comm"]
        group = self.param_groups[0]
        flat["step"] += 1
        beta1, beta2 = group["betas"]
        engine.sync_shadow()
        ranges = state["ranges"]
        # Every bucket range in one launch; the table keeps each range's slice
        # aligned with what the reduce-scatter left in the shard buffer.
        table = flat.get("range_table")
        if table is None:
            rows = [(begin, end - begin, state["shard_offsets"][index])
                    for index, (begin, end) in enumerate(ranges)]
            if any(value % 4 for row in rows for value in row):
                raise ValueError("bucket ranges must be multiples of four elements")
            table = torch.tensor(rows, dtype=torch.int64, device=state["shard"].device)
            flat["range_table"] = table
        comm.adamw_allgather_ranges(
            flat["params"], flat["shadows"], table, state["shard"], flat["exp_avg"],
            flat["exp_avg_sq"], step=flat["step"], lr=group["lr"], beta1=beta1, beta2=beta2,
            eps=group.get("eps", 1e-8), weight_decay=group["weight_decay"], coef=stats[1:2],
            ok=stats[2:3], slot=comm.slots - 1)
        engine.mark_shadow_current()

    def close(self) -> None:
        if self._flat is not None:
            self._flat["params"].close()
            self._flat["shadows"].close()
            self._flat = None
