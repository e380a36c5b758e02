"""Fully sharded data parallelism (ZeRO stage 3) per transformer block.

The reference shards with PyTorch's ``fully_shard`` (FSDP2): one group per block
plus a root group for embeddings, final norm and head, fp32 shards, reshard after
forward, gradient reduce-scatter in backward, ``set_requires_gradient_sync`` for
accumulation (distributed/llmdist/train.py:258-262, 144-145).  This module is an
independent implementation of the same scheme:

* ``ShardedModule`` owns one flat fp32 ``shard`` parameter (1/world of the
  wrapped module's parameters).  Forward all-gathers the flat buffer, lends views
  of it to the wrapped module for the duration of the call, and lets go of it;
  tensors that autograd would save from the gathered buffer are replaced by
  markers and re-gathered when backward reaches the group (saved-tensor hooks),
  which gives reshard-after-forward without recomputation.  Backward
  reduce-scatters the flat gradient (averaged) into ``shard.grad``.
* ``shard_model`` wraps every block and the root modules of a ``TransformerLM``.
* ``clip_grad_norm_sharded`` computes the global norm from disjoint shards.

Works on any backend (gloo included: reduce-scatter falls back to all-reduce +
slice there), so the 2-rank CPU parity tests cover it - the reference cannot run
FSDP on CPU at all.
"""

from __future__ import annotations

import torch
import torch.distributed as dist
from torch import nn


def _backend_supports_reduce_scatter(group) -> bool:
    try:
        return dist.get_backend(group) != "gloo"
    except Exception:
        return False


class _Gather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, shard, owner):
        ctx.owner = owner
        return owner._all_gather(shard.detach())

    @staticmethod
    def backward(ctx, grad_full):
        owner = ctx.owner
        owner._regathered = None          # backward of this group is complete
        grad_full = grad_full.contiguous()
        if not owner.requires_gradient_sync:
            if owner._pending is None:
                owner._pending = grad_full.clone()
            else:
                owner._pending += grad_full
            return None, None
        if owner._pending is not None:
            grad_full = grad_full + owner._pending
            owner._pending = None
        return owner._reduce_scatter(grad_full), None


class ShardedModule(nn.Module):
    """Wraps ``modules`` (one or several) whose parameters become one flat shard."""

    def __init__(self, inner: nn.Module | None, managed: list[nn.Module], group=None):
        super().__init__()
        self.inner = inner
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.requires_gradient_sync = True
        self._pending = None
        self._regathered = None
        self._slots = []        # (module, name, shape, offset, numel)
        self.param_names = []   # qualified names for state reconstruction
        pieces, cursor = [], 0
        for prefix, module in managed:
            for name, p in list(module.named_parameters(recurse=True)):
                holder, leaf = module, name
                while "." in leaf:
                    head, leaf = leaf.split(".", 1)
                    holder = getattr(holder, head)
                if isinstance(holder, ShardedModule) or leaf == "shard":
                    continue
                self._slots.append((holder, leaf, tuple(p.shape), cursor, p.numel()))
                self.param_names.append(f"{prefix}{name}")
                pieces.append(p.detach().reshape(-1))
                cursor += p.numel()
        self.numel = cursor
        self.padded = -(-cursor // self.world) * self.world
        flat = torch.cat(pieces) if pieces else torch.zeros(0)
        if self.padded != cursor:
            flat = torch.cat([flat, flat.new_zeros(self.padded - cursor)])
        per = self.padded // self.world
        self.shard = nn.Parameter(flat[self.rank * per:(self.rank + 1) * per].clone())
        for holder, leaf, *_ in self._slots:
            holder._parameters[leaf] = None     # the full tensors no longer live here

    # ----------------------------------------------------------- collectives --
    def _all_gather(self, shard: torch.Tensor) -> torch.Tensor:
        if self.world == 1:
            return shard.clone()
        full = torch.empty(self.padded, dtype=shard.dtype, device=shard.device)
        dist.all_gather_into_tensor(full, shard.contiguous(), group=self.group)
        return full

    def _reduce_scatter(self, grad_full: torch.Tensor) -> torch.Tensor:
        per = self.padded // self.world
        if self.world == 1:
            return grad_full[:per].clone()
        if _backend_supports_reduce_scatter(self.group):
            out = torch.empty(per, dtype=grad_full.dtype, device=grad_full.device)
            dist.reduce_scatter_tensor(out, grad_full, group=self.group)
        else:
            dist.all_reduce(grad_full, group=self.group)
            out = grad_full[self.rank * per:(self.rank + 1) * per].clone()
        return out.div_(self.world)

    # ---------------------------------------------------------------- lending --
    def _lend(self, full: torch.Tensor) -> None:
        for holder, leaf, shape, offset, numel in self._slots:
            holder._parameters[leaf] = full[offset:offset + numel].view(shape)

    def _reclaim(self) -> None:
        for holder, leaf, *_ in self._slots:
            holder._parameters[leaf] = None

    def _pack(self, full: torch.Tensor):
        base = full.untyped_storage().data_ptr()

        def pack(tensor):
            if (isinstance(tensor, torch.Tensor) and tensor.device == full.device
                    and tensor.numel() > 0 and tensor.untyped_storage().data_ptr() == base):
                return ("sharded", tensor.storage_offset(), tuple(tensor.shape),
                        tuple(tensor.stride()), tensor.dtype)
            return tensor

        def unpack(item):
            if isinstance(item, tuple) and item and item[0] == "sharded":
                if self._regathered is None:
                    with torch.no_grad():
                        self._regathered = self._all_gather(self.shard.detach())
                _, offset, shape, stride, dtype = item
                return torch.as_strided(self._regathered, shape, stride, offset)
            return item

        return torch.autograd.graph.saved_tensors_hooks(pack, unpack)

    def gathered(self):
        """Context manager: parameters of the managed modules are usable inside."""
        return _Lend(self)

    def forward(self, *args, **kwargs):
        with self.gathered():
            return self.inner(*args, **kwargs)

    def full_parameters(self) -> dict[str, torch.Tensor]:
        """Name -> full tensor, gathered now (collective)."""
        with torch.no_grad():
            full = self._all_gather(self.shard.detach())
        return {name: full[offset:offset + numel].view(shape).clone()
                for name, (_, _, shape, offset, numel) in zip(self.param_names, self._slots)}


class _Lend:
    def __init__(self, owner: ShardedModule):
        self.owner = owner
        self.hooks = None

    def __enter__(self):
        owner = self.owner
        if torch.is_grad_enabled():
            full = _Gather.apply(owner.shard, owner)
            self.hooks = owner._pack(full)
            self.hooks.__enter__()
        else:
            full = owner._all_gather(owner.shard.detach())
        owner._lend(full)
        return owner

    def __exit__(self, *exc):
        if self.hooks is not None:
            self.hooks.__exit__(*exc)
        self.owner._reclaim()
        return False


class ShardedTransformer(nn.Module):
    """``TransformerLM`` with every block and the root modules sharded."""

    def __init__(self, model, group=None):
        super().__init__()
        self.model = model
        for index, block in enumerate(model.layers):
            model.layers[index] = ShardedModule(block, [(f"layers.{index}.", block)], group)
        self.root = ShardedModule(None, [("token_embeddings.", model.token_embeddings),
                                         ("ln_final.", model.ln_final),
                                         ("lm_head.", model.lm_head)], group)
        model._fused_disabled = True

    def groups(self) -> list[ShardedModule]:
        return [*self.model.layers, self.root]

    def set_requires_gradient_sync(self, flag: bool) -> None:
        for group in self.groups():
            group.requires_gradient_sync = bool(flag)

    def forward(self, input_ids):
        with self.root.gathered():
            return self.model(input_ids)

    def loss(self, input_ids, targets, scale: float = 1.0):
        with self.root.gathered():
            return self.model.loss(input_ids, targets, scale)

    def full_state_dict(self) -> dict[str, torch.Tensor]:
        state = {}
        for group in self.groups():
            state.update(group.full_parameters())
        return state

    def train(self, mode: bool = True):
        super().train(mode)
        return self


def shard_model(model, group=None) -> ShardedTransformer:
    return ShardedTransformer(model, group)


@torch.no_grad()
def clip_grad_norm_sharded(parameters, max_norm: float, group=None) -> torch.Tensor:
    """Global L2 norm over disjoint shards, then scale every local shard gradient."""
    parameters = [p for p in parameters if p.grad is not None]
    if not parameters:
        raise RuntimeError("sharded model has no gradients to clip")
    total = torch.zeros((), device=parameters[0].device, dtype=torch.float32)
    for p in parameters:
        total += torch.linalg.vector_norm(p.grad, 2, dtype=torch.float32).square()
    if dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(total, group=group)
    norm = total.sqrt()
    if not torch.isfinite(norm):
        raise FloatingPointError("Non-finite global gradient norm")
    coefficient = (max_norm / (norm + 1e-6)).clamp(max=1.0)
    for p in parameters:
        p.grad.mul_(coefficient.to(p.grad.dtype))
    return norm
