"""AdamW over flat buffers with the clip folded in.

``FusedAdamW`` presents the ``torch.optim.AdamW`` interface (``param_groups``,
``state``, ``state_dict`` / ``load_state_dict`` with the same keys and layout) so
checkpoints stay interchangeable with the reference (src/llmlab/train.py:169-170,
265-275), but on a B200 with a fused model it performs the whole update - gradient
clipping coefficient, AdamW on fp32 master weights and moments, and the bf16
shadow refresh - as one pass over HBM instead of the reference's clip + foreach
sequence.  Everywhere else it falls back to ``torch.optim.AdamW`` math on the
same state tensors.

``clip_and_step(max_norm)`` is the fused entry point: it returns the global
gradient norm as a device scalar without a host synchronisation.
"""

from __future__ import annotations

import torch

from .ops import functional as K
from .ops import lib as _lib


class FusedAdamW(torch.optim.AdamW):
    def __init__(self, params, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=1e-2,
                 engine=None):
        super().__init__(params, lr=lr, betas=betas, eps=eps, weight_decay=weight_decay,
                         foreach=False, fused=False)
        self.engine = engine
        self._flat_state = None
        self._step_count = 0

    # -------------------------------------------------------------- fused path --
    def _fused_ready(self) -> bool:
        engine = self.engine
        if engine is None or not _lib.available() or engine.flat_grad is None:
            return False
        if len(self.param_groups) != 1:
            return False
        params = self.param_groups[0]["params"]
        if len(params) != len(engine.params) or {id(p) for p in params} != set(engine.offsets):
            return False
        # Every gradient must already live in the flat buffer.
        for p in engine.params:
            if p.grad is None or p.grad.data_ptr() != engine.grad_view(p).data_ptr():
                return False
        return True

    def _ensure_flat_state(self) -> None:
        if self._flat_state is not None:
            return
        engine = self.engine
        exp_avg = torch.zeros_like(engine.flat_param)
        exp_avg_sq = torch.zeros_like(engine.flat_param)
        steps = torch.zeros(len(engine.params), dtype=torch.float32, device="cpu")
        for i, p in enumerate(engine.params):
            existing = self.state.get(p, {})
            m, v = engine._slice(exp_avg, p), engine._slice(exp_avg_sq, p)
            if "exp_avg" in existing:
                m.copy_(existing["exp_avg"])
                v.copy_(existing["exp_avg_sq"])
                steps[i] = float(existing["step"])
            # 0-d CPU step counters, as torch.optim.AdamW keeps them.
            self.state[p] = {"step": steps[i], "exp_avg": m, "exp_avg_sq": v}
        self._flat_state = (exp_avg, exp_avg_sq, steps)
        self._step_count = int(steps.max().item()) if len(steps) else 0

    @torch.no_grad()
    def clip_and_step(self, max_norm: float, error_if_nonfinite: bool = True) -> torch.Tensor:
        """Clip by global norm and update.  Returns the pre-clip norm (device scalar).

        On the fused path a non-finite norm skips the update on the device and the
        caller finds out when it reads the returned norm; the portable path raises
        like ``clip_grad_norm_(error_if_nonfinite=True)``.
        """
        if not self._fused_ready():
            params = [p for g in self.param_groups for p in g["params"]]
            norm = torch.nn.utils.clip_grad_norm_(params, max_norm,
                                                  error_if_nonfinite=error_if_nonfinite)
            self.step()
            return norm
        engine = self.engine
        self._ensure_flat_state()
        exp_avg, exp_avg_sq, steps = self._flat_state
        group = self.param_groups[0]
        stats = K.grad_norm_and_coef(engine.flat_grad[:engine.total], max_norm)
        self._step_count = int(steps[0].item()) + 1
        steps += 1
        beta1, beta2 = group["betas"]
        K.adamw_step(engine.flat_param, engine.flat_grad, exp_avg, exp_avg_sq, engine.flat_shadow,
                     step=self._step_count, lr=group["lr"], beta1=beta1, beta2=beta2,
                     eps=group["eps"], weight_decay=group["weight_decay"], coef=stats[1:2],
                     ok_flag=stats[2:3])
        engine.mark_shadow_current()
        return stats[0]

    @torch.no_grad()
    def step_with_stats(self, stats: torch.Tensor) -> torch.Tensor:
        """Update with a clip coefficient that is already on the device.

        ``stats`` is ``[norm, coefficient, finite flag]`` as produced by the fused
        gradient reduction (``BucketedDDP.finish``); returns the norm.
        """
        if not self._fused_ready():
            raise RuntimeError("step_with_stats needs gradients in the engine's flat buffer")
        engine = self.engine
        self._ensure_flat_state()
        exp_avg, exp_avg_sq, steps = self._flat_state
        group = self.param_groups[0]
        self._step_count = int(steps[0].item()) + 1
        steps += 1
        beta1, beta2 = group["betas"]
        K.adamw_step(engine.flat_param, engine.flat_grad, exp_avg, exp_avg_sq, engine.flat_shadow,
                     step=self._step_count, lr=group["lr"], beta1=beta1, beta2=beta2,
                     eps=group["eps"], weight_decay=group["weight_decay"], coef=stats[1:2],
                     ok_flag=stats[2:3])
        engine.mark_shadow_current()
        return stats[0]

    @torch.no_grad()
    def step(self, closure=None):
        if self._flat_state is not None and self._fused_ready():
            # Gradients were clipped (or not) by the caller; plain update.
            engine = self.engine
            exp_avg, exp_avg_sq, steps = self._flat_state
            group = self.param_groups[0]
            self._step_count = int(steps[0].item()) + 1
            steps += 1
            beta1, beta2 = group["betas"]
            K.adamw_step(engine.flat_param, engine.flat_grad, exp_avg, exp_avg_sq,
                         engine.flat_shadow, step=self._step_count, lr=group["lr"], beta1=beta1,
                         beta2=beta2, eps=group["eps"], weight_decay=group["weight_decay"])
            engine.mark_shadow_current()
            return None
        return super().step(closure)

    def load_state_dict(self, state_dict) -> None:
        super().load_state_dict(state_dict)
        # Loaded tensors are fresh copies; re-home them in the flat buffers lazily.
        self._flat_state = None
