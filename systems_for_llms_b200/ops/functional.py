"""Tensor-level wrappers of the bandwidth-bound sm_100a kernels (csrc/elementwise.cu).

Each function validates its arguments, allocates outputs with PyTorch and
launches on the current stream.  They are building blocks for the autograd
nodes in models/fused.py and for the fused optimizers; they are not themselves
differentiable.
"""

from __future__ import annotations

import torch

from . import lib as _lib


def _f32(t: torch.Tensor, name: str) -> None:
    if t.dtype != torch.float32 or not t.is_contiguous() or not t.is_cuda:
        raise ValueError(f"{name} must be a contiguous fp32 CUDA tensor")


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float):
    """``x`` fp32 ``[rows, dim]`` -> (bf16 normalised rows, fp32 1/rms per row)."""
    _f32(x, "x")
    rows, dim = x.shape
    y = torch.empty(rows, dim, dtype=torch.bfloat16, device=x.device)
    rstd = torch.empty(rows, dtype=torch.float32, device=x.device)
    code = _lib.lib().sfl_rmsnorm_fwd(x.data_ptr(), weight.data_ptr(), y.data_ptr(),
                                     rstd.data_ptr(), rows, dim, float(eps), _lib.stream_ptr())
    _lib.check(code, "sfl_rmsnorm_fwd")
    return y, rstd


def rmsnorm_bwd(dy: torch.Tensor, x: torch.Tensor, weight: torch.Tensor, rstd: torch.Tensor,
                dres: torch.Tensor | None, dweight: torch.Tensor, accumulate: bool,
                want_bf16: bool = False):
    """Gradient of ``rmsnorm`` fused with the residual-stream add.

    Returns ``(dx, dx_bf16 or None)`` with ``dx = dres + d(norm)/dx``; the weight
    gradient is reduced over rows in a fixed order into ``dweight``.
    """
    rows, dim = x.shape
    handle = _lib.lib()
    blocks = handle.sfl_rmsnorm_bwd_blocks(rows)
    partial = torch.empty(blocks, dim, dtype=torch.float32, device=x.device)
    dx = torch.empty_like(x)
    dx_bf16 = torch.empty(rows, dim, dtype=torch.bfloat16, device=x.device) if want_bf16 else None
    stream = _lib.stream_ptr()
    code = handle.sfl_rmsnorm_bwd(dy.data_ptr(), x.data_ptr(), weight.data_ptr(), rstd.data_ptr(),
                                  _lib.ptr(dres), dx.data_ptr(), _lib.ptr(dx_bf16),
                                  partial.data_ptr(), rows, dim, stream)
    _lib.check(code, "sfl_rmsnorm_bwd")
    code = handle.sfl_rmsnorm_dw_reduce(partial.data_ptr(), blocks, dweight.data_ptr(), dim,
                                        int(accumulate), stream)
    _lib.check(code, "sfl_rmsnorm_dw_reduce")
    return dx, dx_bf16


def cast_bf16(src: torch.Tensor, dst: torch.Tensor | None = None) -> torch.Tensor:
    _f32(src, "src")
    if dst is None:
        dst = torch.empty(src.shape, dtype=torch.bfloat16, device=src.device)
    code = _lib.lib().sfl_cast_f32_to_bf16(src.data_ptr(), dst.data_ptr(), src.numel(),
                                          _lib.stream_ptr())
    _lib.check(code, "sfl_cast_f32_to_bf16")
    return dst


def embedding(weight: torch.Tensor, ids: torch.Tensor) -> torch.Tensor:
    """fp32 rows of ``weight`` for int64 ``ids`` of any shape."""
    flat = ids.reshape(-1).contiguous()
    if flat.dtype != torch.int64:
        flat = flat.to(torch.int64)
    out = torch.empty(flat.numel(), weight.shape[1], dtype=torch.float32, device=weight.device)
    code = _lib.lib().sfl_embedding_fwd(weight.data_ptr(), flat.data_ptr(), out.data_ptr(),
                                       flat.numel(), weight.shape[1], weight.shape[0],
                                       _lib.stream_ptr())
    _lib.check(code, "sfl_embedding_fwd")
    return out.view(*ids.shape, weight.shape[1])


def scale_bf16_unless_one(x: torch.Tensor, coef: torch.Tensor) -> None:
    """In place ``x *= coef`` for contiguous bf16 ``x`` and a one-element fp32 device
    tensor; the kernel returns immediately when the factor is exactly one."""
    if x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("expects a contiguous bf16 tensor")
    if coef.dtype != torch.float32 or coef.numel() != 1 or coef.device != x.device:
        coef = coef.reshape(-1)[:1].to(device=x.device, dtype=torch.float32)
    code = _lib.lib().sfl_scale_bf16_unless_one(x.data_ptr(), x.numel(), coef.data_ptr(),
                                               _lib.stream_ptr())
    _lib.check(code, "sfl_scale_bf16_unless_one")


EMBEDDING_BWD_MAX_ROWS = 51200     # the ids of one call must fit in shared memory


def embedding_bwd(dx: torch.Tensor, ids: torch.Tensor, dweight: torch.Tensor,
                  accumulate: bool) -> bool:
    """``dweight[ids[t]] (+)= dx[t]`` summed in token order (deterministic, no sort, no
    dense temporary).  Returns False, without touching ``dweight``, when the call
    has more tokens than the kernel handles; the caller then uses another route."""
    flat = ids.reshape(-1).contiguous()
    if flat.dtype != torch.int64:
        flat = flat.to(torch.int64)
    rows, dim = flat.numel(), dweight.shape[1]
    if rows > EMBEDDING_BWD_MAX_ROWS:
        return False
    dx2 = dx.reshape(rows, dim)
    if dx2.dtype != torch.float32 or not dx2.is_contiguous():
        dx2 = dx2.float().contiguous()
    if dweight.dtype != torch.float32 or not dweight.is_contiguous():
        raise ValueError("embedding gradients are fp32 and contiguous")
    scratch = torch.empty(rows + dweight.shape[0], dtype=torch.int32, device=dx.device)
    code = _lib.lib().sfl_embedding_bwd(dx2.data_ptr(), flat.data_ptr(), dweight.data_ptr(), rows,
                                       dim, dweight.shape[0], int(accumulate),
                                       scratch.data_ptr(), scratch[rows:].data_ptr(),
                                       _lib.stream_ptr())
    _lib.check(code, "sfl_embedding_bwd")
    return True


def cross_entropy_rows(logits: torch.Tensor, targets: torch.Tensor, vocab: int,
                       dlogits: torch.Tensor | None, grad_scale: float) -> torch.Tensor:
    """Per-row loss of bf16 ``logits[rows, ld]`` over the first ``vocab`` columns.

    When ``dlogits`` is given (it may be ``logits`` itself) it receives
    ``(softmax - onehot) * grad_scale`` in bf16 from the same pass.
    """
    rows = logits.shape[0]
    if targets.dtype != torch.int64 or targets.numel() != rows:
        raise ValueError("targets must be int64 with one entry per row")
    losses = torch.empty(rows, dtype=torch.float32, device=logits.device)
    code = _lib.lib().sfl_cross_entropy(logits.data_ptr(), logits.stride(0), targets.data_ptr(),
                                       losses.data_ptr(), _lib.ptr(dlogits), float(grad_scale),
                                       rows, vocab, _lib.stream_ptr())
    _lib.check(code, "sfl_cross_entropy")
    return losses


def grad_norm_and_coef(flat_grad: torch.Tensor, max_norm: float, sum_scale: float = 1.0,
                       extra_partials: torch.Tensor | None = None) -> torch.Tensor:
    """Device vector ``[norm, clip coefficient, finite flag]`` of a flat fp32 buffer."""
    handle = _lib.lib()
    n = flat_grad.numel()
    blocks = handle.sfl_sqnorm_blocks(n)
    partial = torch.empty(blocks, dtype=torch.float32, device=flat_grad.device)
    stream = _lib.stream_ptr()
    _lib.check(handle.sfl_sqnorm_partial(flat_grad.data_ptr(), n, partial.data_ptr(), stream),
               "sfl_sqnorm_partial")
    if extra_partials is not None:
        partial = torch.cat([partial, extra_partials.reshape(-1)])
    out = torch.empty(3, dtype=torch.float32, device=flat_grad.device)
    _lib.check(handle.sfl_norm_finalize(partial.data_ptr(), partial.numel(), float(sum_scale),
                                        float(max_norm), out.data_ptr(), stream),
               "sfl_norm_finalize")
    return out


def adamw_step(param: torch.Tensor, grad: torch.Tensor, exp_avg: torch.Tensor,
               exp_avg_sq: torch.Tensor, shadow: torch.Tensor | None, *, step: int, lr: float,
               beta1: float, beta2: float, eps: float, weight_decay: float,
               coef: torch.Tensor | None = None, grad_scale: float = 1.0,
               ok_flag: torch.Tensor | None = None) -> None:
    """One AdamW update over flat fp32 ranges; ``coef`` is a device scalar that
    multiplies the gradient (the clip coefficient), ``ok_flag`` a device scalar
    that suppresses the update when zero."""
    n = param.numel()
    code = _lib.lib().sfl_adamw(param.data_ptr(), grad.data_ptr(), exp_avg.data_ptr(),
                               exp_avg_sq.data_ptr(), _lib.ptr(shadow), n, float(lr), float(beta1),
                               float(beta2), float(eps), float(weight_decay),
                               1.0 - beta1 ** step, 1.0 - beta2 ** step, _lib.ptr(coef),
                               float(grad_scale), _lib.ptr(ok_flag), _lib.stream_ptr())
    _lib.check(code, "sfl_adamw")
