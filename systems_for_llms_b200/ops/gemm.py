"""Python front end of the tcgen05 GEMM (csrc/gemm.cu).

``gemm`` is the raw launcher; the helpers below name the products a linear layer
needs.  Operands are bf16 tensors; "mn-major" means the tensor is stored with the
output (M or N) dimension contiguous, so weight- and input-gradient products run
on the tensors as they already sit in memory:

    forward   y[M,N]  = x[M,K]  @ w[N,K]^T     a K-major, b K-major
    dgrad     dx[M,K] = dy[M,N] @ w[N,K]       a K-major, b MN-major
    wgrad     dw[N,K] = dy[M,N]^T @ x[M,K]     a MN-major, b MN-major (reduce over M)
"""

from __future__ import annotations

import ctypes

import torch

from . import lib as _lib
from .lib import (EPI_BF16, EPI_F32, EPI_RESID, EPI_ROPE, EPI_SWIGLU, EPI_SWIGLU_BWD,
                  GemmEpilogue, WgradProblem)

_status_words: dict[torch.device, torch.Tensor] = {}


def status_word(device: torch.device) -> torch.Tensor:
    """Device int32 that kernels set when a bounded wait runs out."""
    device = torch.device(device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    word = _status_words.get(device)
    if word is None:
        word = torch.zeros(1, dtype=torch.int32, device=device)
        _status_words[device] = word
    return word


def check_status(device: torch.device | None = None) -> None:
    """Raises if any kernel on ``device`` reported a timed-out wait (host sync)."""
    for dev, word in list(_status_words.items()):
        if device is not None and torch.device(device) != dev:
            continue
        code = int(word.item())
        if code != 0:
            word.zero_()
            raise RuntimeError(f"sm_100a kernel reported status {code} on {dev}")


def status_report(device: torch.device) -> torch.Tensor:
    """The status word of ``device`` as a one-element fp32 tensor on that device (zero when
    no kernel of this library has run there), for a trainer to append to the values it reads
    back every step anyway: a wait that ran out then stops the run at that step instead of
    letting it continue on incomplete gradients or activations."""
    device = torch.device(device)
    if device.type != "cuda":
        return torch.zeros(1, device=device)
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    word = _status_words.get(device)
    if word is None:
        return torch.zeros(1, device=device)
    return word.to(torch.float32)


def raise_on_status(code: float, device) -> None:
    """Counterpart of ``status_report`` once the value is on the host."""
    if code != 0:
        word = _status_words.get(torch.device(device))
        if word is not None:
            word.zero_()
        raise RuntimeError(f"sm_100a kernel reported status {int(code)} on {device}: a bounded "
                           "wait ran out, so this step's results are incomplete")


def _operand(t: torch.Tensor) -> tuple[int, int]:
    if t.dtype != torch.bfloat16 or t.dim() != 2 or t.stride(1) != 1:
        raise ValueError("GEMM operands must be 2-D bf16 with a contiguous last dimension")
    if t.stride(0) % 8 or t.data_ptr() % 16:
        raise ValueError("GEMM operands need 16-byte aligned rows")
    return t.data_ptr(), t.stride(0)


def gemm(a: torch.Tensor, b: torch.Tensor, M: int, N: int, K: int, epilogue: GemmEpilogue, *,
         a_mn: bool = False, b_mn: bool = False, bn: int = 0, max_ctas: int = 0) -> None:
    a_ptr, lda = _operand(a)
    b_ptr, ldb = _operand(b)
    if epilogue.status is None:
        epilogue.status = status_word(a.device).data_ptr()
    code = _lib.lib().sfl_gemm_bf16(a_ptr, lda, int(a_mn), b_ptr, ldb, int(b_mn), M, N, K,
                                   ctypes.byref(epilogue), bn, max_ctas, _lib.stream_ptr())
    _lib.check(code, "sfl_gemm_bf16")


def supported(*dims: int) -> bool:
    """The kernel needs every leading dimension to be a multiple of 8 elements."""
    return all(d % 8 == 0 and d > 0 for d in dims)


def linear_fwd(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 ``x[M,K] @ w[N,K]^T``."""
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    epi = GemmEpilogue(kind=EPI_BF16, out=out.data_ptr(), ldo=out.stride(0))
    gemm(x, w, M, N, K, epi)
    return out


def linear_fwd_resid(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor,
                     out: torch.Tensor | None = None) -> torch.Tensor:
    """fp32 ``resid + bf16(x @ w^T)`` (the residual-stream update)."""
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32, device=x.device)
    epi = GemmEpilogue(kind=EPI_RESID, out=out.data_ptr(), ldo=out.stride(0),
                       aux=resid.data_ptr(), ldaux=resid.stride(0))
    gemm(x, w, M, N, K, epi)
    return out


def linear_fwd_rope(x: torch.Tensor, w: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                    seq_len: int, rope_cols: int, head_dim: int,
                    out: torch.Tensor | None = None) -> torch.Tensor:
    """Fused q|k|v projection with rotary embedding on the first ``rope_cols`` columns."""
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    epi = GemmEpilogue(kind=EPI_ROPE, out=out.data_ptr(), ldo=out.stride(0),
                       rope_cos=cos.data_ptr(), rope_sin=sin.data_ptr(), rope_T=seq_len,
                       rope_cols=rope_cols, head_dim=head_dim)
    gemm(x, w, M, N, K, epi)
    return out


def swiglu_fwd(x: torch.Tensor, w13: torch.Tensor, d_ff: int) -> tuple[torch.Tensor, torch.Tensor]:
    """``w13`` stacks w1 on w3 ([2*d_ff, K]).  Returns (silu(a1)*a3, [a1 | a3])."""
    M, K = x.shape
    g = torch.empty(M, d_ff, dtype=torch.bfloat16, device=x.device)
    a13 = torch.empty(M, 2 * d_ff, dtype=torch.bfloat16, device=x.device)
    epi = GemmEpilogue(kind=EPI_SWIGLU, out=g.data_ptr(), ldo=g.stride(0), out2=a13.data_ptr(),
                       ldo2=a13.stride(0), dual_offset=d_ff, dual_rows=2 * d_ff)
    gemm(x, w13, M, d_ff, K, epi)
    return g, a13


def swiglu_bwd(dy: torch.Tensor, w2: torch.Tensor, a13: torch.Tensor) -> torch.Tensor:
    """``dy[M,D] @ w2[D,d_ff]`` with the SwiGLU derivative applied: returns [da1 | da3]."""
    M, D = dy.shape
    d_ff = w2.shape[1]
    out = torch.empty(M, 2 * d_ff, dtype=torch.bfloat16, device=dy.device)
    epi = GemmEpilogue(kind=EPI_SWIGLU_BWD, out=out.data_ptr(), ldo=out.stride(0),
                       aux=a13.data_ptr(), ldaux=a13.stride(0))
    gemm(dy, w2, M, d_ff, D, epi, b_mn=True)
    return out


def linear_dgrad(dy: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 ``dy[M,N] @ w[N,K]`` -> [M,K]."""
    M, N = dy.shape
    K = w.shape[1]
    if out is None:
        out = torch.empty(M, K, dtype=torch.bfloat16, device=dy.device)
    epi = GemmEpilogue(kind=EPI_BF16, out=out.data_ptr(), ldo=out.stride(0))
    gemm(dy, w, M, K, N, epi, b_mn=True)
    return out


def linear_wgrad(dy: torch.Tensor, x: torch.Tensor, grad: torch.Tensor, accumulate: bool) -> None:
    """fp32 ``grad[N,K] (+)= dy[M,N]^T @ x[M,K]``; reduces over the M rows."""
    M, N = dy.shape
    K = x.shape[1]
    if grad.dtype != torch.float32 or grad.stride(1) != 1:
        raise ValueError("weight gradients are fp32 and row-contiguous")
    epi = GemmEpilogue(kind=EPI_F32, beta=int(accumulate), out=grad.data_ptr(), ldo=grad.stride(0))
    gemm(dy, x, N, K, M, epi, a_mn=True, b_mn=True)


MAX_WGRAD_GROUP = 4


def _groupable(dy: torch.Tensor, x: torch.Tensor, grad: torch.Tensor) -> bool:
    return (dy.stride(0) % 8 == 0 and x.stride(0) % 8 == 0 and grad.stride(0) % 4 == 0
            and dy.data_ptr() % 16 == 0 and x.data_ptr() % 16 == 0 and grad.data_ptr() % 16 == 0)


def wgrad_grouped(problems) -> None:
    """``grad (+)= dy^T @ x`` for several layers in one persistent launch.

    ``problems`` is a list of ``(dy, x, grad, accumulate)``.  One weight-gradient
    product has too few output tiles to occupy every SM; walking the tiles of a
    whole transformer block's four products in one kernel leaves only the last
    round of the group partially filled.  Products that cannot be addressed by
    TMA fall back to ``linear_wgrad`` one at a time.
    """
    group = []
    for dy, x, grad, accumulate in problems:
        if grad.dtype != torch.float32 or grad.stride(1) != 1:
            raise ValueError("weight gradients are fp32 and row-contiguous")
        if dy.shape[0] != x.shape[0] or grad.shape != (dy.shape[1], x.shape[1]):
            raise ValueError("wgrad shapes: dy[T,N], x[T,K], grad[N,K]")
        if _groupable(dy, x, grad):
            _operand(dy), _operand(x)
            group.append((dy, x, grad, accumulate))
        else:
            linear_wgrad(dy, x, grad, accumulate)
    for start in range(0, len(group), MAX_WGRAD_GROUP):
        chunk = group[start:start + MAX_WGRAD_GROUP]
        if len(chunk) == 1:
            linear_wgrad(*chunk[0])
            continue
        array = (WgradProblem * len(chunk))()
        for slot, (dy, x, grad, accumulate) in zip(array, chunk):
            slot.dy, slot.ld_dy = dy.data_ptr(), dy.stride(0)
            slot.x, slot.ld_x = x.data_ptr(), x.stride(0)
            slot.grad, slot.ld_grad = grad.data_ptr(), grad.stride(0)
            slot.rows, slot.cols, slot.tokens = dy.shape[1], x.shape[1], dy.shape[0]
            slot.accumulate = int(bool(accumulate))
        code = _lib.lib().sfl_gemm_wgrad_grouped(array, len(chunk),
                                                 status_word(chunk[0][0].device).data_ptr(),
                                                 _lib.stream_ptr())
        _lib.check(code, "sfl_gemm_wgrad_grouped")
