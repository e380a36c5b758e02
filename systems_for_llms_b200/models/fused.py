"""The sm_100a execution engine behind ``TransformerLM`` on a B200.

Design (none of this exists in the reference, which runs every operator as an
eager PyTorch call: src/llmlab/model/transformer.py:121-139):

* **Flat storage.**  All parameters are re-pointed into one fp32 buffer (the
  ``nn.Parameter`` objects and ``state_dict`` keys are untouched), with q|k|v
  and w1|w3 adjacent so the fused projections see one matrix.  A bf16 shadow
  of the same layout feeds the tensor cores; it is refreshed by the fused
  optimizer, or by a cast when a parameter was modified through PyTorch.
  Gradients live in a second flat fp32 buffer that weight-gradient GEMMs
  accumulate into directly, and that data-parallel wrappers reduce in place.
* **One autograd node per block.**  Forward is seven kernels (norm, q|k|v+RoPE
  GEMM, flash attention, output GEMM+residual, norm, w1|w3 GEMM+SwiGLU, w2
  GEMM+residual); backward is the matching hand-written chain.  With
  ``activation_checkpointing="block"`` the node stores only its input and
  replays the forward inside backward.
* **Fused head.**  Final norm, vocabulary GEMM, log-sum-exp, loss and the logit
  gradient are one node; fp32 logits never exist.
"""

from __future__ import annotations

import ctypes
import math
import os

import torch

from ..attention import flash
from ..ops import functional as K
from ..ops import gemm as G
from ..ops import lib as _lib

ALIGN = 64  # elements; keeps every parameter 256-byte (fp32) / 128-byte (bf16) aligned


def autocast_bf16_active() -> bool:
    return (torch.is_autocast_enabled("cuda")
            and torch.get_autocast_dtype("cuda") == torch.bfloat16)


def eligible(model) -> bool:
    """Shapes and placement the kernels support; otherwise the portable path runs."""
    if not _lib.available():
        return False
    params = list(model.parameters())
    if not params or any((not p.is_cuda) or p.dtype != torch.float32 for p in params):
        return False
    if len({p.device for p in params}) != 1:
        return False
    d_k = model.d_model // model.num_heads
    first = model.layers[0]
    local_ff = first.ffn.w1.weight.shape[0]            # d_ff, or d_ff / tp under tensor parallelism
    local_attn = first.attn.q_proj.weight.shape[0]     # d_model, or d_model / tp
    return (model.d_model % 64 == 0 and d_k in (64, 128) and local_ff % 8 == 0
            and local_attn % d_k == 0 and (local_attn * model.d_model) % ALIGN == 0
            and (local_ff * model.d_model) % ALIGN == 0
            and model.vocab_size >= 8 and all(layer.attn.rope is not None for layer in model.layers))


def _round_up(value: int, multiple: int) -> int:
    return -(-value // multiple) * multiple


class FusedEngine:
    def __init__(self, model):
        self.model = model
        self.device = next(model.parameters()).device
        self.d_model = model.d_model
        self.d_k = model.d_model // model.num_heads
        first = model.layers[0]
        # Widths held by this rank (the full widths unless tensor parallel).
        self.attn_width = first.attn.q_proj.weight.shape[0]
        self.num_heads = self.attn_width // self.d_k
        self.d_ff = first.ffn.w1.weight.shape[0]
        self.vocab = model.vocab_size
        self.tp = None   # parallel.tensor_parallel.TensorParallelComm when sharded
        self._layout()
        self._flatten()
        self.flat_grad: torch.Tensor | None = None
        self._shadow_views: dict = {}
        self._grad_views: dict = {}
        # Run whole blocks through one library call (csrc/block.cu) instead of one
        # Python-driven launch per kernel; tensor-parallel engines keep the latter.
        self.native_blocks = os.environ.get("SFL_PYTHON_BLOCKS", "0") != "1"
        self._native_args: dict = {}
        self._native_sizes: dict = {}
        self._native_keep: list = []
        self._versions = None
        self._bf16_alias: tuple[int, torch.Tensor] | None = None
        # hook(offset): every gradient at flat offset >= offset is final for this backward
        self.on_block_backward = None
        rope = model.layers[0].attn.rope
        # Tables hold the bf16-rounded values the reference multiplies with.
        self.cos = rope.cos.to(torch.bfloat16).to(torch.float32).contiguous()
        self.sin = rope.sin.to(torch.bfloat16).to(torch.float32).contiguous()

    # ---------------------------------------------------------------- layout --
    def _layout(self) -> None:
        model = self.model
        # Embeddings first and the head last: backward then finalises gradients from
        # the end of the flat buffer towards its start, which is the order in which
        # a data-parallel wrapper can reduce fixed-size buckets.
        order = [model.token_embeddings.weight]
        for layer in model.layers:
            order += [layer.attn_norm.weight, layer.attn.q_proj.weight, layer.attn.k_proj.weight,
                      layer.attn.v_proj.weight, layer.attn.output_proj.weight,
                      layer.ffn_norm.weight, layer.ffn.w1.weight, layer.ffn.w3.weight,
                      layer.ffn.w2.weight]
        order += [model.ln_final.weight, model.lm_head.weight]
        self.params = order
        self.offsets: dict[int, int] = {}
        cursor = 0
        for p in order:
            self.offsets[id(p)] = cursor
            cursor += _round_up(p.numel(), ALIGN)
        self.total = cursor
        # Start offset of every block and of the head in the flat buffers.
        self.layer_ranges = []
        for layer in model.layers:
            begin = self.offsets[id(layer.attn_norm.weight)]
            end = self.offsets[id(layer.ffn.w2.weight)] + _round_up(layer.ffn.w2.weight.numel(), ALIGN)
            self.layer_ranges.append((begin, end))
        self.head_offset = self.offsets[id(model.ln_final.weight)]

    def _flatten(self) -> None:
        flat = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        for p in self.params:
            view = self._slice(flat, p)
            view.copy_(p.data)
            p.data = view
        self.flat_param = flat
        self.flat_shadow = torch.empty(self.total, dtype=torch.bfloat16, device=self.device)

    def _slice(self, flat: torch.Tensor, p: torch.Tensor) -> torch.Tensor:
        begin = self.offsets[id(p)]
        return flat[begin:begin + p.numel()].view(p.shape)

    def shadow(self, p: torch.Tensor, rows: int | None = None) -> torch.Tensor:
        """bf16 view of ``p``; ``rows`` extends it over adjacent matrices (q|k|v, w1|w3).

        Views are cached per (parameter, rows) and rebuilt when the flat buffer is
        replaced: building a slice + view costs microseconds and every kernel
        launch of the block needs one.
        """
        flat = self.flat_shadow
        key = (id(p), rows)
        hit = self._shadow_views.get(key)
        if hit is not None and hit[0] is flat:
            return hit[1]
        begin = self.offsets[id(p)]
        count = p.shape[0] if rows is None else rows
        view = flat[begin:begin + count * p.shape[1]].view(count, p.shape[1])
        self._shadow_views[key] = (flat, view)
        return view

    def relocate(self, flat_param: torch.Tensor | None = None,
                 flat_grad: torch.Tensor | None = None) -> None:
        """Move parameters / gradients into caller-provided flat buffers (for
        example peer-mapped memory owned by a data-parallel wrapper)."""
        if flat_param is not None:
            if flat_param.numel() < self.total or flat_param.dtype != torch.float32:
                raise ValueError("parameter buffer too small or not fp32")
            flat_param[:self.total].copy_(self.flat_param)
            for p in self.params:
                p.data = self._slice(flat_param, p)
            self.flat_param = flat_param
        if flat_grad is not None:
            if flat_grad.numel() < self.total or flat_grad.dtype != torch.float32:
                raise ValueError("gradient buffer too small or not fp32")
            self.flat_grad = flat_grad
            for p in self.params:
                if p.grad is not None:
                    view = self._slice(flat_grad, p)
                    view.copy_(p.grad)
                    p.grad = view

    # ------------------------------------------------------------- gradients --
    def grad_buffer(self) -> torch.Tensor:
        if self.flat_grad is None:
            self.flat_grad = torch.zeros(self.total, dtype=torch.float32, device=self.device)
        return self.flat_grad

    def grad_view(self, p: torch.Tensor, rows: int | None = None) -> torch.Tensor:
        flat = self.grad_buffer()
        key = (id(p), rows)
        hit = self._grad_views.get(key)
        if hit is not None and hit[0] is flat:
            return hit[1]
        begin = self.offsets[id(p)]
        if rows is None:
            view = flat[begin:begin + p.numel()].view(p.shape)
        else:
            view = flat[begin:begin + rows * p.shape[1]].view(rows, p.shape[1])
        self._grad_views[key] = (flat, view)
        return view

    def claim(self, *params: torch.Tensor) -> bool:
        """Attach the flat views as ``.grad`` and say whether to accumulate.

        A parameter whose ``.grad`` is ``None`` (after ``zero_grad``) starts a new
        accumulation: the first kernel overwrites instead of adding, so the flat
        buffer never needs a separate clearing pass.
        """
        fresh = [p.grad is None for p in params]
        if any(fresh) and not all(fresh):
            # Mixed state inside one fused matrix: zero the stragglers, then add.
            for p, is_fresh in zip(params, fresh):
                if is_fresh:
                    self.grad_view(p).zero_()
        accumulate = not all(fresh)
        for p in params:
            view = self.grad_view(p)
            if p.grad is None or p.grad.data_ptr() != view.data_ptr():
                if p.grad is not None:
                    view.copy_(p.grad)
                p.grad = view
        return accumulate

    # ---------------------------------------------------------------- shadow --
    def sync_shadow(self) -> None:
        """Re-cast fp32 -> bf16 if any parameter changed through PyTorch."""
        versions = tuple(p._version for p in self.params)
        if versions != self._versions:
            K.cast_bf16(self.flat_param, self.flat_shadow)
            self._versions = versions

    def prepare_block(self, index: int, backward: bool) -> None:
        """Called before block ``index`` runs (forward or backward).  The base engine
        has every weight resident; sharded engines gather the block here."""

    def embedding_table(self) -> torch.Tensor:
        return self.model.token_embeddings.weight

    def mark_shadow_current(self) -> None:
        """Called by the fused optimizer, which writes the shadow itself."""
        self._versions = tuple(p._version for p in self.params)

    # --------------------------------------------------------------- forward --
    def _prepare(self, input_ids: torch.Tensor):
        self.sync_shadow()
        ids = input_ids.reshape(-1, input_ids.shape[-1])
        return ids, ids.shape[0], ids.shape[1]

    def _trunk(self, ids: torch.Tensor, B: int, T: int) -> torch.Tensor:
        model = self.model
        grad = torch.is_grad_enabled()
        if grad:
            x = _Embed.apply(model.token_embeddings.weight, ids, self)
        else:
            x = K.embedding(self.embedding_table(), ids)
        recompute = model.activation_checkpointing == "block" and model.training and grad
        for index in range(len(model.layers)):
            if grad:
                x = _Block.apply(x, self, index, B, T, recompute)
            else:
                x = block_forward(self, index, x, B, T)[0]
        return x

    def logits(self, input_ids: torch.Tensor) -> torch.Tensor:
        ids, B, T = self._prepare(input_ids)
        x = self._trunk(ids, B, T)
        if torch.is_grad_enabled():
            out = _Logits.apply(x, self)
        else:
            out = head_logits(self, x)[0]
        return out[:, :self.vocab].reshape(*input_ids.shape, self.vocab)

    def loss(self, input_ids: torch.Tensor, targets: torch.Tensor, scale: float) -> torch.Tensor:
        ids, B, T = self._prepare(input_ids)
        x = self._trunk(ids, B, T)
        flat_targets = targets.reshape(-1).contiguous()
        if torch.is_grad_enabled():
            return _HeadLoss.apply(x, flat_targets, self, float(scale))
        logits = head_logits(self, x)[0]
        rows = K.cross_entropy_rows(logits, flat_targets, self.vocab, None, 0.0)
        return rows.sum() * (scale / rows.numel())


# ----------------------------------------------------- native block runner --
def _native_args(engine: FusedEngine, index: int, B: int, T: int) -> "_lib.BlockArgs":
    """The constant part of a block's argument record; pointers that change per call
    (activations, weights of sharded engines) are filled in by the callers."""
    cache = engine._native_args
    key = (index, B, T)
    args = cache.get(key)
    if args is None:
        layer = engine.model.layers[index]
        args = _lib.BlockArgs()
        args.batch, args.seq_len, args.d_model = B, T, engine.d_model
        args.heads, args.head_dim, args.d_ff = engine.num_heads, engine.d_k, engine.d_ff
        args.eps1, args.eps2 = layer.attn_norm.eps, layer.ffn_norm.eps
        args.attn_scale = engine.d_k ** -0.5
        args.rope_cos, args.rope_sin = engine.cos.data_ptr(), engine.sin.data_ptr()
        mask = flash.causal_mask(engine.device, T)
        args.mask = ctypes.addressof(mask.struct)
        args.status = G.status_word(engine.device).data_ptr()
        handle = _lib.lib()
        sizes = (handle.sfl_block_saved_bytes(ctypes.byref(args)),
                 handle.sfl_block_scratch_bytes(ctypes.byref(args)))
        if min(sizes) <= 0:
            raise RuntimeError("block shape not supported by the native runner")
        cache[key] = args
        engine._native_sizes[key] = sizes
        engine._native_keep.append(mask)      # the record points into the mask
    return args


def _native_weights(engine: FusedEngine, args, layer) -> None:
    aw, dff = engine.attn_width, engine.d_ff
    args.wqkv = engine.shadow(layer.attn.q_proj.weight, 3 * aw).data_ptr()
    args.wo = engine.shadow(layer.attn.output_proj.weight).data_ptr()
    args.w13 = engine.shadow(layer.ffn.w1.weight, 2 * dff).data_ptr()
    args.w2 = engine.shadow(layer.ffn.w2.weight).data_ptr()
    args.norm1 = layer.attn_norm.weight.data_ptr()
    args.norm2 = layer.ffn_norm.weight.data_ptr()


def native_block_forward(engine: FusedEngine, index: int, x: torch.Tensor, B: int, T: int):
    """``block_forward`` through one library call (csrc/block.cu)."""
    layer = engine.model.layers[index]
    engine.prepare_block(index, False)
    args = _native_args(engine, index, B, T)
    x2 = x.reshape(B * T, engine.d_model)
    if not x2.is_contiguous():
        x2 = x2.contiguous()
    saved = torch.empty(engine._native_sizes[(index, B, T)][0], dtype=torch.uint8, device=x.device)
    _native_weights(engine, args, layer)
    if engine.tp is None:
        out = torch.empty_like(x2)
        args.x_out = out.data_ptr()
    else:   # results land in the symmetric pool on every rank
        out = engine.tp.fill_block_args(args, index, B * T, engine.d_model)
    args.x, args.saved = x2.data_ptr(), saved.data_ptr()
    code = _lib.lib().sfl_block_forward(ctypes.byref(args), _lib.stream_ptr())
    _lib.check(code, "sfl_block_forward")
    return out.view(B, T, engine.d_model), (x2, saved)


def native_block_backward(engine: FusedEngine, index: int, saved, d_out: torch.Tensor, B: int,
                          T: int):
    layer = engine.model.layers[index]
    attn_p, ffn = layer.attn, layer.ffn
    d, aw, dff = engine.d_model, engine.attn_width, engine.d_ff
    x2, buffer = saved
    args = _native_args(engine, index, B, T)
    dres = d_out.reshape(B * T, d)
    if not dres.is_contiguous():
        dres = dres.contiguous()
    alias = engine._bf16_alias
    engine._bf16_alias = None
    scratch = torch.empty(engine._native_sizes[(index, B, T)][1], dtype=torch.uint8,
                          device=dres.device)
    dx = torch.empty_like(dres)
    dx_bf16 = torch.empty(B * T, d, dtype=torch.bfloat16, device=dres.device)
    _native_weights(engine, args, layer)
    args.x, args.saved, args.scratch = x2.data_ptr(), buffer.data_ptr(), scratch.data_ptr()
    args.d_out = dres.data_ptr()
    args.d_out_bf16 = (alias[1].data_ptr()
                       if alias is not None and alias[0] == dres.data_ptr() else None)
    args.dx, args.dx_bf16 = dx.data_ptr(), dx_bf16.data_ptr()
    args.acc_w2 = engine.claim(ffn.w2.weight)
    args.acc_w13 = engine.claim(ffn.w1.weight, ffn.w3.weight)
    args.acc_norm2 = engine.claim(layer.ffn_norm.weight)
    args.acc_wo = engine.claim(attn_p.output_proj.weight)
    args.acc_wqkv = engine.claim(attn_p.q_proj.weight, attn_p.k_proj.weight, attn_p.v_proj.weight)
    args.acc_norm1 = engine.claim(layer.attn_norm.weight)
    args.g_w2 = engine.grad_view(ffn.w2.weight).data_ptr()
    args.g_w13 = engine.grad_view(ffn.w1.weight, 2 * dff).data_ptr()
    args.g_norm2 = engine.grad_view(layer.ffn_norm.weight).data_ptr()
    args.g_wo = engine.grad_view(attn_p.output_proj.weight).data_ptr()
    args.g_wqkv = engine.grad_view(attn_p.q_proj.weight, 3 * aw).data_ptr()
    args.g_norm1 = engine.grad_view(layer.attn_norm.weight).data_ptr()
    if engine.tp is not None:
        engine.tp.fill_block_args(args, index, B * T, d)
    code = _lib.lib().sfl_block_backward(ctypes.byref(args), _lib.stream_ptr())
    _lib.check(code, "sfl_block_backward")
    engine._bf16_alias = (dx.data_ptr(), dx_bf16)
    if engine.on_block_backward is not None:
        engine.on_block_backward(engine.layer_ranges[index][0])
    return dx.view(B, T, d)


def _use_native(engine: FusedEngine) -> bool:
    """One library call per block; tensor-parallel engines qualify when their
    reductions can run inside the GEMM kernels."""
    if not engine.native_blocks:
        return False
    return engine.tp is None or engine.tp.can_fuse(engine.d_model)


# ------------------------------------------------------------ block kernels --
def block_forward(engine: FusedEngine, index: int, x: torch.Tensor, B: int, T: int):
    """Returns ``(x_out, saved)`` where ``saved`` holds what backward needs."""
    if _use_native(engine):
        return native_block_forward(engine, index, x, B, T)
    layer = engine.model.layers[index]
    d, dk, H, dff, aw = engine.d_model, engine.d_k, engine.num_heads, engine.d_ff, engine.attn_width
    tp = engine.tp
    M = B * T
    engine.prepare_block(index, False)
    x2 = x.reshape(M, d)
    h1, rstd1 = K.rmsnorm(x2, layer.attn_norm.weight, layer.attn_norm.eps)
    wqkv = engine.shadow(layer.attn.q_proj.weight, 3 * aw)
    qkv = G.linear_fwd_rope(h1, wqkv, engine.cos, engine.sin, T, 2 * aw, dk)
    heads = qkv.view(B, T, 3, H, dk)
    q, k, v = (heads[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    attn = torch.empty(M, aw, dtype=torch.bfloat16, device=x.device)
    lse = torch.empty(B, H, T, dtype=torch.float32, device=x.device)
    mask = flash.causal_mask(x.device, T)
    flash.flash_fwd(q, k, v, attn.view(B, T, H, dk).permute(0, 2, 1, 3), lse, mask, dk ** -0.5)
    wo = engine.shadow(layer.attn.output_proj.weight)
    if tp is None:
        x_mid = G.linear_fwd_resid(attn, wo, x2)
    elif tp.can_fuse(d):   # row-parallel: GEMM, sum over ranks and residual add in one kernel
        x_mid = tp.gemm_reduce_residual(attn, wo, x2, 2 * index)
    else:   # bf16 partial sums -> a second kernel sums peers and adds the residual
        x_mid = tp.reduce_residual(G.linear_fwd(attn, wo, tp.partial(M, d)), x2, 2 * index)
    h2, rstd2 = K.rmsnorm(x_mid, layer.ffn_norm.weight, layer.ffn_norm.eps)
    g, a13 = G.swiglu_fwd(h2, engine.shadow(layer.ffn.w1.weight, 2 * dff), dff)
    w2 = engine.shadow(layer.ffn.w2.weight)
    if tp is None:
        x_out = G.linear_fwd_resid(g, w2, x_mid)
    elif tp.can_fuse(d):
        x_out = tp.gemm_reduce_residual(g, w2, x_mid, 2 * index + 1)
    else:
        x_out = tp.reduce_residual(G.linear_fwd(g, w2, tp.partial(M, d)), x_mid, 2 * index + 1)
    saved = (x2, rstd1, h1, qkv, attn, lse, x_mid, rstd2, h2, a13, g)
    return x_out.view(B, T, d), saved


def block_backward(engine: FusedEngine, index: int, saved, d_out: torch.Tensor, B: int, T: int):
    if _use_native(engine):
        return native_block_backward(engine, index, saved, d_out, B, T)
    layer = engine.model.layers[index]
    d, dk, H, dff, aw = engine.d_model, engine.d_k, engine.num_heads, engine.d_ff, engine.attn_width
    tp = engine.tp
    M = B * T
    x2, rstd1, h1, qkv, attn, lse, x_mid, rstd2, h2, a13, g = saved
    dres = d_out.reshape(M, d)
    if not dres.is_contiguous():
        dres = dres.contiguous()
    alias = engine._bf16_alias
    if alias is not None and alias[0] == dres.data_ptr():
        dres_bf16 = alias[1]
    else:
        dres_bf16 = K.cast_bf16(dres)
    engine._bf16_alias = None
    attn_p, ffn = layer.attn, layer.ffn

    # ---- feed-forward half
    d13 = G.swiglu_bwd(dres_bf16, engine.shadow(ffn.w2.weight), a13)
    # the four weight gradients of the block run as one grouped launch at the end
    wgrads = [(dres_bf16, g, engine.grad_view(ffn.w2.weight), engine.claim(ffn.w2.weight))]
    if tp is None:
        dh2 = G.linear_dgrad(d13, engine.shadow(ffn.w1.weight, 2 * dff))
    elif tp.can_fuse(d):   # column-parallel input gradient: GEMM + sum over ranks, one kernel
        dh2 = tp.gemm_reduce_bf16(d13, engine.shadow(ffn.w1.weight, 2 * dff))
    else:
        dh2 = tp.reduce_bf16(G.linear_dgrad(d13, engine.shadow(ffn.w1.weight, 2 * dff),
                                            tp.partial(M, d)))
    wgrads.append((d13, h2, engine.grad_view(ffn.w1.weight, 2 * dff),
                   engine.claim(ffn.w1.weight, ffn.w3.weight)))
    acc = engine.claim(layer.ffn_norm.weight)
    dres2, dres2_bf16 = K.rmsnorm_bwd(dh2, x_mid, layer.ffn_norm.weight, rstd2, dres,
                                      engine.grad_view(layer.ffn_norm.weight), acc, want_bf16=True)
    # ---- attention half
    d_attn = G.linear_dgrad(dres2_bf16, engine.shadow(attn_p.output_proj.weight))
    wgrads.append((dres2_bf16, attn, engine.grad_view(attn_p.output_proj.weight),
                   engine.claim(attn_p.output_proj.weight)))
    dqkv = torch.empty_like(qkv)
    heads = qkv.view(B, T, 3, H, dk)
    dheads = dqkv.view(B, T, 3, H, dk)
    q, k, v = (heads[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    dq, dkk, dv = (dheads[:, :, i].permute(0, 2, 1, 3) for i in range(3))
    as_heads = lambda t: t.view(B, T, H, dk).permute(0, 2, 1, 3)
    mask = flash.causal_mask(d_out.device, T)
    flash.flash_bwd(q, k, v, as_heads(attn), as_heads(d_attn), lse, dq, dkk, dv, mask, dk ** -0.5,
                    rope=(engine.cos, engine.sin))   # dq, dk come back un-rotated
    if tp is None:
        dh1 = G.linear_dgrad(dqkv, engine.shadow(attn_p.q_proj.weight, 3 * aw))
    elif tp.can_fuse(d):
        dh1 = tp.gemm_reduce_bf16(dqkv, engine.shadow(attn_p.q_proj.weight, 3 * aw))
    else:
        dh1 = tp.reduce_bf16(G.linear_dgrad(dqkv, engine.shadow(attn_p.q_proj.weight, 3 * aw),
                                            tp.partial(M, d)))
    wgrads.append((dqkv, h1, engine.grad_view(attn_p.q_proj.weight, 3 * aw),
                   engine.claim(attn_p.q_proj.weight, attn_p.k_proj.weight, attn_p.v_proj.weight)))
    G.wgrad_grouped(wgrads)
    acc = engine.claim(layer.attn_norm.weight)
    dx, dx_bf16 = K.rmsnorm_bwd(dh1, x2, layer.attn_norm.weight, rstd1, dres2,
                                engine.grad_view(layer.attn_norm.weight), acc, want_bf16=True)
    engine._bf16_alias = (dx.data_ptr(), dx_bf16)
    if engine.on_block_backward is not None:
        engine.on_block_backward(engine.layer_ranges[index][0])
    return dx.view(B, T, d)


def head_logits(engine: FusedEngine, x: torch.Tensor):
    model = engine.model
    x2 = x.reshape(-1, engine.d_model)
    h, rstd = K.rmsnorm(x2, model.ln_final.weight, model.ln_final.eps)
    ld = _round_up(engine.vocab, 8)
    logits = torch.empty(x2.shape[0], ld, dtype=torch.bfloat16, device=x.device)
    G.linear_fwd(h, engine.shadow(model.lm_head.weight), logits)
    return logits, (x2, h, rstd)


def head_backward(engine: FusedEngine, saved, dlogits: torch.Tensor) -> torch.Tensor:
    """``dlogits`` is bf16 ``[M, ld]`` (columns beyond the vocabulary are ignored)."""
    model = engine.model
    x2, h, rstd = saved
    V = engine.vocab
    w = engine.shadow(model.lm_head.weight)
    dl = dlogits[:, :V] if dlogits.shape[1] != V else dlogits
    dh = torch.empty_like(h)
    epi = G.GemmEpilogue(kind=G.EPI_BF16, out=dh.data_ptr(), ldo=dh.stride(0))
    G.gemm(dl, w, h.shape[0], engine.d_model, V, epi, b_mn=True)
    acc = engine.claim(model.lm_head.weight)
    grad = engine.grad_view(model.lm_head.weight)
    epi = G.GemmEpilogue(kind=G.EPI_F32, beta=int(acc), out=grad.data_ptr(), ldo=grad.stride(0))
    G.gemm(dl, h, V, engine.d_model, h.shape[0], epi, a_mn=True, b_mn=True)
    acc = engine.claim(model.ln_final.weight)
    dx, dx_bf16 = K.rmsnorm_bwd(dh, x2, model.ln_final.weight, rstd, None,
                                engine.grad_view(model.ln_final.weight), acc, want_bf16=True)
    engine._bf16_alias = (dx.data_ptr(), dx_bf16)
    if engine.on_block_backward is not None:
        engine.on_block_backward(engine.head_offset)
    return dx


# ------------------------------------------------------------ autograd nodes --
class _Embed(torch.autograd.Function):
    @staticmethod
    def forward(ctx, weight, ids, engine):
        ctx.engine = engine
        ctx.save_for_backward(ids)
        ctx.weight = weight
        return K.embedding(engine.embedding_table(), ids)

    @staticmethod
    def backward(ctx, grad):
        (ids,) = ctx.saved_tensors
        engine, weight = ctx.engine, ctx.weight
        accumulate = engine.claim(weight)
        view = engine.grad_view(weight)
        if not K.embedding_bwd(grad, ids, view, accumulate):    # more tokens than the kernel takes
            dense = torch.ops.aten.embedding_dense_backward(
                grad.reshape(-1, grad.shape[-1]), ids.reshape(-1), weight.shape[0], -1, False)
            if accumulate:
                view.add_(dense)
            else:
                view.copy_(dense)
        if engine.on_block_backward is not None:
            engine.on_block_backward(0)
        return None, None, None


class _Block(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, engine, index, B, T, recompute):
        out, saved = block_forward(engine, index, x, B, T)
        ctx.engine, ctx.index, ctx.B, ctx.T, ctx.recompute = engine, index, B, T, recompute
        if recompute:
            ctx.save_for_backward(x)
        else:
            ctx.save_for_backward(*saved)
        return out

    @staticmethod
    def backward(ctx, grad):
        ctx.engine.prepare_block(ctx.index, True)
        if ctx.recompute:
            (x,) = ctx.saved_tensors
            saved = block_forward(ctx.engine, ctx.index, x, ctx.B, ctx.T)[1]
        else:
            saved = ctx.saved_tensors
        dx = block_backward(ctx.engine, ctx.index, saved, grad, ctx.B, ctx.T)
        return dx, None, None, None, None, None


class _Logits(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, engine):
        logits, saved = head_logits(engine, x)
        ctx.engine = engine
        ctx.shape = x.shape
        ctx.save_for_backward(*saved)
        return logits

    @staticmethod
    def backward(ctx, grad):
        grad = grad.contiguous() if not grad.is_contiguous() else grad
        dx = head_backward(ctx.engine, ctx.saved_tensors, grad.to(torch.bfloat16))
        return dx.view(ctx.shape), None


class _HeadLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, targets, engine, scale):
        logits, saved = head_logits(engine, x)
        rows = logits.shape[0]
        # The logit gradient overwrites the logits: one pass produces both.
        losses = K.cross_entropy_rows(logits, targets, engine.vocab, logits, scale / rows)
        ctx.engine, ctx.shape = engine, x.shape
        ctx.save_for_backward(logits, *saved)
        return losses.sum() * (scale / rows)

    @staticmethod
    def backward(ctx, grad):
        dlogits, *saved = ctx.saved_tensors
        K.scale_bf16_unless_one(dlogits, grad)    # the incoming gradient is normally 1
        dx = head_backward(ctx.engine, saved, dlogits)
        return dx.view(ctx.shape), None, None, None
