// One transformer block, forward or backward, as a single call into the library.
//
// The fused engine used to drive every kernel of a block from Python: 7 launches
// forward and 11 backward per layer, each with its own tensor allocations, views
// and ctypes call.  At 324M parameters that host work (≈15 ms per microbatch)
// equalled the GPU time of the kernels themselves, so the step was bound by the
// interpreter.  These two entry points issue the same kernels, in the same order
// and with the same arguments, from C++: Python allocates one activation buffer
// and one scratch buffer per block and makes one call.
//
// The arithmetic is that of the reference block (src/llmlab/model/transformer.py:
// 33-47: x + attn(norm(x)), then x + ffn(norm(x))) with the epilogue fusions of
// gemm.cu; gradients follow models/fused.py:block_backward, which remains the
// implementation for engines the runner does not cover.  Under tensor
// parallelism (SflBlockArgs::tp_pool) the four products whose reduction dimension
// is sharded are issued as GEMM + all-reduce in one kernel (sfl_gemm_tp_reduce).
#include <cuda_runtime.h>
#include <stdint.h>

#include "sfl.h"

namespace {

constexpr long kAlign = 256;

long round_up(long bytes) { return (bytes + kAlign - 1) / kAlign * kAlign; }

struct Dims {
  long M, d, aw, dff;
  int B, T, H, dk;
};

Dims dims_of(const SflBlockArgs& a) {
  Dims s;
  s.B = a.batch;
  s.T = a.seq_len;
  s.H = a.heads;
  s.dk = a.head_dim;
  s.M = static_cast<long>(a.batch) * a.seq_len;
  s.d = a.d_model;
  s.aw = static_cast<long>(a.heads) * a.head_dim;
  s.dff = a.d_ff;
  return s;
}

// Activations kept from forward to backward, carved out of one buffer.
struct Saved {
  uint8_t *h1, *rstd1, *qkv, *attn, *lse, *x_mid, *rstd2, *h2, *a13, *g;
  long bytes;
};

Saved carve_saved(const Dims& s, void* base) {
  uint8_t* p = static_cast<uint8_t*>(base);
  long off = 0;
  auto take = [&](long bytes) {
    uint8_t* ptr = p == nullptr ? nullptr : p + off;
    off += round_up(bytes);
    return ptr;
  };
  Saved v;
  v.h1 = take(s.M * s.d * 2);
  v.rstd1 = take(s.M * 4);
  v.qkv = take(s.M * 3 * s.aw * 2);
  v.attn = take(s.M * s.aw * 2);
  v.lse = take(static_cast<long>(s.B) * s.H * s.T * 4);
  v.x_mid = take(s.M * s.d * 4);
  v.rstd2 = take(s.M * 4);
  v.h2 = take(s.M * s.d * 2);
  v.a13 = take(s.M * 2 * s.dff * 2);
  v.g = take(s.M * s.dff * 2);
  v.bytes = off;
  return v;
}

// Temporaries of the backward pass.
struct Scratch {
  uint8_t *dres_bf16, *d13, *dh2, *dres2, *dres2_bf16, *d_attn, *dqkv, *delta, *dh1, *partial,
      *partial1;
  long bytes;
};

Scratch carve_scratch(const Dims& s, void* base) {
  uint8_t* p = static_cast<uint8_t*>(base);
  long off = 0;
  auto take = [&](long bytes) {
    uint8_t* ptr = p == nullptr ? nullptr : p + off;
    off += round_up(bytes);
    return ptr;
  };
  Scratch v;
  v.dres_bf16 = take(s.M * s.d * 2);
  v.d13 = take(s.M * 2 * s.dff * 2);
  v.dh2 = take(s.M * s.d * 2);
  v.dres2 = take(s.M * s.d * 4);
  v.dres2_bf16 = take(s.M * s.d * 2);
  v.d_attn = take(s.M * s.aw * 2);
  v.dqkv = take(s.M * 3 * s.aw * 2);
  v.delta = take(static_cast<long>(s.B) * s.H * s.T * 4);
  v.dh1 = take(s.M * s.d * 2);
  v.partial = take(static_cast<long>(sfl_rmsnorm_bwd_blocks(static_cast<int>(s.M))) * s.d * 4);
  v.partial1 = take(static_cast<long>(sfl_rmsnorm_bwd_blocks(static_cast<int>(s.M))) * s.d * 4);
  v.bytes = off;
  return v;
}

bool shape_ok(const SflBlockArgs& a) {
  return a.batch > 0 && a.seq_len > 0 && a.d_model > 0 && a.heads > 0 && a.d_ff > 0 &&
         (a.head_dim == 64 || a.head_dim == 128) && a.d_model % 8 == 0 && a.d_ff % 8 == 0 &&
         static_cast<long>(a.batch) * a.seq_len < (1l << 31);
}

SflAttnTensor head_view(void* base, long column, long row_pitch, const Dims& s) {
  SflAttnTensor t;
  t.ptr = static_cast<uint8_t*>(base) + column * 2;
  t.stride_b = static_cast<long>(s.T) * row_pitch;
  t.stride_h = s.dk;
  t.stride_t = row_pitch;
  return t;
}

SflGemmEpilogue epilogue(int kind, void* out, long ldo, int* status) {
  SflGemmEpilogue e{};
  e.kind = kind;
  e.out = out;
  e.ldo = ldo;
  e.status = status;
  return e;
}

// Epilogue kinds of sfl_gemm_bf16 (gemm.cu).
enum { kBf16 = 0, kF32 = 1, kResid = 2, kRope = 3, kSwiglu = 4, kSwigluBwd = 5 };

#define SFL_TRY(call)              \
  do {                             \
    const int rc_ = (call);        \
    if (rc_ != 0) return rc_;      \
  } while (0)

}  // namespace

extern "C" long sfl_block_saved_bytes(const SflBlockArgs* a) {
  if (a == nullptr || !shape_ok(*a)) return -1;
  return carve_saved(dims_of(*a), nullptr).bytes;
}

extern "C" long sfl_block_scratch_bytes(const SflBlockArgs* a) {
  if (a == nullptr || !shape_ok(*a)) return -1;
  return carve_scratch(dims_of(*a), nullptr).bytes;
}

namespace {

// Local base of a fused product's result buffer.
uint8_t* tp_local(const SflTpFuse* t) {
  return t == nullptr || t->rank < 0 || t->rank >= 8 ? nullptr
                                                     : static_cast<uint8_t*>(t->out[t->rank]);
}

}  // namespace

extern "C" int sfl_block_forward(const SflBlockArgs* a, void* stream) {
  if (a == nullptr || !shape_ok(*a) || a->x == nullptr || a->saved == nullptr ||
      a->mask == nullptr)
    return -2;
  const bool tp = a->tp_pool != nullptr;
  if (!tp && a->x_out == nullptr) return -2;
  if (tp && tp_local(a->tp_pool) == nullptr) return -2;
  const Dims s = dims_of(*a);
  Saved v = carve_saved(s, a->saved);
  float* x_out = a->x_out;
  if (tp) {
    v.x_mid = tp_local(a->tp_pool) + a->tp_off_mid;
    x_out = reinterpret_cast<float*>(tp_local(a->tp_pool) + a->tp_off_out);
  }
  const int M = static_cast<int>(s.M);
  const int d = static_cast<int>(s.d), aw = static_cast<int>(s.aw), dff = static_cast<int>(s.dff);

  // attention half: x_mid = x + Wo attn(rope(Wqkv norm(x)))
  SFL_TRY(sfl_rmsnorm_fwd(a->x, a->norm1, v.h1, reinterpret_cast<float*>(v.rstd1), M, d, a->eps1,
                          stream));
  SflGemmEpilogue rope = epilogue(kRope, v.qkv, 3 * s.aw, a->status);
  rope.rope_cos = a->rope_cos;
  rope.rope_sin = a->rope_sin;
  rope.rope_T = s.T;
  rope.rope_cols = 2 * aw;
  rope.head_dim = s.dk;
  SFL_TRY(sfl_gemm_bf16(v.h1, s.d, 0, a->wqkv, s.d, 0, M, 3 * aw, d, &rope, 0, 0, stream));
  const SflAttnTensor q = head_view(v.qkv, 0, 3 * s.aw, s);
  const SflAttnTensor k = head_view(v.qkv, s.aw, 3 * s.aw, s);
  const SflAttnTensor vv = head_view(v.qkv, 2 * s.aw, 3 * s.aw, s);
  const SflAttnTensor o = head_view(v.attn, 0, s.aw, s);
  SFL_TRY(sfl_attn_fwd(&q, &k, &vv, &o, reinterpret_cast<float*>(v.lse), s.B, s.H, s.T, s.dk,
                       a->attn_scale, a->mask, 0, a->status, stream));
  if (tp) {
    SFL_TRY(sfl_gemm_tp_reduce(v.attn, s.aw, a->wo, s.aw, 0, M, d, aw, a->tp_pool, a->tp_off_mid, 0,
                               a->x, s.d, a->tp_slot[0], a->tp_epoch[0], a->tp_tile_epoch[0],
                               a->status, stream));
  } else {
    SflGemmEpilogue resid = epilogue(kResid, v.x_mid, s.d, a->status);
    resid.aux = a->x;
    resid.ldaux = s.d;
    SFL_TRY(sfl_gemm_bf16(v.attn, s.aw, 0, a->wo, s.aw, 0, M, d, aw, &resid, 0, 0, stream));
  }

  // feed-forward half: x_out = x_mid + W2 (silu(W1 h) * W3 h), h = norm(x_mid)
  SFL_TRY(sfl_rmsnorm_fwd(reinterpret_cast<const float*>(v.x_mid), a->norm2, v.h2,
                          reinterpret_cast<float*>(v.rstd2), M, d, a->eps2, stream));
  SflGemmEpilogue gate = epilogue(kSwiglu, v.g, s.dff, a->status);
  gate.out2 = v.a13;
  gate.ldo2 = 2 * s.dff;
  gate.dual_offset = dff;
  gate.dual_rows = 2 * dff;
  SFL_TRY(sfl_gemm_bf16(v.h2, s.d, 0, a->w13, s.d, 0, M, dff, d, &gate, 0, 0, stream));
  if (tp) {
    SFL_TRY(sfl_gemm_tp_reduce(v.g, s.dff, a->w2, s.dff, 0, M, d, dff, a->tp_pool, a->tp_off_out, 0,
                               reinterpret_cast<const float*>(v.x_mid), s.d, a->tp_slot[1],
                               a->tp_epoch[1], a->tp_tile_epoch[1], a->status, stream));
  } else {
    SflGemmEpilogue out = epilogue(kResid, x_out, s.d, a->status);
    out.aux = v.x_mid;
    out.ldaux = s.d;
    SFL_TRY(sfl_gemm_bf16(v.g, s.dff, 0, a->w2, s.dff, 0, M, d, dff, &out, 0, 0, stream));
  }
  return 0;
}

extern "C" int sfl_block_backward(const SflBlockArgs* a, void* stream) {
  if (a == nullptr || !shape_ok(*a) || a->x == nullptr || a->saved == nullptr ||
      a->mask == nullptr || a->d_out == nullptr || a->dx == nullptr || a->dx_bf16 == nullptr ||
      a->scratch == nullptr || a->g_wqkv == nullptr || a->g_wo == nullptr ||
      a->g_w13 == nullptr || a->g_w2 == nullptr || a->g_norm1 == nullptr ||
      a->g_norm2 == nullptr)
    return -2;
  const bool tp = a->tp_pool != nullptr;
  if (tp && (tp_local(a->tp_pool) == nullptr || tp_local(a->tp_small) == nullptr)) return -2;
  const Dims s = dims_of(*a);
  Saved v = carve_saved(s, a->saved);
  Scratch t = carve_scratch(s, a->scratch);
  if (tp) {
    v.x_mid = tp_local(a->tp_pool) + a->tp_off_mid;
    t.dh2 = t.dh1 = tp_local(a->tp_small);  // used one after the other
  }
  const int M = static_cast<int>(s.M);
  const int d = static_cast<int>(s.d), aw = static_cast<int>(s.aw), dff = static_cast<int>(s.dff);
  const int blocks = sfl_rmsnorm_bwd_blocks(M);
  // weight-gradient partials of the two norms; both are folded by one launch at the end
  float* partial = reinterpret_cast<float*>(t.partial);
  float* partial1 = reinterpret_cast<float*>(t.partial1);

  const void* dres_bf16 = a->d_out_bf16;
  if (dres_bf16 == nullptr) {
    SFL_TRY(sfl_cast_f32_to_bf16(a->d_out, t.dres_bf16, s.M * s.d, stream));
    dres_bf16 = t.dres_bf16;
  }

  // ---- feed-forward half
  SflGemmEpilogue act = epilogue(kSwigluBwd, t.d13, 2 * s.dff, a->status);
  act.aux = v.a13;
  act.ldaux = 2 * s.dff;
  SFL_TRY(sfl_gemm_bf16(dres_bf16, s.d, 0, a->w2, s.dff, 1, M, dff, d, &act, 0, 0, stream));
  SflGemmEpilogue plain = epilogue(kBf16, t.dh2, s.d, a->status);
  if (tp) {
    SFL_TRY(sfl_gemm_tp_reduce(t.d13, 2 * s.dff, a->w13, s.d, 1, M, d, 2 * dff, a->tp_small, 0, 1,
                               nullptr, 0, a->tp_slot[0], a->tp_epoch[0], a->tp_tile_epoch[0],
                               a->status, stream));
  } else {
    SFL_TRY(sfl_gemm_bf16(t.d13, 2 * s.dff, 0, a->w13, s.d, 1, M, d, 2 * dff, &plain, 0, 0,
                          stream));
  }
  SFL_TRY(sfl_rmsnorm_bwd(t.dh2, reinterpret_cast<const float*>(v.x_mid), a->norm2,
                          reinterpret_cast<const float*>(v.rstd2), a->d_out,
                          reinterpret_cast<float*>(t.dres2), t.dres2_bf16, partial, M, d, stream));

  // ---- attention half
  plain = epilogue(kBf16, t.d_attn, s.aw, a->status);
  SFL_TRY(sfl_gemm_bf16(t.dres2_bf16, s.d, 0, a->wo, s.aw, 1, M, aw, d, &plain, 0, 0, stream));
  const SflAttnTensor q = head_view(v.qkv, 0, 3 * s.aw, s);
  const SflAttnTensor k = head_view(v.qkv, s.aw, 3 * s.aw, s);
  const SflAttnTensor vv = head_view(v.qkv, 2 * s.aw, 3 * s.aw, s);
  const SflAttnTensor o = head_view(v.attn, 0, s.aw, s);
  const SflAttnTensor d_o = head_view(t.d_attn, 0, s.aw, s);
  const SflAttnTensor dq = head_view(t.dqkv, 0, 3 * s.aw, s);
  const SflAttnTensor dk = head_view(t.dqkv, s.aw, 3 * s.aw, s);
  const SflAttnTensor dv = head_view(t.dqkv, 2 * s.aw, 3 * s.aw, s);
  SFL_TRY(sfl_attn_bwd(&q, &k, &vv, &o, &d_o, reinterpret_cast<const float*>(v.lse),
                       reinterpret_cast<float*>(t.delta), &dq, &dk, &dv, s.B, s.H, s.T, s.dk,
                       a->attn_scale, a->mask, 0, a->status, a->rope_cos, a->rope_sin, stream));
  if (tp) {
    SFL_TRY(sfl_gemm_tp_reduce(t.dqkv, 3 * s.aw, a->wqkv, s.d, 1, M, d, 3 * aw, a->tp_small, 0, 1,
                               nullptr, 0, a->tp_slot[1], a->tp_epoch[1], a->tp_tile_epoch[1],
                               a->status, stream));
  } else {
    plain = epilogue(kBf16, t.dh1, s.d, a->status);
    SFL_TRY(sfl_gemm_bf16(t.dqkv, 3 * s.aw, 0, a->wqkv, s.d, 1, M, d, 3 * aw, &plain, 0, 0,
                          stream));
  }

  // ---- the four weight gradients as one grouped launch
  SflWgradProblem w[4] = {
      {dres_bf16, s.d, v.g, s.dff, a->g_w2, s.dff, d, dff, M, a->acc_w2},
      {t.d13, 2 * s.dff, v.h2, s.d, a->g_w13, s.d, 2 * dff, d, M, a->acc_w13},
      {t.dres2_bf16, s.d, v.attn, s.aw, a->g_wo, s.aw, d, aw, M, a->acc_wo},
      {t.dqkv, 3 * s.aw, v.h1, s.d, a->g_wqkv, s.d, 3 * aw, d, M, a->acc_wqkv},
  };
  SFL_TRY(sfl_gemm_wgrad_grouped(w, 4, a->status, stream));

  SFL_TRY(sfl_rmsnorm_bwd(t.dh1, a->x, a->norm1, reinterpret_cast<const float*>(v.rstd1),
                          reinterpret_cast<const float*>(t.dres2), a->dx, a->dx_bf16, partial1, M,
                          d, stream));
  SFL_TRY(sfl_rmsnorm_dw_reduce2(partial, a->g_norm2, a->acc_norm2, partial1, a->g_norm1,
                                 a->acc_norm1, blocks, d, stream));
  return 0;
}
