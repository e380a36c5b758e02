// Persistent warp-specialised bf16 GEMM for sm_100a.
//
//   D[M,N] = A[M,K] * B[N,K]^T      (fp32 accumulation in tensor memory)
//
// One CTA per SM walks output tiles of 128 x BN.  Warp 0 streams operand tiles
// into a shared-memory ring with TMA, warp 1 issues tcgen05.mma into one of two
// TMEM accumulator stages, warps 2-9 drain the other stage through a fused
// epilogue (two warps per TMEM lane quarter, alternating column chunks), so the
// epilogue of tile i overlaps the main loop of tile i+1.
//
// Either operand may be "K-major" (reduction dimension contiguous in memory) or
// "MN-major" (the M/N dimension contiguous), which lets one kernel serve the
// forward (x W^T), input-gradient (dy W) and weight-gradient (dy^T x) products
// of a linear layer without transposing anything in memory.  The reference
// computes these through einsum/cuBLAS (src/llmlab/model/layers.py:35).
//
// Fused epilogues replace the reference's separate elementwise kernels:
//   EPI_BF16        plain bf16 store
//   EPI_F32         fp32 store or accumulate (weight gradients, beta in {0,1})
//   EPI_RESID       fp32 residual stream update  out = resid + bf16(acc)
//                   (src/llmlab/model/transformer.py:46-47)
//   EPI_ROPE        bf16 store of a fused q|k|v projection with interleaved-pair
//                   rotary embedding on the q and k columns
//                   (src/llmlab/model/attention.py:44-58)
//   EPI_SWIGLU      dual accumulator (w1 x | w3 x): stores both and
//                   silu(w1 x) * w3 x   (src/llmlab/model/layers.py:114-115)
//   EPI_SWIGLU_BWD  acc = d(silu(a1)*a3); stores d a1 | d a3
//
// Epilogue data path.  When the output (and auxiliary) matrices satisfy TMA's
// alignment rules, each epilogue warp owns a private strip of shared memory:
// accumulator rows come out of TMEM one row per thread, are converted and
// written into a 128-byte-swizzled 32-row staging tile, and one lane hands the
// tile to the TMA engine (bulk tensor store, or bulk reduce-add for beta = 1), so
// global traffic is fully coalesced and asynchronous.  Auxiliary operands
// (the residual stream, the saved SwiGLU pre-activations) arrive the same way,
// one chunk ahead of their use.  Matrices that break the alignment rules take
// the direct path: each thread stores its own row.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdlib.h>

#include <map>
#include <mutex>
#include <tuple>

#include "comm.cuh"
#include "launch.cuh"
#include "ptx.cuh"
#include "sfl.h"
#include "tensormap.cuh"

namespace sfl {

enum Epilogue : int {
  EPI_BF16 = 0,
  EPI_F32 = 1,
  EPI_RESID = 2,
  EPI_ROPE = 3,
  EPI_SWIGLU = 4,
  EPI_SWIGLU_BWD = 5,
};

struct GemmParams {
  int M, N, K;
  int num_m_tiles, num_n_tiles;
  void* out;
  long ldo;
  void* out2;
  long ldo2;
  const void* aux;
  long ldaux;
  int beta;
  // rotary embedding
  const float* rope_cos;  // [T, head_dim/2]
  const float* rope_sin;
  int rope_T;        // sequence length: position = row % rope_T
  int rope_cols;     // columns [0, rope_cols) are rotated (q and k)
  int head_dim;
  // SwiGLU
  int dual_offset;   // row offset of the second weight matrix inside B
  int* status;
};

constexpr int BM = 128;
constexpr int BK = 64;
constexpr int kEpiWarps = 8;  // two per TMEM lane quarter
constexpr int kThreads = 64 + 32 * kEpiWarps;
constexpr int kTileABytes = BM * BK * 2;

// Per-epilogue shape of the staged (TMA) data path: accumulator columns handled
// per step, and how many 4 KB (32 rows x 128 B) tiles each epilogue warp owns.
// Auxiliary inputs are loaded into the very tiles the results are stored from.
template <int EPI>
struct EpiTraits;
template <> struct EpiTraits<EPI_BF16> { static constexpr int kChunk = 64, kTiles = 1; };
template <> struct EpiTraits<EPI_F32> { static constexpr int kChunk = 32, kTiles = 1; };
template <> struct EpiTraits<EPI_RESID> { static constexpr int kChunk = 32, kTiles = 1; };
template <> struct EpiTraits<EPI_ROPE> { static constexpr int kChunk = 64, kTiles = 1; };
template <> struct EpiTraits<EPI_SWIGLU> { static constexpr int kChunk = 64, kTiles = 1; };
template <> struct EpiTraits<EPI_SWIGLU_BWD> { static constexpr int kChunk = 64, kTiles = 2; };

constexpr int kEpiTileBytes = 32 * 128;
constexpr int kMaxSmemBytes = 232448;  // 227 KB opt-in limit per CTA

template <int BN, int EPI, bool STAGED>
struct GemmConfig {
  static constexpr int kTileBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kTileABytes + kTileBBytes;
  static constexpr int kEpiWarpBytes = STAGED ? EpiTraits<EPI>::kTiles * kEpiTileBytes : 0;
  static constexpr int kEpiBytes = kEpiWarps * kEpiWarpBytes;
  static constexpr int kFixedBytes = 1024 /*align*/ + 512 /*barriers*/ + kEpiBytes;
  static constexpr int kWantStages = (BN == 256) ? 4 : 6;
  static constexpr int kFitStages = (kMaxSmemBytes - kFixedBytes) / kStageBytes;
  static constexpr int kStages = kFitStages < kWantStages ? kFitStages : kWantStages;
  static_assert(kStages >= 3, "operand ring too shallow");
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kSmemBytes = kStages * kStageBytes + kFixedBytes;
};

struct EpiMaps {
  // Role of each map per epilogue:
  //   BF16 / F32 / ROPE : m[0] output
  //   RESID             : m[0] output, m[1] residual input
  //   SWIGLU            : m[0] gated output, m[1] w1 x, m[2] w3 x
  //   SWIGLU_BWD        : m[0] d a1, m[1] d a3, m[2] a1, m[3] a3
  CUtensorMap m[4];
};

struct __align__(8) GemmBarriers {
  uint64_t full[8];
  uint64_t empty[8];
  uint64_t tmem_full[2];
  uint64_t tmem_empty[2];
  uint64_t aux_full[kEpiWarps];  // per epilogue warp: its auxiliary tile(s) have landed
  uint32_t tmem_base;
  int abort;
};

// Gives up after about two seconds by the global timer (an iteration count alone is no bound:
// mbarrier.try_wait may suspend the thread for an implementation-defined time per call).
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort) {
  unsigned long long started = 0;
  for (uint32_t spin = 0; spin < (1u << 26); ++spin) {
    if (mbar_try_wait(bar, parity)) return true;
    if (spin > 2048) {
      __nanosleep(256);
      if (*abort) return false;
      if ((spin & 1023) == 0) {
        unsigned long long now;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
        if (started == 0) started = now;
        if (now - started > 2000000000ull) return false;
      }
    }
  }
  return false;
}

// ------------------------------------------------------------- epilogues ----
// silu(a) * b and its derivatives, with the fast reciprocal: results are rounded
// to bf16 afterwards, far coarser than the two-ulp error of the approximation.
// sigmoid(a) = (1 + tanh(a / 2)) / 2: one special-function instruction (tanh.approx,
// relative error 2^-11, far inside the bf16 rounding of the results) instead of the two of
// 1 / (1 + exp(-a)); the SwiGLU epilogues are bound by that unit.
__device__ __forceinline__ float fast_sigmoid(float a) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * a));
  return fmaf(t, 0.5f, 0.5f);
}

template <int EPI>
struct EpilogueOp;

__device__ __forceinline__ void store_bf16_row(__nv_bfloat16* dst, const float (&v)[32], int col0,
                                               int N, bool vec_ok) {
  if (vec_ok && col0 + 32 <= N) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 q;
      q.x = pack_bf16(v[8 * j + 0], v[8 * j + 1]);
      q.y = pack_bf16(v[8 * j + 2], v[8 * j + 3]);
      q.z = pack_bf16(v[8 * j + 4], v[8 * j + 5]);
      q.w = pack_bf16(v[8 * j + 6], v[8 * j + 7]);
      *reinterpret_cast<uint4*>(dst + 8 * j) = q;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j < N) dst[j] = __float2bfloat16_rn(v[j]);
  }
}

template <>
struct EpilogueOp<EPI_BF16> {
  static __device__ __forceinline__ void apply(const GemmParams& p, int row, int col0,
                                               float (&v)[32], float (&)[32]) {
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + static_cast<long>(row) * p.ldo + col0;
    store_bf16_row(dst, v, col0, p.N, (p.ldo & 7) == 0);
  }
};

template <>
struct EpilogueOp<EPI_F32> {
  static __device__ __forceinline__ void apply(const GemmParams& p, int row, int col0,
                                               float (&v)[32], float (&)[32]) {
    float* dst = static_cast<float*>(p.out) + static_cast<long>(row) * p.ldo + col0;
    if ((p.ldo & 3) == 0 && col0 + 32 <= p.N) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 q = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        if (p.beta) {
          float4 o = *reinterpret_cast<const float4*>(dst + 4 * j);
          q.x += o.x; q.y += o.y; q.z += o.z; q.w += o.w;
        }
        *reinterpret_cast<float4*>(dst + 4 * j) = q;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) dst[j] = p.beta ? dst[j] + v[j] : v[j];
    }
  }
};

template <>
struct EpilogueOp<EPI_RESID> {
  static __device__ __forceinline__ void apply(const GemmParams& p, int row, int col0,
                                               float (&v)[32], float (&)[32]) {
    float* dst = static_cast<float*>(p.out) + static_cast<long>(row) * p.ldo + col0;
    const float* res = static_cast<const float*>(p.aux) + static_cast<long>(row) * p.ldaux + col0;
    if ((p.ldo & 3) == 0 && (p.ldaux & 3) == 0 && col0 + 32 <= p.N) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float4 r = *reinterpret_cast<const float4*>(res + 4 * j);
        r.x += bf16_round(v[4 * j]);
        r.y += bf16_round(v[4 * j + 1]);
        r.z += bf16_round(v[4 * j + 2]);
        r.w += bf16_round(v[4 * j + 3]);
        *reinterpret_cast<float4*>(dst + 4 * j) = r;
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col0 + j < p.N) dst[j] = res[j] + bf16_round(v[j]);
    }
  }
};

template <>
struct EpilogueOp<EPI_ROPE> {
  static __device__ __forceinline__ void apply(const GemmParams& p, int row, int col0,
                                               float (&v)[32], float (&)[32]) {
    if (col0 < p.rope_cols) {
      // A 32-column chunk never straddles a head because head_dim is a multiple
      // of 32 here (checked on the host); pairs (2i, 2i+1) are rotated together.
      const int pos = row % p.rope_T;
      const int half = p.head_dim >> 1;
      const int pair0 = (col0 % p.head_dim) >> 1;
      const float* cs = p.rope_cos + static_cast<long>(pos) * half + pair0;
      const float* sn = p.rope_sin + static_cast<long>(pos) * half + pair0;
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        // The projection output is bf16 before the rotation, as in the reference.
        const float xe = bf16_round(v[2 * j]);
        const float xo = bf16_round(v[2 * j + 1]);
        const float c = cs[j];
        const float s = sn[j];
        v[2 * j] = xe * c - xo * s;
        v[2 * j + 1] = xe * s + xo * c;
      }
    }
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + static_cast<long>(row) * p.ldo + col0;
    store_bf16_row(dst, v, col0, p.N, (p.ldo & 7) == 0);
  }
};

template <>
struct EpilogueOp<EPI_SWIGLU> {
  // v = w1 x chunk, w = w3 x chunk (same columns)
  static __device__ __forceinline__ void apply(const GemmParams& p, int row, int col0,
                                               float (&v)[32], float (&w)[32]) {
    __nv_bfloat16* a13 = static_cast<__nv_bfloat16*>(p.out2) + static_cast<long>(row) * p.ldo2;
    const bool vec2 = (p.ldo2 & 7) == 0 && (p.N & 7) == 0;
    store_bf16_row(a13 + col0, v, col0, p.N, vec2);
    store_bf16_row(a13 + p.N + col0, w, col0, p.N, vec2);
    float g[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float a = bf16_round(v[j]);
      const float b = bf16_round(w[j]);
      g[j] = a * fast_sigmoid(a) * b;
    }
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + static_cast<long>(row) * p.ldo + col0;
    store_bf16_row(dst, g, col0, p.N, (p.ldo & 7) == 0);
  }
};

// Loads 32 consecutive bf16 values of a row as fp32 (vectorised when aligned).
__device__ __forceinline__ void load_bf16_row(const __nv_bfloat16* src, float (&v)[32], int col0,
                                              int N, bool vec_ok) {
  if (vec_ok && col0 + 32 <= N) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint4 q = *reinterpret_cast<const uint4*>(src + 8 * j);
      const float2 a = unpack_bf16(q.x), b = unpack_bf16(q.y), c = unpack_bf16(q.z),
                   d = unpack_bf16(q.w);
      v[8 * j + 0] = a.x; v[8 * j + 1] = a.y; v[8 * j + 2] = b.x; v[8 * j + 3] = b.y;
      v[8 * j + 4] = c.x; v[8 * j + 5] = c.y; v[8 * j + 6] = d.x; v[8 * j + 7] = d.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = col0 + j < N ? __bfloat162float(src[j]) : 0.f;
  }
}

template <>
struct EpilogueOp<EPI_SWIGLU_BWD> {
  static __device__ __forceinline__ void apply(const GemmParams& p, int row, int col0,
                                               float (&v)[32], float (&)[32]) {
    const __nv_bfloat16* a13 =
        static_cast<const __nv_bfloat16*>(p.aux) + static_cast<long>(row) * p.ldaux;
    const bool vec_in = (p.ldaux & 7) == 0 && (p.N & 7) == 0;
    float a1[32], a3[32];
    load_bf16_row(a13 + col0, a1, col0, p.N, vec_in);
    load_bf16_row(a13 + p.N + col0, a3, col0, p.N, vec_in);
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      const float a = a1[j];
      const float dg = bf16_round(v[j]);
      const float sig = fast_sigmoid(a);
      const float silu = a * sig;
      a1[j] = dg * a3[j] * (sig + silu * (1.0f - sig));  // d a1
      a3[j] = dg * silu;                                  // d a3
    }
    __nv_bfloat16* dst = static_cast<__nv_bfloat16*>(p.out) + static_cast<long>(row) * p.ldo;
    const bool vec = (p.ldo & 7) == 0 && (p.N & 7) == 0;
    store_bf16_row(dst + col0, a1, col0, p.N, vec);
    store_bf16_row(dst + p.N + col0, a3, col0, p.N, vec);
  }
};


// ------------------------------------------------- staged (TMA) epilogue ----
// A staging tile is 32 rows of 128 bytes in the 128-byte swizzle the tensor maps
// use: 16-byte chunk c of row r lives at chunk position c ^ (r & 7).  With one
// row per lane, the eight lanes of a quarter-warp hit eight different chunk
// positions, so 16-byte accesses are free of bank conflicts.
__device__ __forceinline__ uint8_t* staged_chunk(uint8_t* tile, int row, int chunk) {
  return tile + row * 128 + ((chunk ^ (row & 7)) << 4);
}

__device__ __forceinline__ void stage_bf16_half(uint8_t* tile, int row, int half,
                                                const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    uint4 q;
    q.x = pack_bf16(v[8 * j + 0], v[8 * j + 1]);
    q.y = pack_bf16(v[8 * j + 2], v[8 * j + 3]);
    q.z = pack_bf16(v[8 * j + 4], v[8 * j + 5]);
    q.w = pack_bf16(v[8 * j + 6], v[8 * j + 7]);
    *reinterpret_cast<uint4*>(staged_chunk(tile, row, 4 * half + j)) = q;
  }
}

__device__ __forceinline__ void stage_f32(uint8_t* tile, int row, const float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 8; ++j)
    *reinterpret_cast<float4*>(staged_chunk(tile, row, j)) =
        make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
}

__device__ __forceinline__ void unstage_f32(uint8_t* tile, int row, float (&v)[32]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const float4 q = *reinterpret_cast<const float4*>(staged_chunk(tile, row, j));
    v[4 * j] = q.x; v[4 * j + 1] = q.y; v[4 * j + 2] = q.z; v[4 * j + 3] = q.w;
  }
}

__device__ __forceinline__ void unpack_bf16x8(const uint4& q, float* v) {
  const float2 a = unpack_bf16(q.x), b = unpack_bf16(q.y), c = unpack_bf16(q.z),
               d = unpack_bf16(q.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
  v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}

__device__ __forceinline__ void load_acc32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  tmem_ld_32x32(taddr, r);
  tmem_ld_wait();
#pragma unroll
  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
}

// Rotates the 16 interleaved pairs of a 32-column run that starts at `col`.
__device__ __forceinline__ void rope_rotate32(const GemmParams& p, int row, int col,
                                              float (&v)[32]) {
  const int pos = row % p.rope_T;
  const int half = p.head_dim >> 1;
  const int pair0 = (col % p.head_dim) >> 1;
  const float4* cs = reinterpret_cast<const float4*>(p.rope_cos + static_cast<long>(pos) * half + pair0);
  const float4* sn = reinterpret_cast<const float4*>(p.rope_sin + static_cast<long>(pos) * half + pair0);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float4 c4 = cs[j], s4 = sn[j];
    const float c[4] = {c4.x, c4.y, c4.z, c4.w};
    const float sv[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float xe = bf16_round(v[8 * j + 2 * i]);
      const float xo = bf16_round(v[8 * j + 2 * i + 1]);
      v[8 * j + 2 * i] = xe * c[i] - xo * sv[i];
      v[8 * j + 2 * i + 1] = xe * sv[i] + xo * c[i];
    }
  }
}

// Two warps serve each TMEM lane quarter (a warp may only read the 32 lanes
// selected by warp_id % 4); `part` 0/1 takes the even/odd column chunks of every
// tile, so each scheduler has two epilogue warps to hide latency with.
template <int BN, int EPI>
__device__ __forceinline__ void staged_epilogue(const GemmParams& p, const EpiMaps& em,
                                                GemmBarriers* bars, uint8_t* warp_smem,
                                                uint32_t tmem_base, int quarter, int part,
                                                int lane, int num_tiles, volatile int* abort) {
  using T = EpiTraits<EPI>;
  constexpr bool kDual = (EPI == EPI_SWIGLU);
  constexpr bool kHasAux = (EPI == EPI_RESID || EPI == EPI_SWIGLU_BWD);
  constexpr int BN_OUT = kDual ? BN / 2 : BN;
  constexpr int CW = T::kChunk;
  constexpr int kChunksPerTile = BN_OUT / CW;
  uint8_t* tile0 = warp_smem;
  uint8_t* tile1 = warp_smem + kEpiTileBytes;  // only epilogues with two tiles touch it
  uint64_t* aux_bar = &bars->aux_full[part * 4 + quarter];
  uint32_t aux_phase = 0;
  int acc = 0;
  uint32_t acc_phase = 0;

  auto chunks_in = [&](int tile) {
    const int n = (p.N - (tile / p.num_m_tiles) * BN_OUT + CW - 1) / CW;
    return n < kChunksPerTile ? n : kChunksPerTile;
  };
  // Auxiliary operands land in the tiles the results are later stored from.
  auto load_aux = [&](int tile, int c) {  // one lane
    const int y = (tile % p.num_m_tiles) * BM + quarter * 32;
    const int x = (tile / p.num_m_tiles) * BN_OUT + c * CW;
    if constexpr (EPI == EPI_RESID) {
      mbar_expect_tx(aux_bar, kEpiTileBytes);
      tma_load_2d(tile0, &em.m[1], aux_bar, x, y);
    } else if constexpr (EPI == EPI_SWIGLU_BWD) {
      mbar_expect_tx(aux_bar, 2 * kEpiTileBytes);
      tma_load_2d(tile0, &em.m[2], aux_bar, x, y);
      tma_load_2d(tile1, &em.m[3], aux_bar, x, y);
    }
  };
  // First chunk of this warp at or after (tile, c): returns false when none is left.
  auto next_chunk = [&](int& tile, int& c) {
    while (tile < num_tiles) {
      if (c < chunks_in(tile)) return true;
      tile += gridDim.x;
      c = part;
    }
    return false;
  };
  if constexpr (kHasAux) {
    if (lane == 0) {
      int t = blockIdx.x, c = part;
      if (next_chunk(t, c)) load_aux(t, c);
    }
  }

  bool ok = true;
  for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
    const int m0 = (tile % p.num_m_tiles) * BM;
    const int n0 = (tile / p.num_m_tiles) * BN_OUT;
    const int nchunks = chunks_in(tile);
    if (!wait_or_abort(&bars->tmem_full[acc], acc_phase, abort)) {
      report_status(p.status, kStatusTimeoutTmemFull);
      *abort = 1;
      break;
    }
    tc_fence_after();
    const int row0 = m0 + quarter * 32;
    const int row = row0 + lane;
    const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
    for (int c = part; c < nchunks; c += 2) {
      const int col0 = n0 + c * CW;
      if constexpr (kHasAux) {
        if (!wait_or_abort(aux_bar, aux_phase, abort)) {
          report_status(p.status, kStatusTimeoutFull);
          *abort = 1;
          ok = false;
          break;
        }
        aux_phase ^= 1;
      }
      if constexpr (EPI == EPI_BF16 || EPI == EPI_ROPE) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float v[32];
          load_acc32(t_row + c * CW + h * 32, v);
          if constexpr (EPI == EPI_ROPE) {
            if (col0 + h * 32 < p.rope_cols) rope_rotate32(p, row, col0 + h * 32, v);
          }
          if (h == 0) {
            if (lane == 0) tma_store_wait_read<0>();  // previous store has left the tile
            __syncwarp();
          }
          stage_bf16_half(tile0, lane, h, v);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&em.m[0], tile0, col0, row0);
          tma_store_commit();
        }
      } else if constexpr (EPI == EPI_F32) {
        float v[32];
        load_acc32(t_row + c * CW, v);
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
        stage_f32(tile0, lane, v);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (p.beta) tma_reduce_add_2d(&em.m[0], tile0, col0, row0);
          else tma_store_2d(&em.m[0], tile0, col0, row0);
          tma_store_commit();
        }
      } else if constexpr (EPI == EPI_RESID) {
        float v[32], res[32];
        unstage_f32(tile0, lane, res);
        load_acc32(t_row + c * CW, v);
#pragma unroll
        for (int j = 0; j < 32; ++j) res[j] += bf16_round(v[j]);
        stage_f32(tile0, lane, res);  // each lane rewrites exactly the bytes it read
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&em.m[0], tile0, col0, row0);
          tma_store_commit();
          int t = tile, cn = c + 2;
          if (next_chunk(t, cn)) {
            tma_store_wait_read<0>();  // the tile is refilled only after the store has read it
            load_aux(t, cn);
          }
        }
      } else if constexpr (EPI == EPI_SWIGLU) {
        // One tile, used three times: w1 x, w3 x, then the gated product.
        uint4 keep3[8], gated[8];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float v[32], w[32];
          {
            uint32_t r[32], r2[32];
            tmem_ld_32x32(t_row + c * CW + h * 32, r);
            tmem_ld_32x32(t_row + BN / 2 + c * CW + h * 32, r2);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              v[j] = __uint_as_float(r[j]);
              w[j] = __uint_as_float(r2[j]);
            }
          }
          if (h == 0) {
            if (lane == 0) tma_store_wait_read<0>();
            __syncwarp();
          }
          stage_bf16_half(tile0, lane, h, v);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            keep3[4 * h + j].x = pack_bf16(w[8 * j + 0], w[8 * j + 1]);
            keep3[4 * h + j].y = pack_bf16(w[8 * j + 2], w[8 * j + 3]);
            keep3[4 * h + j].z = pack_bf16(w[8 * j + 4], w[8 * j + 5]);
            keep3[4 * h + j].w = pack_bf16(w[8 * j + 6], w[8 * j + 7]);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float a = bf16_round(v[j]);
            v[j] = a * fast_sigmoid(a) * bf16_round(w[j]);
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            gated[4 * h + j].x = pack_bf16(v[8 * j + 0], v[8 * j + 1]);
            gated[4 * h + j].y = pack_bf16(v[8 * j + 2], v[8 * j + 3]);
            gated[4 * h + j].z = pack_bf16(v[8 * j + 4], v[8 * j + 5]);
            gated[4 * h + j].w = pack_bf16(v[8 * j + 6], v[8 * j + 7]);
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&em.m[1], tile0, col0, row0);
          tma_store_commit();
          tma_store_wait_read<0>();
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(staged_chunk(tile0, lane, j)) = keep3[j];
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&em.m[2], tile0, col0, row0);
          tma_store_commit();
          tma_store_wait_read<0>();
        }
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j)
          *reinterpret_cast<uint4*>(staged_chunk(tile0, lane, j)) = gated[j];
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&em.m[0], tile0, col0, row0);
          tma_store_commit();
        }
      } else if constexpr (EPI == EPI_SWIGLU_BWD) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          float v[32], a1[32], a3[32];
          load_acc32(t_row + c * CW + h * 32, v);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            unpack_bf16x8(*reinterpret_cast<const uint4*>(staged_chunk(tile0, lane, 4 * h + j)),
                          a1 + 8 * j);
            unpack_bf16x8(*reinterpret_cast<const uint4*>(staged_chunk(tile1, lane, 4 * h + j)),
                          a3 + 8 * j);
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float a = a1[j];
            const float dg = bf16_round(v[j]);
            const float sig = fast_sigmoid(a);
            const float silu = a * sig;
            a1[j] = dg * a3[j] * (sig + silu * (1.0f - sig));
            a3[j] = dg * silu;
          }
          stage_bf16_half(tile0, lane, h, a1);  // results replace the inputs they came from
          stage_bf16_half(tile1, lane, h, a3);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&em.m[0], tile0, col0, row0);
          tma_store_2d(&em.m[1], tile1, col0, row0);
          tma_store_commit();
          int t = tile, cn = c + 2;
          if (next_chunk(t, cn)) {
            tma_store_wait_read<0>();
            load_aux(t, cn);
          }
        }
      }
    }
    tc_fence_before();
    mbar_arrive(&bars->tmem_empty[acc]);
    if (++acc == 2) {
      acc = 0;
      acc_phase ^= 1;
    }
  }
  if (lane == 0) tma_store_wait<0>();
}

// Staged instantiations exist for the operand layouts the model uses; anything
// else goes through the direct epilogue.
template <int EPI, bool A_MN, bool B_MN>
constexpr bool staged_supported() {
  switch (EPI) {
    case EPI_BF16: return !A_MN;
    case EPI_F32: return A_MN && B_MN;
    case EPI_RESID: return !A_MN && !B_MN;
    case EPI_ROPE: return !A_MN && !B_MN;
    case EPI_SWIGLU: return !A_MN && !B_MN;
    case EPI_SWIGLU_BWD: return !A_MN && B_MN;
    default: return false;
  }
}

// ---------------------------------------------------------------- kernel ----
template <int BN, bool A_MN, bool B_MN, int EPI, bool STAGED>
__global__ void __launch_bounds__(kThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
            const __grid_constant__ EpiMaps em, const GemmParams p) {
  using Cfg = GemmConfig<BN, EPI, STAGED>;
  constexpr bool kDual = (EPI == EPI_SWIGLU);
  // In dual mode the logical N tile is BN/2 wide: the B tile stacks BN/2 rows of
  // the first matrix on BN/2 rows of the second.
  constexpr int BN_OUT = kDual ? BN / 2 : BN;
  static_assert(!(kDual && B_MN), "dual epilogue expects K-major weights");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi_smem = smem + Cfg::kStages * Cfg::kStageBytes;  // 1024-byte aligned
  GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(epi_smem + Cfg::kEpiBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->tmem_full[s], 1);
      mbar_init(&bars->tmem_empty[s], 32 * kEpiWarps);
    }
    for (int s = 0; s < kEpiWarps; ++s) mbar_init(&bars->aux_full[s], 1);
    bars->abort = 0;
    mbar_fence_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
    if constexpr (STAGED) {
      for (int i = 0; i < 4; ++i) prefetch_tensormap(&em.m[i]);
    }
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  volatile int* abort = &bars->abort;
  // Set-up is done without touching global data: let the next kernel in the stream
  // begin its own set-up, then wait for the previous kernel's results.
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer ----
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % p.num_m_tiles) * BM;
        const int n0 = (tile / p.num_m_tiles) * BN_OUT;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&bars->empty[stage], phase ^ 1, abort)) {
            report_status(p.status, kStatusTimeoutEmpty);
            *abort = 1;
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * Cfg::kStageBytes;
          uint8_t* sB = sA + kTileABytes;
          mbar_expect_tx(&bars->full[stage], Cfg::kStageBytes);
          const int k0 = kb * BK;
          if constexpr (A_MN) {
#pragma unroll
            for (int i = 0; i < BM / 64; ++i)
              tma_load_2d(sA + i * (BK * 128), &tmA, &bars->full[stage], m0 + i * 64, k0);
          } else {
            tma_load_2d(sA, &tmA, &bars->full[stage], k0, m0);
          }
          if constexpr (B_MN) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_2d(sB + i * (BK * 128), &tmB, &bars->full[stage], n0 + i * 64, k0);
          } else if constexpr (kDual) {
            tma_load_2d(sB, &tmB, &bars->full[stage], k0, n0);
            tma_load_2d(sB + (BN / 2) * 128, &tmB, &bars->full[stage], k0, p.dual_offset + n0);
          } else {
            tma_load_2d(sB, &tmB, &bars->full[stage], k0, n0);
          }
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer ----
    // The whole warp walks the loops and waits on the barriers; one elected lane
    // issues.  Control flow and every operand (descriptors, tensor-memory address,
    // counters) are then warp-uniform and live in uniform registers, which is where
    // tcgen05.mma reads its operands: issued from inside a one-lane branch each MMA
    // pays for moving them there, which costs more than a 128 x 128 x 16 product takes.
    {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, A_MN, B_MN);
      const uint32_t smem_base = smem_u32(smem);
      const uint64_t a_desc0 = A_MN ? umma_smem_desc(smem_base, BK * 128, 1024)
                                    : umma_smem_desc(smem_base, 16, 1024);
      const uint64_t b_desc0 = B_MN ? umma_smem_desc(smem_base + kTileABytes, BK * 128, 1024)
                                    : umma_smem_desc(smem_base + kTileABytes, 16, 1024);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!wait_or_abort(&bars->tmem_empty[acc], acc_phase ^ 1, abort)) {
          report_status(p.status, kStatusTimeoutTmemEmpty);
          *abort = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&bars->full[stage], phase, abort)) {
            report_status(p.status, kStatusTimeoutFull);
            *abort = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t a_stage = umma_desc_advance(a_desc0, stage * Cfg::kStageBytes);
          const uint64_t b_stage = umma_desc_advance(b_desc0, stage * Cfg::kStageBytes);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_bf16_ss(d_tmem, umma_desc_advance(a_stage, k * (A_MN ? 2048 : 32)),
                           umma_desc_advance(b_stage, k * (B_MN ? 2048 : 32)), idesc,
                           (kb | k) != 0);
            umma_commit(&bars->empty[stage]);
            if (kb == num_kb - 1) umma_commit(&bars->tmem_full[acc]);
          }
          __syncwarp();
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else if constexpr (STAGED) {
    const int quarter = warp & 3;  // TMEM lanes this warp may read
    const int part = (warp - 2) >> 2;
    staged_epilogue<BN, EPI>(p, em, bars, epi_smem + (warp - 2) * Cfg::kEpiWarpBytes, tmem_base,
                             quarter, part, lane, num_tiles, abort);
  } else {
    // --------------------------------------------------- direct epilogue ----
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;  // even / odd 32-column chunks
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int m0 = (tile % p.num_m_tiles) * BM;
      const int n0 = (tile / p.num_m_tiles) * BN_OUT;
      if (!wait_or_abort(&bars->tmem_full[acc], acc_phase, abort)) {
        report_status(p.status, kStatusTimeoutTmemFull);
        *abort = 1;
        break;
      }
      tc_fence_after();
      const int row = m0 + quarter * 32 + lane;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
#pragma unroll 1
      for (int c = part; c < BN_OUT / 32; c += 2) {
        const int col0 = n0 + c * 32;
        if (col0 >= p.N) break;  // warp-uniform
        uint32_t r[32];
        float v[32], w[32];
        tmem_ld_32x32(t_row + c * 32, r);
        if constexpr (kDual) {
          uint32_t r2[32];
          tmem_ld_32x32(t_row + BN / 2 + c * 32, r2);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) w[j] = __uint_as_float(r2[j]);
        } else {
          tmem_ld_wait();
        }
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (row < p.M &&
            SFL_BOUNDS_OK(row >= 0 && col0 >= 0 && col0 < p.N && tile < num_tiles && n0 < p.N,
                          p.status))
          EpilogueOp<EPI>::apply(p, row, col0, v, w);
      }
      tc_fence_before();
      mbar_arrive(&bars->tmem_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}


// ------------------------------------------------- grouped weight gradients ----
// The weight gradients of one transformer block are up to four products
// dW_g[N_g, K_g] (+)= dY_g[T, N_g]^T X_g[T, K_g] with a long reduction (T tokens) and
// small outputs: launched one by one, none of them has enough 128 x 256 tiles to
// fill 148 SMs.  This kernel walks the tiles of all problems in one persistent
// launch, so only the last round of the whole group is partially filled.  Operand
// and output tensor maps are per problem; the pipeline is the one of gemm_kernel
// with MN-major operands and the staged fp32 epilogue (store, or TMA reduce-add
// when the gradient accumulates).
constexpr int kMaxGroup = 4;
constexpr int kGroupBN = 256;

struct GroupedProblem {
  int m_tiles, n_tiles;  // 128-row x 256-column tiles of the output
  int num_kb;            // 64-deep steps of the reduction
  int tile_begin;        // first global tile index of this problem
  int cols;              // output columns (K_g)
  int beta;
};

struct GroupedParams {
  int count;
  int total_tiles;
  GroupedProblem prob[kMaxGroup];
  int* status;
};

struct GroupedMaps {
  CUtensorMap a[kMaxGroup];    // dY_g as MN-major A
  CUtensorMap b[kMaxGroup];    // X_g as MN-major B
  CUtensorMap out[kMaxGroup];  // fp32 gradient
};

__device__ __forceinline__ int grouped_find(const GroupedParams& p, int tile) {
  int g = p.count - 1;
  while (g > 0 && tile < p.prob[g].tile_begin) --g;
  return g;
}

__global__ void __launch_bounds__(kThreads, 1)
wgrad_grouped_kernel(const __grid_constant__ GroupedMaps maps,
                     const __grid_constant__ GroupedParams p) {
  using Cfg = GemmConfig<kGroupBN, EPI_F32, true>;
  constexpr int BN = kGroupBN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi_smem = smem + Cfg::kStages * Cfg::kStageBytes;
  GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(epi_smem + Cfg::kEpiBytes);
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->tmem_full[s], 1);
      mbar_init(&bars->tmem_empty[s], 32 * kEpiWarps);
    }
    bars->abort = 0;
    mbar_fence_init();
    for (int g = 0; g < p.count; ++g) {
      prefetch_tensormap(&maps.a[g]);
      prefetch_tensormap(&maps.b[g]);
      prefetch_tensormap(&maps.out[g]);
    }
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  volatile int* abort = &bars->abort;
  // Set-up is done without touching global data: let the next kernel in the stream
  // begin its own set-up, then wait for the previous kernel's results.
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
        const int g = grouped_find(p, tile);
        const GroupedProblem& q = p.prob[g];
        const int local = tile - q.tile_begin;
        const int m0 = (local % q.m_tiles) * BM;
        const int n0 = (local / q.m_tiles) * BN;
        for (int kb = 0; kb < q.num_kb; ++kb) {
          if (!wait_or_abort(&bars->empty[stage], phase ^ 1, abort)) {
            report_status(p.status, kStatusTimeoutEmpty);
            *abort = 1;
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * Cfg::kStageBytes;
          uint8_t* sB = sA + kTileABytes;
          mbar_expect_tx(&bars->full[stage], Cfg::kStageBytes);
          const int k0 = kb * BK;
#pragma unroll
          for (int i = 0; i < BM / 64; ++i)
            tma_load_2d(sA + i * (BK * 128), &maps.a[g], &bars->full[stage], m0 + i * 64, k0);
#pragma unroll
          for (int i = 0; i < BN / 64; ++i)
            tma_load_2d(sB + i * (BK * 128), &maps.b[g], &bars->full[stage], n0 + i * 64, k0);
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // converged warp, one elected issuing lane (see gemm_kernel)
    {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, true, true);
      const uint32_t smem_base = smem_u32(smem);
      const uint64_t a_desc0 = umma_smem_desc(smem_base, BK * 128, 1024);
      const uint64_t b_desc0 = umma_smem_desc(smem_base + kTileABytes, BK * 128, 1024);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < p.total_tiles && ok; tile += gridDim.x) {
        const int num_kb = p.prob[grouped_find(p, tile)].num_kb;
        if (!wait_or_abort(&bars->tmem_empty[acc], acc_phase ^ 1, abort)) {
          report_status(p.status, kStatusTimeoutTmemEmpty);
          *abort = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&bars->full[stage], phase, abort)) {
            report_status(p.status, kStatusTimeoutFull);
            *abort = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t a_stage = umma_desc_advance(a_desc0, stage * Cfg::kStageBytes);
          const uint64_t b_stage = umma_desc_advance(b_desc0, stage * Cfg::kStageBytes);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_bf16_ss(d_tmem, umma_desc_advance(a_stage, k * 2048),
                           umma_desc_advance(b_stage, k * 2048), idesc, (kb | k) != 0);
            umma_commit(&bars->empty[stage]);
            if (kb == num_kb - 1) umma_commit(&bars->tmem_full[acc]);
          }
          __syncwarp();
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;
    uint8_t* tile0 = epi_smem + (warp - 2) * Cfg::kEpiWarpBytes;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int tile = blockIdx.x; tile < p.total_tiles; tile += gridDim.x) {
      const int g = grouped_find(p, tile);
      const GroupedProblem& q = p.prob[g];
      const int local = tile - q.tile_begin;
      const int m0 = (local % q.m_tiles) * BM;
      const int n0 = (local / q.m_tiles) * BN;
      int nchunks = (q.cols - n0 + 31) / 32;
      if (nchunks > BN / 32) nchunks = BN / 32;
      if (!wait_or_abort(&bars->tmem_full[acc], acc_phase, abort)) {
        report_status(p.status, kStatusTimeoutTmemFull);
        *abort = 1;
        break;
      }
      tc_fence_after();
      const int row0 = m0 + quarter * 32;
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      for (int c = part; c < nchunks; c += 2) {
        float v[32];
        load_acc32(t_row + c * 32, v);
        if (lane == 0) tma_store_wait_read<0>();
        __syncwarp();
        stage_f32(tile0, lane, v);
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (q.beta) tma_reduce_add_2d(&maps.out[g], tile0, n0 + c * 32, row0);
          else tma_store_2d(&maps.out[g], tile0, n0 + c * 32, row0);
          tma_store_commit();
        }
      }
      tc_fence_before();
      mbar_arrive(&bars->tmem_empty[acc]);
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    if (lane == 0) tma_store_wait<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}

// ------------------------------------------------------------------ host ----
// --------------------------------- GEMM fused with its all-reduce (tensor parallel) ----
// Under tensor parallelism the output projection and the down projection (forward)
// and the input gradients of the column-parallel layers (backward) are products
// whose reduction dimension is split over the ranks: every rank holds a partial
// [M, N] result and all of them need the sum (the reference all-reduces after
// F.linear: distributed/llmdist/tensor_parallel.py:40-45 for the forward sums of
// the output and down projections, :25-36 for the input gradients of the
// column-parallel layers).  This kernel is the GEMM and
// that all-reduce in one launch, tile by tile over NVLink peer memory:
//
//   * the 128-row tile strips are owned round-robin by the ranks;
//   * a CTA that finishes a tile owned by a peer converts the accumulator to bf16
//     and stores it straight into that peer's staging buffer, then publishes one
//     flag word per epilogue warp (system-scope release);
//   * a CTA that finishes a tile it owns waits for the other ranks' strips of the
//     same tile, adds them to its own accumulator in rank order (so the sum is the
//     same on every run), applies the epilogue (fp32 residual add, or a plain bf16
//     result) and stores the finished rows into the result buffer of every rank.
//
// With two ranks (ONE_SHOT) ownership is dropped: each rank sends every strip to the
// other, waits for the other's strip of the same tile and finishes all rows
// itself, so the matrix crosses the link once as bf16 in a single phase and no
// rank's result depends on a peer's stores.
//
// A peer may only write here once this rank has entered the kernel (ready flags,
// polled while the first main loop runs), and with owned tiles the kernel ends only
// after every rank has reported that all its stores are done.  Owned and foreign tiles are
// the same function of the tile index on every rank and CTAs walk tiles in the
// same order, so a wait is always for a tile that its producer reaches without
// waiting for this rank; every wait is bounded and reports through the status
// word.  Stores to peers go through the swizzled staging tile of each epilogue
// warp and leave as full 128-byte rows.
//
// Requirements the host entry point enforces or relies on: the grid is the same on
// every rank (it is min(tiles, SM count) of identical shapes on identical GPUs) and
// never exceeds the SM count, so that with one CTA per SM every CTA of the grid is
// resident at once; CTA x only ever waits for CTA x of a peer, so no wait depends on
// a CTA that cannot be scheduled.  Running another kernel that pins SMs for the whole
// duration on the same device at the same time would void that argument.  Once a peer
// wait has run out the warp reports it, stops the CTA's pipeline and touches no peer
// memory again.
struct TpFuse {
  int rank, world;
  char* stage[kMaxPeers];           // [source rank][tile][4 strips][4 chunks] 4 KB blocks
  char* out[kMaxPeers];             // result buffers
  uint32_t* tile_flags[kMaxPeers];  // [tile][source rank][epilogue warp]
  uint32_t* flags[kMaxPeers];       // barrier flags of the communicator
  long out_off;                     // byte offset of the result inside `out`
  const float* resid;               // local fp32 residual (fp32 output only)
  long ldresid;
  int slot;
  uint32_t epoch, tile_epoch;
  unsigned long long* trace;        // optional: phase times of CTA 0 (nanoseconds, summed)
};

__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

constexpr int kTpBN = 256;
// Same budget as the collectives (comm.cu: about ten seconds by default, sized for the
// skew between training ranks); sfl_comm_set_spin_limit sets both.
__device__ uint32_t g_tp_spin_limit = 48u << 20;

__device__ __forceinline__ bool tp_wait_flag(const uint32_t* flag, uint32_t epoch) {
  const uint32_t limit = g_tp_spin_limit;
  for (uint32_t spin = 0; spin < limit; ++spin) {
    if (reached(ld_acquire_sys(flag), epoch)) return true;
    if (spin > 64) __nanosleep(200);
  }
  return false;
}

// The warp's 32-row x 128-byte staging tile goes to `dst` (row pitch in bytes),
// four complete rows per store instruction.
__device__ __forceinline__ void tile_to_global(char* dst, long pitch, uint8_t* tile, int lane,
                                               int rows_valid) {
  const int ch = lane & 7;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int r = i * 4 + (lane >> 3);
    const uint4 q = *reinterpret_cast<const uint4*>(staged_chunk(tile, r, ch));
    if (r < rows_valid) st_peer_u4(dst + r * pitch + ch * 16, q);
  }
}

// The staging tile as it is (swizzle included) to 4 KB of contiguous memory: every
// store instruction of the warp covers 512 consecutive bytes.  The reader undoes
// the swizzle (staged_chunk on the address).  Plain (weak) stores: the release
// store of the flag that follows orders them.
__device__ __forceinline__ void tile_to_block(char* dst, const uint8_t* tile, int lane) {
#pragma unroll
  for (int i = 0; i < 8; ++i)
    *reinterpret_cast<uint4*>(dst + i * 512 + lane * 16) =
        *reinterpret_cast<const uint4*>(tile + i * 512 + lane * 16);
}

template <bool B_MN, bool OUT_BF16, bool ONE_SHOT>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const GemmParams p, const TpFuse f) {
  using Cfg = GemmConfig<kTpBN, EPI_F32, true>;  // one 4 KB staging tile per epilogue warp
  constexpr int BN = kTpBN;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* epi_smem = smem + Cfg::kStages * Cfg::kStageBytes;
  GemmBarriers* bars = reinterpret_cast<GemmBarriers*>(epi_smem + Cfg::kEpiBytes);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int num_tiles = p.num_m_tiles * p.num_n_tiles;
  const int num_kb = (p.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    for (int s = 0; s < Cfg::kStages; ++s) {
      mbar_init(&bars->full[s], 1);
      mbar_init(&bars->empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->tmem_full[s], 1);
      mbar_init(&bars->tmem_empty[s], 32 * kEpiWarps);
    }
    bars->abort = 0;
    mbar_fence_init();
    prefetch_tensormap(&tmA);
    prefetch_tensormap(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, Cfg::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = bars->tmem_base;
  volatile int* abort = &bars->abort;
  pdl_launch_dependents();
  pdl_wait();

  if (warp == 0) {
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int m0 = (tile % p.num_m_tiles) * BM;
        const int n0 = (tile / p.num_m_tiles) * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&bars->empty[stage], phase ^ 1, abort)) {
            report_status(p.status, kStatusTimeoutEmpty);
            *abort = 1;
            ok = false;
            break;
          }
          uint8_t* sA = smem + stage * Cfg::kStageBytes;
          uint8_t* sB = sA + kTileABytes;
          mbar_expect_tx(&bars->full[stage], Cfg::kStageBytes);
          const int k0 = kb * BK;
          tma_load_2d(sA, &tmA, &bars->full[stage], k0, m0);
          if constexpr (B_MN) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i)
              tma_load_2d(sB + i * (BK * 128), &tmB, &bars->full[stage], n0 + i * 64, k0);
          } else {
            tma_load_2d(sB, &tmB, &bars->full[stage], k0, n0);
          }
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // converged warp, one elected issuing lane (see gemm_kernel)
    {
      constexpr uint32_t idesc = umma_idesc_bf16(BM, BN, false, B_MN);
      const uint32_t smem_base = smem_u32(smem);
      const uint64_t a_desc0 = umma_smem_desc(smem_base, 16, 1024);
      const uint64_t b_desc0 = B_MN ? umma_smem_desc(smem_base + kTileABytes, BK * 128, 1024)
                                    : umma_smem_desc(smem_base + kTileABytes, 16, 1024);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        if (!wait_or_abort(&bars->tmem_empty[acc], acc_phase ^ 1, abort)) {
          report_status(p.status, kStatusTimeoutTmemEmpty);
          *abort = 1;
          break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!wait_or_abort(&bars->full[stage], phase, abort)) {
            report_status(p.status, kStatusTimeoutFull);
            *abort = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t a_stage = umma_desc_advance(a_desc0, stage * Cfg::kStageBytes);
          const uint64_t b_stage = umma_desc_advance(b_desc0, stage * Cfg::kStageBytes);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BK / 16; ++k)
              umma_bf16_ss(d_tmem, umma_desc_advance(a_stage, k * 32),
                           umma_desc_advance(b_stage, k * (B_MN ? 2048 : 32)), idesc,
                           (kb | k) != 0);
            umma_commit(&bars->empty[stage]);
            if (kb == num_kb - 1) umma_commit(&bars->tmem_full[acc]);
          }
          __syncwarp();
          if (++stage == Cfg::kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        if (++acc == 2) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else {
    // ------------------------------------------- epilogue + collective ----
    const int quarter = warp & 3;
    const int part = (warp - 2) >> 2;
    const int wslot = warp - 2;
    uint8_t* tile_smem = epi_smem + wslot * Cfg::kEpiWarpBytes;
    // "This rank has entered": everything that used the buffers before is done.
    if (blockIdx.x == 0 && wslot == 0 && lane < f.world) {
      __threadfence_system();
      st_release_sys(flag_ptr(f.flags[lane], f.slot, 0, f.rank), f.epoch);
    }
    bool peers_ready = false;
    bool peer_failed = false;  // warp-uniform: a peer wait ran out, no further peer traffic
    int acc = 0;
    uint32_t acc_phase = 0;
    // Phase times of the first tile of CTA 0's first epilogue warp, when asked for:
    // start -> accumulator ready -> peers ready -> strip sent -> peers' strips here -> done.
    const bool tracing = f.trace != nullptr && blockIdx.x == 0 && wslot == 0 && lane == 0;
    unsigned long long stamp = tracing ? global_ns() : 0;
    int trace_at = 0;
    auto mark = [&]() {
      if (tracing && trace_at < 5) {
        const unsigned long long now = global_ns();
        atomicAdd(f.trace + trace_at, now - stamp);
        stamp = now;
        ++trace_at;
      }
    };
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      const int m_tile = tile % p.num_m_tiles;
      const int m0 = m_tile * BM;
      const int n0 = (tile / p.num_m_tiles) * BN;
      if (!wait_or_abort(&bars->tmem_full[acc], acc_phase, abort)) {
        report_status(p.status, kStatusTimeoutTmemFull);
        *abort = 1;
        break;
      }
      tc_fence_after();
      mark();
      if (!peers_ready) {
        const bool ok = lane >= f.world ||
                        tp_wait_flag(flag_ptr(f.flags[f.rank], f.slot, 0, lane), f.epoch);
        if (!__all_sync(0xffffffffu, ok)) {
          // A peer never entered the kernel: nothing may be stored into its buffers.
          // Stop this CTA's pipeline and leave without any peer access.
          if (lane == 0) {
            report_status(p.status, kStatusTimeoutPeer);
            *abort = 1;
          }
          peer_failed = true;
          break;
        }
        peers_ready = true;
      }
      mark();
      const int owner = ONE_SHOT ? f.rank : m_tile % f.world;
      const int strip = quarter * 32;            // first row of this warp inside the tile
      const int rows_valid = p.M - (m0 + strip);  // rows of the strip that exist (may exceed 32)
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(strip) << 16) + acc * BN;
      const long tile_elems = static_cast<long>(BM) * BN;
      // A strip in a staging buffer: four 4 KB blocks (32 rows x 64 columns of bf16),
      // one per 64-column chunk, each an image of the sender's staging tile.
      const long my_strip = ((static_cast<long>(f.rank) * num_tiles + tile) * tile_elems +
                             static_cast<long>(strip) * BN) * 2;
      const long flag_word = (static_cast<long>(tile) * kMaxPeers + f.rank) * kEpiWarps + wslot;
      if (ONE_SHOT || owner != f.rank) {
        // ---- bf16 strip into the staging buffer of the owner (or of every peer) ----
        for (int c = part; c < BN / 64; c += 2) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            float v[32];
            load_acc32(t_row + c * 64 + h * 32, v);
            stage_bf16_half(tile_smem, lane, h, v);
          }
          __syncwarp();
          if constexpr (ONE_SHOT) {
            for (int peer = 0; peer < f.world; ++peer)
              if (peer != f.rank)
                tile_to_block(f.stage[peer] + my_strip + c * kEpiTileBytes, tile_smem, lane);
          } else {
            tile_to_block(f.stage[owner] + my_strip + c * kEpiTileBytes, tile_smem, lane);
          }
          __syncwarp();
        }
        // The warp barrier orders every lane's stores before the flag lanes' release
        // stores, which are cumulative: one system-scope release per flag instead of
        // a system fence in each of the 32 lanes (measured: 25 -> 19 us per strip).
        __syncwarp();
        if constexpr (ONE_SHOT) {
          if (lane < f.world && lane != f.rank)
            st_release_sys(f.tile_flags[lane] + flag_word, f.tile_epoch);
        } else {
          tc_fence_before();
          mbar_arrive(&bars->tmem_empty[acc]);
          if (lane == 0) st_release_sys(f.tile_flags[owner] + flag_word, f.tile_epoch);
        }
      }
      mark();
      if (owner == f.rank) {
        // ---- add the peers' strips in rank order, finish the rows, store them ----
        bool ok = true;
        if (lane < f.world && lane != f.rank)
          ok = tp_wait_flag(f.tile_flags[f.rank] +
                                (static_cast<long>(tile) * kMaxPeers + lane) * kEpiWarps + wslot,
                            f.tile_epoch);
        if (!__all_sync(0xffffffffu, ok)) {
          // The strips of this tile never arrived: the sum would be wrong, so no row
          // of it is stored anywhere and the CTA stops.
          if (lane == 0) {
            report_status(p.status, kStatusTimeoutPeer);
            *abort = 1;
          }
          peer_failed = true;
          break;
        }
        mark();
        const int row = m0 + strip + lane;
        const bool row_ok = row < p.M;
        const long strip_at = (static_cast<long>(tile) * tile_elems +
                               static_cast<long>(strip) * BN) * 2;
        constexpr int CW = OUT_BF16 ? 64 : 32;
        for (int c = part; c < BN / CW; c += 2) {
          const int col0 = n0 + c * CW;
#pragma unroll
          for (int h = 0; h < CW / 32; ++h) {
            float v[32], sum[32];
            load_acc32(t_row + c * CW + h * 32, v);
#pragma unroll
            for (int j = 0; j < 32; ++j) sum[j] = 0.f;
            for (int src = 0; src < f.world; ++src) {
              if (src == f.rank) {
#pragma unroll
                for (int j = 0; j < 32; ++j) sum[j] += bf16_round(v[j]);
              } else {
                const int col = c * CW + h * 32;  // first of 32 columns inside the tile
                const char* block = f.stage[f.rank] + strip_at +
                                    static_cast<long>(src) * num_tiles * tile_elems * 2 +
                                    (col >> 6) * kEpiTileBytes;
                const int first = (col & 63) >> 3;  // 16-byte chunk of the row
                uint4 q[4];
#pragma unroll
                for (int j = 0; j < 4; ++j)
                  q[j] = ld_peer_u4(staged_chunk(
                      reinterpret_cast<uint8_t*>(const_cast<char*>(block)), lane, first + j));
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  float u[8];
                  unpack_bf16x8(q[j], u);
#pragma unroll
                  for (int i = 0; i < 8; ++i) sum[8 * j + i] += u[i];
                }
              }
            }
            if constexpr (OUT_BF16) {
              stage_bf16_half(tile_smem, lane, h, sum);
            } else {
              float res[32];
              const float* rp = f.resid + static_cast<long>(row_ok ? row : 0) * f.ldresid + col0;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const float4 r4 = *reinterpret_cast<const float4*>(rp + 4 * j);
                res[4 * j] = r4.x + bf16_round(sum[4 * j]);
                res[4 * j + 1] = r4.y + bf16_round(sum[4 * j + 1]);
                res[4 * j + 2] = r4.z + bf16_round(sum[4 * j + 2]);
                res[4 * j + 3] = r4.w + bf16_round(sum[4 * j + 3]);
              }
              stage_f32(tile_smem, lane, res);
            }
          }
          __syncwarp();
          const long pitch = static_cast<long>(p.N) * (OUT_BF16 ? 2 : 4);
          const long at = f.out_off + static_cast<long>(m0 + strip) * pitch +
                          static_cast<long>(col0) * (OUT_BF16 ? 2 : 4);
          if constexpr (ONE_SHOT) {
            tile_to_global(f.out[f.rank] + at, pitch, tile_smem, lane, rows_valid);
          } else {
            for (int peer = 0; peer < f.world; ++peer)
              tile_to_global(f.out[peer] + at, pitch, tile_smem, lane, rows_valid);
          }
          __syncwarp();
        }
        tc_fence_before();
        mbar_arrive(&bars->tmem_empty[acc]);
      }
      mark();
      if (tracing && trace_at == 5) {
        atomicAdd(f.trace + 5, 1ull);
        trace_at = 6;
      }
      if (++acc == 2) {
        acc = 0;
        acc_phase ^= 1;
      }
    }
    // ---- all stores of this warp are out; the last warp of the grid trades "done" ----
    // (Not needed when every rank finishes its own copy: nothing of this rank's
    // result is written by a peer, and staging is protected by the ready flags.)
    __syncwarp();
    int last = 0;
    if (!ONE_SHOT && lane == 0) {
      __threadfence_system();  // after the warp barrier: covers every lane's stores
      const uint32_t arrived = atomicAdd(counter_ptr(f.flags[f.rank], f.slot), 1u);
      last = arrived == gridDim.x * kEpiWarps - 1;
    }
    last = __shfl_sync(0xffffffffu, last, 0);
    if (last) {
      // The counter is reset whatever happened, so the slot can be used again; "done" is
      // only traded when no wait of this launch has run out on this rank.
      if (lane == 0) *counter_ptr(f.flags[f.rank], f.slot) = 0;
      const bool healthy = !peer_failed && *abort == 0 &&
                           (p.status == nullptr || *static_cast<volatile int*>(p.status) == 0);
      if (healthy && lane < f.world) {
        st_release_sys(flag_ptr(f.flags[lane], f.slot, 1, f.rank), f.epoch);
        if (!tp_wait_flag(flag_ptr(f.flags[f.rank], f.slot, 1, lane), f.epoch))
          report_status(p.status, kStatusTimeoutPeer);
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, Cfg::kTmemCols);
  }
}


namespace {

struct MapKey {
  const void* base;
  uint64_t inner, outer, ld;
  uint32_t box_inner, box_outer;
  int elem_bytes;
  bool operator<(const MapKey& o) const {
    return std::tie(base, inner, outer, ld, box_inner, box_outer, elem_bytes) <
           std::tie(o.base, o.inner, o.outer, o.ld, o.box_inner, o.box_outer, o.elem_bytes);
  }
};

// Encoding a tensor map costs a few microseconds on the host; training reuses a
// small set of (pointer, shape) combinations every step, so keep them.
int cached_map(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer, uint64_t ld,
               uint32_t box_inner, uint32_t box_outer, int elem_bytes = 2) {
  static std::map<MapKey, CUtensorMap> cache;
  static std::mutex mu;
  MapKey key{base, inner, outer, ld, box_inner, box_outer, elem_bytes};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  int rc = make_tensormap_2d(out, base, elem_bytes, inner, outer, ld, box_inner, box_outer);
  if (rc == 0) {
    if (cache.size() > 8192) cache.clear();
    cache.emplace(key, *out);
  }
  return rc;
}

int sm_count() {
  static int count = 0;
  if (count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
    if (count <= 0) count = 148;
  }
  return count;
}

template <int BN, bool A_MN, bool B_MN, int EPI, bool STAGED>
int launch_one(const CUtensorMap& tmA, const CUtensorMap& tmB, const EpiMaps& em,
               const GemmParams& p, int max_ctas, cudaStream_t stream) {
  using Cfg = GemmConfig<BN, EPI, STAGED>;
  auto kernel = gemm_kernel<BN, A_MN, B_MN, EPI, STAGED>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const int tiles = p.num_m_tiles * p.num_n_tiles;
  int grid = tiles < sm_count() ? tiles : sm_count();
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  return launch_pdl(kernel, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, stream, tmA, tmB, em, p);
}

template <int BN, bool A_MN, bool B_MN, int EPI>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const EpiMaps* em, const GemmParams& p,
           int max_ctas, cudaStream_t stream) {
  if constexpr (staged_supported<EPI, A_MN, B_MN>()) {
    if (em != nullptr)
      return launch_one<BN, A_MN, B_MN, EPI, true>(tmA, tmB, *em, p, max_ctas, stream);
  }
  static const EpiMaps none{};
  return launch_one<BN, A_MN, B_MN, EPI, false>(tmA, tmB, none, p, max_ctas, stream);
}

template <int BN, int EPI>
int launch_major(bool a_mn, bool b_mn, const CUtensorMap& tmA, const CUtensorMap& tmB,
                 const EpiMaps* em, const GemmParams& p, int max_ctas, cudaStream_t stream) {
  if constexpr (EPI == EPI_SWIGLU) {
    if (a_mn || b_mn) return -3;
    return launch<BN, false, false, EPI>(tmA, tmB, em, p, max_ctas, stream);
  } else {
    if (!a_mn && !b_mn) return launch<BN, false, false, EPI>(tmA, tmB, em, p, max_ctas, stream);
    if (!a_mn && b_mn) return launch<BN, false, true, EPI>(tmA, tmB, em, p, max_ctas, stream);
    if (a_mn && b_mn) return launch<BN, true, true, EPI>(tmA, tmB, em, p, max_ctas, stream);
    return launch<BN, true, false, EPI>(tmA, tmB, em, p, max_ctas, stream);
  }
}

}  // namespace
}  // namespace sfl

using namespace sfl;

// a: K-major -> [M,K] row-major with pitch lda; MN-major -> [K,M] row-major.
// b: K-major -> [N,K] row-major with pitch ldb; MN-major -> [K,N] row-major.
extern "C" int sfl_gemm_bf16(const void* a, long lda, int a_mn, const void* b, long ldb, int b_mn,
                             int M, int N, int K, const SflGemmEpilogue* epi, int bn_hint,
                             int max_ctas, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0 || K <= 0 || epi == nullptr) return -2;
  if ((lda & 7) || (ldb & 7)) return -2;  // TMA needs 16-byte row pitches
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15)) return -2;
  const int kind = epi->kind;
  const bool dual = kind == EPI_SWIGLU;

  GemmParams p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.out = epi->out;
  p.ldo = epi->ldo;
  p.out2 = epi->out2;
  p.ldo2 = epi->ldo2;
  p.aux = epi->aux;
  p.ldaux = epi->ldaux;
  p.beta = epi->beta;
  p.rope_cos = epi->rope_cos;
  p.rope_sin = epi->rope_sin;
  p.rope_T = epi->rope_T;
  p.rope_cols = epi->rope_cols;
  p.head_dim = epi->head_dim;
  p.dual_offset = epi->dual_offset;
  p.status = epi->status;
  if (kind == EPI_ROPE && (p.head_dim % 32 != 0 || p.rope_T <= 0)) return -2;

  // Tile width: pick the one that needs the fewest "tile-time units" of waves.
  int bn = bn_hint;
  // SFL_GEMM_BN=128|256 overrides the automatic choice (for A/B measurements).
  static const int forced_bn = [] {
    const char* v = getenv("SFL_GEMM_BN");
    return v == nullptr ? 0 : atoi(v);
  }();
  if (forced_bn == 128 || forced_bn == 256) bn = forced_bn;
  if (dual) {
    bn = 256;  // 128 columns of each of the two products
  } else if (bn != 128 && bn != 256) {
    // 256-wide tiles run the tensor cores measurably closer to peak than 128-wide
    // ones (the 128-row A tile is re-read from shared memory half as often), so
    // narrow tiles are only worth it when wide ones would leave more than half
    // of the SMs without work.
    const long tiles256 = static_cast<long>((M + BM - 1) / BM) * ((N + 255) / 256);
    bn = (N <= 128 || 2 * tiles256 <= sm_count()) ? 128 : 256;
  }
  const int bn_out = dual ? bn / 2 : bn;
  p.num_m_tiles = (M + BM - 1) / BM;
  p.num_n_tiles = (N + bn_out - 1) / bn_out;

  // Staged epilogue: every matrix it touches must be addressable by TMA (16-byte
  // aligned base and row pitch); otherwise the direct epilogue is used.
  EpiMaps em{};
  bool staged = false;
  {
    auto ok16 = [](const void* ptr, long ld, int elem) {
      return ptr != nullptr && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 &&
             (ld * elem) % 16 == 0 && ld > 0;
    };
    auto row_map = [&](CUtensorMap* m, const void* base, long ld, int elem, int cols) {
      return cached_map(m, base, static_cast<uint64_t>(cols), static_cast<uint64_t>(M),
                        static_cast<uint64_t>(ld), 128 / elem, 32, elem) == 0;
    };
    const __nv_bfloat16* out_b = static_cast<const __nv_bfloat16*>(p.out);
    const __nv_bfloat16* out2_b = static_cast<const __nv_bfloat16*>(p.out2);
    const __nv_bfloat16* aux_b = static_cast<const __nv_bfloat16*>(p.aux);
    switch (kind) {
      case EPI_BF16:
        staged = ok16(p.out, p.ldo, 2) && row_map(&em.m[0], p.out, p.ldo, 2, N);
        break;
      case EPI_ROPE:
        staged = ok16(p.out, p.ldo, 2) && p.head_dim % 64 == 0 && p.rope_cols % 64 == 0 &&
                 (reinterpret_cast<uintptr_t>(p.rope_cos) & 15) == 0 &&
                 (reinterpret_cast<uintptr_t>(p.rope_sin) & 15) == 0 &&
                 row_map(&em.m[0], p.out, p.ldo, 2, N);
        break;
      case EPI_F32:
        staged = ok16(p.out, p.ldo, 4) && row_map(&em.m[0], p.out, p.ldo, 4, N);
        break;
      case EPI_RESID:
        staged = ok16(p.out, p.ldo, 4) && ok16(p.aux, p.ldaux, 4) &&
                 row_map(&em.m[0], p.out, p.ldo, 4, N) && row_map(&em.m[1], p.aux, p.ldaux, 4, N);
        break;
      case EPI_SWIGLU:
        staged = ok16(p.out, p.ldo, 2) && ok16(p.out2, p.ldo2, 2) && N % 8 == 0 &&
                 row_map(&em.m[0], p.out, p.ldo, 2, N) &&
                 row_map(&em.m[1], out2_b, p.ldo2, 2, N) &&
                 row_map(&em.m[2], out2_b + N, p.ldo2, 2, N);
        break;
      case EPI_SWIGLU_BWD:
        staged = ok16(p.out, p.ldo, 2) && ok16(p.aux, p.ldaux, 2) && N % 8 == 0 &&
                 row_map(&em.m[0], out_b, p.ldo, 2, N) && row_map(&em.m[1], out_b + N, p.ldo, 2, N) &&
                 row_map(&em.m[2], aux_b, p.ldaux, 2, N) &&
                 row_map(&em.m[3], aux_b + N, p.ldaux, 2, N);
        break;
      default:
        break;
    }
  }
  // SFL_GEMM_DIRECT_EPILOGUE=1 forces the direct path (for A/B measurements).
  static const bool force_direct = [] {
    const char* v = getenv("SFL_GEMM_DIRECT_EPILOGUE");
    return v != nullptr && v[0] == '1';
  }();
  const EpiMaps* em_ptr = (staged && !force_direct) ? &em : nullptr;

  CUtensorMap tmA, tmB;
  int rc;
  if (a_mn)
    rc = cached_map(&tmA, a, M, K, lda, 64, BK);
  else
    rc = cached_map(&tmA, a, K, M, lda, BK, BM);
  if (rc) return 1000 + rc;
  const uint64_t b_rows = dual ? static_cast<uint64_t>(epi->dual_rows) : static_cast<uint64_t>(N);
  if (b_mn)
    rc = cached_map(&tmB, b, N, K, ldb, 64, BK);
  else
    rc = cached_map(&tmB, b, K, b_rows, ldb, BK, dual ? bn / 2 : bn);
  if (rc) return 1000 + rc;

#define SFL_DISPATCH(EPI_)                                                                    \
  case EPI_:                                                                                  \
    return bn == 256 ? launch_major<256, EPI_>(a_mn, b_mn, tmA, tmB, em_ptr, p, max_ctas, stream) \
                     : launch_major<128, EPI_>(a_mn, b_mn, tmA, tmB, em_ptr, p, max_ctas, stream);
  switch (kind) {
    SFL_DISPATCH(EPI_BF16)
    SFL_DISPATCH(EPI_F32)
    SFL_DISPATCH(EPI_RESID)
    SFL_DISPATCH(EPI_ROPE)
    SFL_DISPATCH(EPI_SWIGLU_BWD)
    case EPI_SWIGLU:
      return launch_major<256, EPI_SWIGLU>(a_mn, b_mn, tmA, tmB, em_ptr, p, max_ctas, stream);
    default:
      return -2;
  }
#undef SFL_DISPATCH
}

// Weight gradients of up to four linear layers in one launch; see the kernel.
// Every matrix must be addressable by TMA (16-byte aligned base and pitch);
// returns -2 otherwise so the caller can fall back to one product at a time.
extern "C" int sfl_gemm_tp_set_spin_limit(unsigned iterations) {
  return static_cast<int>(cudaMemcpyToSymbol(sfl::g_tp_spin_limit, &iterations, sizeof(iterations)));
}

extern "C" int sfl_gemm_wgrad_grouped(const SflWgradProblem* problems, int count, int* status,
                                      void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (problems == nullptr || count <= 0 || count > kMaxGroup) return -2;
  GroupedMaps maps{};
  GroupedParams p{};
  p.count = count;
  p.status = status;
  int tiles = 0;
  for (int g = 0; g < count; ++g) {
    const SflWgradProblem& w = problems[g];
    if (w.rows <= 0 || w.cols <= 0 || w.tokens <= 0) return -2;
    auto aligned = [](const void* ptr, long ld, int elem) {
      return ptr != nullptr && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && ld > 0 &&
             (ld * elem) % 16 == 0;
    };
    if (!aligned(w.dy, w.ld_dy, 2) || !aligned(w.x, w.ld_x, 2) || !aligned(w.grad, w.ld_grad, 4))
      return -2;
    int rc = cached_map(&maps.a[g], w.dy, w.rows, w.tokens, w.ld_dy, 64, BK);
    if (rc == 0) rc = cached_map(&maps.b[g], w.x, w.cols, w.tokens, w.ld_x, 64, BK);
    if (rc == 0)
      rc = cached_map(&maps.out[g], w.grad, w.cols, w.rows, w.ld_grad, 32, 32, 4);
    if (rc) return 1000 + rc;
    GroupedProblem& q = p.prob[g];
    q.m_tiles = (w.rows + BM - 1) / BM;
    q.n_tiles = (w.cols + kGroupBN - 1) / kGroupBN;
    q.num_kb = (w.tokens + BK - 1) / BK;
    q.tile_begin = tiles;
    q.cols = w.cols;
    q.beta = w.accumulate;
    tiles += q.m_tiles * q.n_tiles;
  }
  p.total_tiles = tiles;
  using Cfg = GemmConfig<kGroupBN, EPI_F32, true>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(wgrad_grouped_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Cfg::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  const int grid = tiles < sm_count() ? tiles : sm_count();
  return launch_pdl(wgrad_grouped_kernel, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, stream, maps, p);
}

// ---- GEMM + all-reduce over peer memory (see gemm_tp_kernel) ----
namespace {
unsigned long long* g_tp_trace = nullptr;

long tp_tiles(int M, int N) {
  return static_cast<long>((M + BM - 1) / BM) * ((N + kTpBN - 1) / kTpBN);
}
}  // namespace

// Six 64-bit counters in device memory (or NULL to stop): summed nanoseconds of the
// five phases of CTA 0's first tile in every later sfl_gemm_tp_reduce, and a count.
extern "C" int sfl_gemm_tp_set_trace(void* counters) {
  g_tp_trace = static_cast<unsigned long long*>(counters);
  return 0;
}

extern "C" long sfl_gemm_tp_stage_bytes(int M, int N, int world) {
  if (M <= 0 || N <= 0 || world <= 0) return 0;
  return static_cast<long>(world) * tp_tiles(M, N) * BM * kTpBN * 2;
}

extern "C" long sfl_gemm_tp_tile_flag_bytes(int M, int N) {
  if (M <= 0 || N <= 0) return 0;
  return tp_tiles(M, N) * kMaxPeers * kEpiWarps * static_cast<long>(sizeof(uint32_t));
}

extern "C" int sfl_gemm_tp_reduce(const void* a, long lda, const void* b, long ldb, int b_mn, int M,
                                  int N, int K, const SflTpFuse* tp, long out_off_bytes,
                                  int out_bf16, const float* resid, long ldresid, int slot,
                                  unsigned epoch, unsigned tile_epoch, int* status,
                                  void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (tp == nullptr || M <= 0 || N <= 0 || K <= 0) return -2;
  if (tp->world < 2 || tp->world > kMaxPeers || tp->rank < 0 || tp->rank >= tp->world) return -2;
  if (N % kTpBN != 0 || (lda & 7) || (ldb & 7) || (out_off_bytes & 15)) return -2;
  if (slot < 0 || slot >= kSlots) return -2;
  if ((reinterpret_cast<uintptr_t>(a) & 15) || (reinterpret_cast<uintptr_t>(b) & 15)) return -2;
  if (!out_bf16 &&
      (resid == nullptr || (reinterpret_cast<uintptr_t>(resid) & 15) || (ldresid & 3)))
    return -2;

  GemmParams p{};
  p.M = M;
  p.N = N;
  p.K = K;
  p.num_m_tiles = (M + BM - 1) / BM;
  p.num_n_tiles = N / kTpBN;
  p.status = status;
  TpFuse f{};
  f.rank = tp->rank;
  f.world = tp->world;
  for (int i = 0; i < tp->world; ++i) {
    if (tp->stage[i] == nullptr || tp->out[i] == nullptr || tp->tile_flags[i] == nullptr ||
        tp->flags[i] == nullptr)
      return -2;
    f.stage[i] = static_cast<char*>(tp->stage[i]);
    f.out[i] = static_cast<char*>(tp->out[i]);
    f.tile_flags[i] = static_cast<uint32_t*>(tp->tile_flags[i]);
    f.flags[i] = static_cast<uint32_t*>(tp->flags[i]);
  }
  f.out_off = out_off_bytes;
  f.resid = resid;
  f.ldresid = ldresid;
  f.slot = slot;
  f.epoch = epoch;
  f.tile_epoch = tile_epoch;
  f.trace = g_tp_trace;

  CUtensorMap tmA, tmB;
  int rc = cached_map(&tmA, a, K, M, lda, BK, BM);
  if (rc) return 1000 + rc;
  if (b_mn)
    rc = cached_map(&tmB, b, N, K, ldb, 64, BK);
  else
    rc = cached_map(&tmB, b, K, N, ldb, BK, kTpBN);
  if (rc) return 1000 + rc;

  using Cfg = GemmConfig<kTpBN, EPI_F32, true>;
  const long tiles = tp_tiles(M, N);
  const int grid = tiles < sm_count() ? static_cast<int>(tiles) : sm_count();
  auto go = [&](auto kernel) -> int {
    cudaError_t e =
        cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    return launch_pdl(kernel, dim3(grid), dim3(kThreads), Cfg::kSmemBytes, stream, tmA, tmB, p, f);
  };
  // Two ranks: each sends its whole bf16 partial to the other and both finish every
  // row themselves (one transfer phase, 2 bytes per element).  More ranks: tiles are
  // owned round-robin, partials go to the owner and finished rows to everyone
  // (2 (W-1)/W transfers of the matrix instead of W-1).  SFL_TP_ONE_SHOT=0|1 overrides.
  static const int forced = [] {
    const char* v = getenv("SFL_TP_ONE_SHOT");
    return v == nullptr ? -1 : atoi(v);
  }();
  const bool one_shot = forced < 0 ? tp->world == 2 : forced != 0;
  if (one_shot) {
    if (b_mn)
      return out_bf16 ? go(gemm_tp_kernel<true, true, true>) : go(gemm_tp_kernel<true, false, true>);
    return out_bf16 ? go(gemm_tp_kernel<false, true, true>) : go(gemm_tp_kernel<false, false, true>);
  }
  if (b_mn)
    return out_bf16 ? go(gemm_tp_kernel<true, true, false>) : go(gemm_tp_kernel<true, false, false>);
  return out_bf16 ? go(gemm_tp_kernel<false, true, false>) : go(gemm_tp_kernel<false, false, false>);
}
