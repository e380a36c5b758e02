// Block-sparse flash attention for sm_100a: forward, dQ and dK/dV kernels.
//
// All three kernels share one structure.  A CTA owns a 128-row tile (queries for
// forward/dQ, keys for dK/dV) of one (batch, head) and walks the 128-wide tiles
// of the other sequence that a block schedule retains.  Warp 0 streams tiles in
// with TMA, warp 1 issues tcgen05.mma into tensor memory, and four warps (one
// thread per tile row) do the softmax math on accumulators read with tcgen05.ld,
// write the probability / dS tile back to shared memory in the 128-byte-swizzled
// layout the next MMA reads, and finish with the epilogue.
//
// Schedules come in two forms, as in the reference (attention_lab/
// triton_attention.py:125-323): a CSR over query tiles (row_ptr, col_idx, a
// "full" flag per stored tile, plus a 64-bit bitmap of the 16x16 sub-blocks that
// are present so schedules compiled at finer granularity keep their meaning), or
// an interval form whose tile range is derived from the window arithmetically.
// Partial tiles evaluate the token-level predicate (causal, left/right window,
// same-document); full tiles skip it.  Math follows the reference: scores are
// scaled after the dot product, softmax statistics are fp32, P is rounded to the
// input dtype before P V, rows without any visible key give O = 0, LSE = -inf,
// and LSE is a natural logarithm.  The backward pass mirrors attention_lab/
// backward.py:64-142: delta = rowsum(O dO); dQ owned by query tiles; dK/dV owned
// by key tiles walking the transposed schedule; no atomics.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdlib.h>

#include "launch.cuh"
#include "ptx.cuh"
#include "sfl.h"
#include "tensormap.cuh"

namespace sfl {

constexpr int kTile = 128;          // rows and columns of a score tile
constexpr int kAttnThreads = 192;   // forward: producer warp, MMA warp, 4 softmax warps
constexpr int kBwdThreads = 320;    // backward: producer, MMA, two compute warpgroups
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

struct AttnSchedule {
  int mode;  // 0 = CSR, 1 = interval
  const int* row_ptr;
  const int* col_idx;
  const uint8_t* full;
  const unsigned long long* bitmap;  // optional; bit (qs*8+ks) = 16x16 sub-block present
  int causal;
  int window_left;   // -1 = unbounded
  int window_right;  // -1 = unbounded
  const int* doc;    // optional document label per position
};

struct AttnParams {
  int B, H, N;
  float scale;
  AttnSchedule sched;
  // forward outputs / backward inputs
  void* o;
  const void* d_o;        // backward: upstream gradient, laid out like O
  long o_sb, o_sh, o_st;  // element strides of O (and dO) for batch, head, token
  float* lse;             // [B,H,N]
  float* delta;           // [B,H,N]
  // backward outputs (same element strides as the q/k/v they mirror)
  void* dq;
  void* dk;
  void* dv;
  long g_sb, g_sh, g_st;
  // Optional: dQ and dK leave the kernel already multiplied by the transposed
  // rotary matrix of their position (tables are [N, D/2], interleaved pairs).
  const float* rope_cos;
  const float* rope_sin;
  int is_fp16;
  int* status;
};

// ---- element type helpers -------------------------------------------------
template <bool FP16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (FP16) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  } else {
    return pack_bf16(a, b);
  }
}
template <bool FP16>
__device__ __forceinline__ float2 unpack2(uint32_t v) {
  if constexpr (FP16) {
    return __half22float2(*reinterpret_cast<__half2*>(&v));
  } else {
    return unpack_bf16(v);
  }
}
template <bool FP16>
__device__ __forceinline__ float round_elem(float a) {
  if constexpr (FP16) return __half2float(__float2half_rn(a));
  return bf16_round(a);
}
template <bool FP16>
__device__ __forceinline__ float load_elem(const void* p, long i) {
  if constexpr (FP16) return __half2float(static_cast<const __half*>(p)[i]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}

__host__ __device__ constexpr uint32_t idesc_16bit(bool fp16, int m, int n, bool a_mn, bool b_mn) {
  const uint32_t fmt = fp16 ? 0u : 1u;
  return (1u << 4) | (fmt << 7) | (fmt << 10) | (static_cast<uint32_t>(a_mn) << 15) |
         (static_cast<uint32_t>(b_mn) << 16) | (static_cast<uint32_t>(n >> 3) << 17) |
         (static_cast<uint32_t>(m >> 4) << 24);
}

// ---- schedule walking -----------------------------------------------------
struct TileRange {
  int begin, end;            // CSR: [row_ptr[r], row_ptr[r+1]); interval: tile indices
  int full_begin, full_end;  // interval mode only
};

// Tiles of the other sequence retained for `tile` (a query tile, or a key tile
// when `transposed`).  Interval bounds follow the same arithmetic as the host
// mirror in attention/flash.py (interval_regions).
__device__ __forceinline__ TileRange tile_range(const AttnSchedule& s, int tile, int N,
                                                bool transposed) {
  TileRange r;
  if (s.mode == 0) {
    r.begin = s.row_ptr[tile];
    r.end = s.row_ptr[tile + 1];
    r.full_begin = r.full_end = 0;
    return r;
  }
  const int first = tile * kTile;
  const int last = min(first + kTile, N) - 1;
  // For a query tile: keys in [q - L, q + R].  For a key tile the roles of the
  // windows swap: queries in [k - R, k + L].
  int left = transposed ? (s.causal ? 0 : s.window_right) : s.window_left;
  int right = transposed ? s.window_left : (s.causal ? 0 : s.window_right);
  const int lo = left < 0 ? 0 : max(0, first - left);
  const int hi = right < 0 ? N - 1 : min(N - 1, last + right);
  r.begin = lo / kTile;
  r.end = hi / kTile + 1;
  const int first_full = left < 0 ? 0 : max(0, last - left);
  int fb = (first_full + kTile - 1) / kTile;
  fb = min(r.end, max(r.begin, fb));
  int fe = (right < 0 || first + right >= N - 1) ? r.end : (first + right + 1) / kTile;
  fe = max(fb, min(r.end, fe));
  r.full_begin = fb;
  r.full_end = fe;
  return r;
}

struct TileInfo {
  int other;  // index of the tile of the other sequence
  bool full;
  unsigned long long bitmap;
};

__device__ __forceinline__ TileInfo tile_info(const AttnSchedule& s, const TileRange& r, int it) {
  TileInfo t;
  if (s.mode == 0) {
    const int e = r.begin + it;
    t.other = s.col_idx[e];
    t.full = s.full[e] != 0;
    t.bitmap = s.bitmap != nullptr ? s.bitmap[e] : ~0ull;
  } else {
    t.other = r.begin + it;
    t.full = t.other >= r.full_begin && t.other < r.full_end;
    t.bitmap = ~0ull;
  }
  return t;
}

// Token-level predicate in interval form.  For the thread that owns one row of a
// score tile, the permitted columns c (relative to the tile's first column) are
// exactly those with (unsigned)(c - rel_lo) < len; document labels and dropped
// sub-blocks are applied on top.  Keeping the test to one subtract, one compare
// and one select per element keeps the unrolled loops small.
struct RowMask {
  int rel_lo;
  uint32_t len;
};

// Thread owns query q; columns are keys col0 + c.
__device__ __forceinline__ RowMask row_mask_for_query(const AttnSchedule& s, int q, int col0,
                                                      int N) {
  const int lo = s.window_left < 0 ? 0 : max(0, q - s.window_left);
  int hi = s.causal ? q : (s.window_right < 0 ? N - 1 : q + s.window_right);
  hi = min(hi, N - 1);
  RowMask m;
  m.rel_lo = lo - col0;
  m.len = (q < N && hi >= lo) ? static_cast<uint32_t>(hi - lo + 1) : 0u;
  return m;
}

// Thread owns key k; columns are queries col0 + c.
__device__ __forceinline__ RowMask row_mask_for_key(const AttnSchedule& s, int k, int col0, int N) {
  const int lo = s.causal ? k : (s.window_right < 0 ? 0 : max(0, k - s.window_right));
  const int hi = s.window_left < 0 ? N - 1 : min(N - 1, k + s.window_left);
  RowMask m;
  m.rel_lo = lo - col0;
  m.len = (k < N && hi >= lo) ? static_cast<uint32_t>(hi - lo + 1) : 0u;
  return m;
}

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Sets masked scores to -inf.  `group_bits` has bit g set when columns
// [16g, 16g+16) of this row's sub-block row are present in the schedule.
__device__ __forceinline__ void apply_mask(float (&x)[kTile], const RowMask& m,
                                           uint32_t group_bits) {
#pragma unroll
  for (int g = 0; g < kTile / 16; ++g) {
    const uint32_t len = (group_bits >> g) & 1u ? m.len : 0u;
#pragma unroll
    for (int c = g * 16; c < g * 16 + 16; ++c)
      x[c] = static_cast<uint32_t>(c - m.rel_lo) < len ? x[c] : -INFINITY;
  }
}

__device__ __forceinline__ void apply_doc_mask(float (&x)[kTile], const int* col_doc, int my_doc) {
#pragma unroll
  for (int c = 0; c < kTile; ++c) x[c] = col_doc[c] == my_doc ? x[c] : -INFINITY;
}

// ---- shared-memory tile writer -------------------------------------------
// Writes one row (128 values, already packed in pairs) of a [128 x 128] 16-bit
// tile into the K-major 128-byte-swizzled layout: two column halves of
// [128 rows][128 bytes]; 16-byte chunk c of row r lives at chunk (c ^ (r & 7)).
__device__ __forceinline__ void store_row_swizzled(uint8_t* tile, int row,
                                                   const uint32_t (&packed)[64]) {
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    uint8_t* base = tile + half * (kTile * 128) + row * 128;
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint4 v = make_uint4(packed[half * 32 + c * 4 + 0], packed[half * 32 + c * 4 + 1],
                           packed[half * 32 + c * 4 + 2], packed[half * 32 + c * 4 + 3]);
      *reinterpret_cast<uint4*>(base + ((c ^ (row & 7)) << 4)) = v;
    }
  }
}

// Descriptors of the k-th 16-wide reduction step.
//   K-major tile of [rows][W] 16-bit elements stored as W/64 column halves.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t base, int rows, int k) {
  return umma_smem_desc(base + (k >> 2) * (rows * 128) + (k & 3) * 32, 16, 1024);
}
//   MN-major view of a [128 reduction rows][W] tile: step k covers rows 16k..16k+15.
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t base, int k) {
  return umma_smem_desc(base + k * 2048, kTile * 128, 1024);
}

__device__ __forceinline__ void named_barrier_128() {
  asm volatile("bar.sync 1, 128;" ::: "memory");
}

__device__ __forceinline__ void tmem_ld_32x32f(uint32_t taddr, float* dst) {
  uint32_t r[32];
  tmem_ld_32x32(taddr, r);
#pragma unroll
  for (int i = 0; i < 32; ++i) dst[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const float* src) {
  uint32_t a[16], b[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    a[i] = __float_as_uint(src[i]);
    b[i] = __float_as_uint(src[16 + i]);
  }
  tmem_st_32x16(taddr, a);
  tmem_st_32x16(taddr + 16, b);
}

// A wait gives up after about two seconds by the global timer.  (An iteration count alone
// is no bound: mbarrier.try_wait may suspend the thread for an implementation-defined time
// per call, and millions of such calls have taken minutes on a barrier that never completed.)
__device__ __forceinline__ bool bounded_wait(uint64_t* bar, uint32_t parity, volatile int* abort,
                                             int* status, int code) {
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
        if (now - started > 2000000000ull) break;
      }
    }
  }
  report_status(status, code);
  *abort = 1;
  return false;
}

// Load the operand tile(s) for rows [row0, row0+128) of (b, h): D/64 boxes.
template <int D>
__device__ __forceinline__ void load_rows(uint8_t* dst, const CUtensorMap* map, uint64_t* bar,
                                          int row0, int h, int b) {
#pragma unroll
  for (int i = 0; i < D / 64; ++i)
    tma_load_4d(dst + i * (kTile * 128), map, bar, i * 64, row0, h, b);
}

// ============================================================== forward ====
template <int D>
struct FwdSmem {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kPBytes = kTile * kTile * 2;
  static constexpr int kPBufs = (D == 64) ? 2 : 1;
  static constexpr int kStages = 2;
  // two query tiles (the next work item's is prefetched), K and V rings, P tiles
  static constexpr int kBytes = kTileBytes * (2 + 2 * kStages) + kPBytes * kPBufs + 1024 + 1024;
};

struct FwdBarriers {
  uint64_t q_full[2], q_empty[2];
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full[2];
  uint64_t p_ready[2];
  uint64_t pv_done[2];
  uint32_t tmem_base;
  int abort;
  int col_doc[kTile];  // document labels of the current key tile
};

// Persistent forward kernel.  A work item is one 128-row query tile of one
// (batch, head); items are numbered heaviest first (last query tiles of every
// head before earlier ones) and dealt to the CTAs in rounds of alternating
// direction (CTA c takes item c, then 2 grid - 1 - c, then 2 grid + c, ...), which
// evens out the causal imbalance: 8+4+4 and 6+6+2+2 key tiles rather than
// 8+6+4+2 and 6+4+2.
// Barriers, tensor memory and the operand rings are set up once per CTA; every
// role keeps running counters, so stage indices and barrier phases continue
// across items and the next item's query tile and first scores are already in
// flight while the current item's last P V products and its epilogue finish.
template <int D, bool FP16>
__global__ void __launch_bounds__(kAttnThreads, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
  using L = FwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;  // two tiles
  uint8_t* sK = sQ + 2 * L::kTileBytes;
  uint8_t* sV = sK + L::kStages * L::kTileBytes;
  uint8_t* sP = sV + L::kStages * L::kTileBytes;
  FwdBarriers* bars = reinterpret_cast<FwdBarriers*>(sP + L::kPBufs * L::kPBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_q_tiles = (p.N + kTile - 1) / kTile;
  const int BH = p.B * p.H;
  const int num_items = num_q_tiles * BH;
  const int rounds = (num_items + static_cast<int>(gridDim.x) - 1) / static_cast<int>(gridDim.x);
  auto item_tile = [&](int w) { return num_q_tiles - 1 - w / BH; };
  // item of this CTA in round r, or -1 when the last round has none for it
  auto item_at = [&](int r) {
    const int G = gridDim.x, c = blockIdx.x;
    const int w = r * G + ((r & 1) ? G - 1 - c : c);
    return w < num_items ? w : -1;
  };

  if (threadIdx.x == 0) {
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->q_full[s], 1);
      mbar_init(&bars->q_empty[s], 1);
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->p_ready[s], 128);
      mbar_init(&bars->pv_done[s], 1);
    }
    bars->abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  pdl_launch_dependents();  // set-up done: the next kernel may start its own
  pdl_wait();               // inputs of this kernel are complete from here on
  const uint32_t tS = tmem;        // two score buffers: columns [0,128) and [128,256)
  const uint32_t tO = tmem + 256;  // output accumulator: D columns
  volatile int* abort = &bars->abort;
  constexpr int PB = L::kPBufs;

  if (warp == 0) {
    // ------------------------------------------------------ TMA producer ----
    if (lane == 0) {
      uint32_t it = 0;  // key tiles loaded so far (all items)
      uint32_t qi = 0;  // query tiles loaded so far
      bool ok = true;
      for (int r = 0; r < rounds && ok; ++r) {
        const int w = item_at(r);
        if (w < 0) continue;
        const int q_tile = item_tile(w), bh = w % BH;
        const int b = bh / p.H, h = bh % p.H;
        const TileRange range = tile_range(p.sched, q_tile, p.N, false);
        const int n_tiles = range.end - range.begin;
        if (n_tiles <= 0) continue;
        const int qb = qi & 1;
        if (!bounded_wait(&bars->q_empty[qb], ((qi >> 1) & 1) ^ 1, abort, p.status,
                          kStatusTimeoutEmpty))
          break;
        mbar_expect_tx(&bars->q_full[qb], L::kTileBytes);
        load_rows<D>(sQ + qb * L::kTileBytes, &tmQ, &bars->q_full[qb], q_tile * kTile, h, b);
        ++qi;
        for (int j = 0; j < n_tiles; ++j, ++it) {
          const TileInfo t = tile_info(p.sched, range, j);
          const int s = it & 1;
          const uint32_t ph = ((it >> 1) & 1) ^ 1;
          if (!bounded_wait(&bars->k_empty[s], ph, abort, p.status, kStatusTimeoutEmpty) ) {
            ok = false;
            break;
          }
          mbar_expect_tx(&bars->k_full[s], L::kTileBytes);
          load_rows<D>(sK + s * L::kTileBytes, &tmK, &bars->k_full[s], t.other * kTile, h, b);
          if (!bounded_wait(&bars->v_empty[s], ph, abort, p.status, kStatusTimeoutEmpty)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&bars->v_full[s], L::kTileBytes);
          load_rows<D>(sV + s * L::kTileBytes, &tmV, &bars->v_full[s], t.other * kTile, h, b);
        }
      }
    }
  } else if (warp == 1) {
    // -------------------------------------------------------- MMA issuer ----
    if (lane == 0) {
      constexpr uint32_t idesc_qk = idesc_16bit(FP16, kTile, kTile, false, false);
      constexpr uint32_t idesc_pv = idesc_16bit(FP16, kTile, D, false, true);
      // Cursor of the score products, which run two key tiles ahead of P V and
      // therefore cross into the next work item before the current one is done.
      int qr = 0, qj = 0, qn = 0;  // round, tile within the item, tiles of the item
      uint32_t q_it = 0, q_qi = 0;
      auto seek = [&]() {  // first round at or after qr whose item has key tiles
        qj = 0;
        qn = 0;
        for (; qr < rounds; ++qr) {
          const int w = item_at(qr);
          if (w < 0) continue;
          const TileRange t = tile_range(p.sched, item_tile(w), p.N, false);
          if (t.end - t.begin > 0) {
            qn = t.end - t.begin;
            return;
          }
        }
      };
      auto issue_qk = [&]() -> bool {
        if (qn == 0) return true;  // no work item left
        const int qb = q_qi & 1;
        if (qj == 0 &&
            !bounded_wait(&bars->q_full[qb], (q_qi >> 1) & 1, abort, p.status, kStatusTimeoutFull))
          return false;
        const int s = q_it & 1;
        if (!bounded_wait(&bars->k_full[s], (q_it >> 1) & 1, abort, p.status, kStatusTimeoutFull))
          return false;
        tc_fence_after();
        const uint32_t q_addr = smem_u32(sQ + qb * L::kTileBytes);
        const uint32_t k_addr = smem_u32(sK + s * L::kTileBytes);
#pragma unroll
        for (int k = 0; k < D / 16; ++k)
          umma_bf16_ss(tS + s * kTile, desc_kmajor(q_addr, kTile, k), desc_kmajor(k_addr, kTile, k),
                       idesc_qk, k != 0);
        umma_commit(&bars->k_empty[s]);
        umma_commit(&bars->s_full[s]);
        ++q_it;
        if (++qj == qn) {  // last score product of the item: its query tile is free
          umma_commit(&bars->q_empty[qb]);
          ++q_qi;
          ++qr;
          seek();
        }
        return true;
      };
      seek();
      bool ok = issue_qk();
      if (ok) ok = issue_qk();
      uint32_t it = 0;
      for (int r = 0; r < rounds && ok; ++r) {
        const int w = item_at(r);
        if (w < 0) continue;
        const TileRange range = tile_range(p.sched, item_tile(w), p.N, false);
        const int n_tiles = range.end - range.begin;
        for (int j = 0; j < n_tiles && ok; ++j, ++it) {
          const int pb = it % PB;
          const int s = it & 1;
          if (!bounded_wait(&bars->p_ready[pb], (it / PB) & 1, abort, p.status,
                            kStatusTimeoutTmemFull) ||
              !bounded_wait(&bars->v_full[s], (it >> 1) & 1, abort, p.status,
                            kStatusTimeoutFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t p_addr = smem_u32(sP + pb * L::kPBytes);
          const uint32_t v_addr = smem_u32(sV + s * L::kTileBytes);
#pragma unroll
          for (int k = 0; k < kTile / 16; ++k)
            umma_bf16_ss(tO, desc_kmajor(p_addr, kTile, k), desc_mnmajor(v_addr, k), idesc_pv,
                         (j | k) != 0);
          umma_commit(&bars->v_empty[s]);
          umma_commit(&bars->pv_done[pb]);
          // the score buffer of tile it + 2 is the one tile `it` just released
          ok = issue_qk();
        }
      }
    }
  } else {
    // ------------------------------------------------ softmax + epilogue ----
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float scale_log2 = p.scale * kLog2e;
    uint32_t it = 0;
    bool ok = true;
    for (int r = 0; r < rounds && ok; ++r) {
      const int w = item_at(r);
      if (w < 0) continue;
      const int q_tile = item_tile(w), bh = w % BH;
      const int b = bh / p.H, h = bh % p.H;
      const TileRange range = tile_range(p.sched, q_tile, p.N, false);
      const int n_tiles = range.end - range.begin;
      const int q = q_tile * kTile + row;
      float m_used = -INFINITY;
      float l = 0.f;
      for (int j = 0; j < n_tiles && ok; ++j, ++it) {
        const TileInfo t = tile_info(p.sched, range, j);
        const int s = it & 1;
        const int pb = it % PB;
        if (!bounded_wait(&bars->s_full[s], (it >> 1) & 1, abort, p.status,
                          kStatusTimeoutTmemFull)) {
          ok = false;
          break;
        }
        tc_fence_after();
        float x[kTile];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_32x32f(tS + lane_base + s * kTile + c * 32, x + c * 32);
        tmem_ld_wait();
        const int k0 = t.other * kTile;
        const bool ragged = (k0 + kTile > p.N) || (q_tile * kTile + kTile > p.N);
        if (!t.full || ragged) {
          const RowMask rm = row_mask_for_query(p.sched, q, k0, p.N);
          apply_mask(x, rm, static_cast<uint32_t>(t.bitmap >> ((row >> 4) * 8)) & 0xffu);
          if (p.sched.doc != nullptr) {
            named_barrier_128();  // previous readers of the label tile are done
            bars->col_doc[row] = k0 + row < p.N ? p.sched.doc[k0 + row] : -1;
            named_barrier_128();
            apply_doc_mask(x, bars->col_doc, q < p.N ? p.sched.doc[q] : -2);
          }
        }
        // Row maximum of the raw scores; the positive scale preserves the order.
        // (eight independent chains: one 127-long dependent chain of max operations
        // would cost its full latency on a warp that has its scheduler to itself)
        float mx8[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) mx8[c] = x[c];
#pragma unroll
        for (int c = 8; c < kTile; ++c) mx8[c & 7] = fmaxf(mx8[c & 7], x[c]);
        float mx = fmaxf(fmaxf(fmaxf(mx8[0], mx8[1]), fmaxf(mx8[2], mx8[3])),
                         fmaxf(fmaxf(mx8[4], mx8[5]), fmaxf(mx8[6], mx8[7])));
        mx *= scale_log2;
        // Lazy rescale: keep a stale maximum until it is off by more than 2^8.
        const bool grow = mx > m_used + 8.0f;
        if (__any_sync(0xffffffffu, grow)) {
          if (j > 0) {
            if (!bounded_wait(&bars->pv_done[(it - 1) % PB], ((it - 1) / PB) & 1, abort, p.status,
                              kStatusTimeoutTmemFull)) {
              ok = false;
              break;
            }
            tc_fence_after();
            const float alpha = grow ? fast_exp2(m_used - mx) : 1.0f;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              float o[32];
              tmem_ld_32x32f(tO + lane_base + c * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] *= alpha;
              tmem_st_32x32(tO + lane_base + c * 32, o);
            }
            tmem_st_wait();
            l *= alpha;
          }
          if (grow) m_used = mx;
        }
        uint32_t packed[64];
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};  // independent partial sums, same reason
        // A row that has seen no key yet keeps m_used = -inf; subtract 0 instead so
        // masked scores (-inf) still map to probability 0 rather than NaN.
        const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
#pragma unroll
        for (int c = 0; c < kTile; c += 2) {
          const float p0 = fast_exp2(fmaf(x[c], scale_log2, neg_m));
          const float p1 = fast_exp2(fmaf(x[c + 1], scale_log2, neg_m));
          sum4[(c >> 1) & 3] += p0 + p1;
          packed[c >> 1] = pack2<FP16>(p0, p1);
        }
        l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        // the P tile is free once the product that read it PB tiles ago is done
        if (it >= PB && !bounded_wait(&bars->pv_done[pb], ((it - PB) / PB) & 1, abort, p.status,
                                      kStatusTimeoutTmemFull)) {
          ok = false;
          break;
        }
        store_row_swizzled(sP + pb * L::kPBytes, row, packed);
        fence_proxy_async_smem();
        tc_fence_before();
        mbar_arrive(&bars->p_ready[pb]);
      }
      if (ok && n_tiles > 0)
        ok = bounded_wait(&bars->pv_done[(it - 1) % PB], ((it - 1) / PB) & 1, abort, p.status,
                          kStatusTimeoutTmemFull);
      if (!ok) break;
      tc_fence_after();
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      uint8_t* orow = static_cast<uint8_t*>(p.o) +
                      2 * (b * p.o_sb + h * p.o_sh + static_cast<long>(q) * p.o_st);
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        float o[32];
        if (n_tiles > 0) {
          tmem_ld_32x32f(tO + lane_base + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0.f;
        }
        if (q < p.N && SFL_BOUNDS_OK(q >= 0 && b >= 0 && b < p.B && h >= 0 && h < p.H, p.status)) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack2<FP16>(o[8 * i + 0] * inv, o[8 * i + 1] * inv);
            v.y = pack2<FP16>(o[8 * i + 2] * inv, o[8 * i + 3] * inv);
            v.z = pack2<FP16>(o[8 * i + 4] * inv, o[8 * i + 5] * inv);
            v.w = pack2<FP16>(o[8 * i + 6] * inv, o[8 * i + 7] * inv);
            *reinterpret_cast<uint4*>(orow + (c * 32 + i * 8) * 2) = v;
          }
        }
      }
      if (q < p.N && p.lse != nullptr)
        p.lse[(static_cast<long>(b) * p.H + h) * p.N + q] =
            l > 0.f ? (m_used + log2f(l)) * kLn2 : -INFINITY;
      // The accumulator is overwritten by the next item's first P V product, which
      // waits for this warp's next p_ready arrival - i.e. after the reads above.
      tc_fence_before();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ===================================================== forward, two streams ====
// Head dimension 64.  With one 128-row query tile per CTA the tensor pipe finishes
// a score tile and a P V product in about 500 cycles while the softmax of the tile
// needs 16,384 exponentials - over 1,000 cycles of the SM's special-function units -
// and every hand-over between the two costs a barrier round trip, so a CTA that
// alternates them leaves both units idle most of the time.  Here a CTA runs TWO
// independent streams of work items (slots).  Each slot is a complete pipeline of
// its own: a TMA warp, an MMA warp, a softmax warpgroup, a query tile, K/V rings, a
// score tile and an output accumulator in tensor memory.  The slots share nothing
// but the SM, so whenever one of them waits (for its scores, for its probabilities)
// the other one has the tensor pipe and the special-function units:
//
//   tensor pipe :  S0=Q0 K0(j)^T | O1+=P1 V1(j-1), S1=Q1 K1(j)^T | O0+=P0 V0(j), S0=... |
//   softmax 0   :                  max/exp of S0(j) ........... P0 |                      ...
//   softmax 1   :  ... exp of S1(j-1) .. P1 |                        max/exp of S1(j) ..
//
// P is written back over its own score tile in tensor memory as packed 16-bit
// pairs and fed to the P V product as the A operand from tensor memory
// (tcgen05.mma with a tensor-memory A operand), which also lifts the shared-memory
// read limit of 128 x 64 x 16 products (4 KB of A per instruction); P_TMEM = false
// keeps P in a swizzled shared-memory tile instead.
//
// Work items are numbered heaviest first and dealt to the 2 x grid slots in rounds
// of alternating direction, as in the one-stream kernel below.
//
// Inside a slot the softmax warps copy a finished score tile into registers and hand
// the tensor-memory tile straight back (s_free), so the MMA warp issues S(j+1) while
// the softmax of tile j is still computing: when its P tile is written, the next
// scores are already there and the turn-around of the tensor pipe (barrier, issue,
// execution, commit: about 2,000 cycles) is off the critical path.  P therefore has
// columns of its own next to the score tile (per slot: S 128, P 64, O 64 columns of
// tensor memory).  Before the softmax warps touch P or the accumulator again they
// wait for the previous P V product (pv_done), which by then has long finished.
constexpr int kFwd2Threads = 384;  // per slot: TMA warp, MMA warp, softmax warpgroup

template <bool P_TMEM>
struct Fwd2Smem {
  static constexpr int kTileBytes = kTile * 64 * 2;  // one 128 x 64 operand tile
  static constexpr int kPBytes = kTile * kTile * 2;
  static constexpr int kQBufs = P_TMEM ? 2 : 1;  // next item's query tile prefetched
  static constexpr int kStages = 2;
  static constexpr int kSlotBytes =
      kTileBytes * (kQBufs + 2 * kStages) + (P_TMEM ? 0 : kPBytes);
  static constexpr int kSharedBytes = 1536;  // Fwd2Shared
  static constexpr int kBytes = 2 * kSlotBytes + kSharedBytes + 1024;
};

struct Fwd2SlotBars {
  uint64_t q_full[2], q_empty[2];
  uint64_t k_full[2], k_empty[2], v_full[2], v_empty[2];
  uint64_t s_full;   // score tile complete (MMA commit)
  uint64_t s_free;   // score tile copied to registers (128 arrivals)
  uint64_t p_ready;  // P tile written, accumulator rescaled (128 arrivals)
  uint64_t pv_done;  // P V product complete (MMA commit); the item's last one ends it
  uint64_t o_free;   // epilogue has read the accumulator (128 arrivals)
  int col_doc[kTile];
};

struct Fwd2Shared {
  Fwd2SlotBars slot[2];
  uint32_t tmem_base;
  int abort;
};
static_assert(sizeof(Fwd2Shared) <= Fwd2Smem<true>::kSharedBytes, "shared control block too large");

// Work items of one slot: item w covers query tile (num_q_tiles - 1 - w / BH) of
// (batch, head) w % BH; slot g of G takes w = r G + (r odd ? G - 1 - g : g).
struct SlotWalk {
  int G, g, rounds, num_items, r;
  __device__ __forceinline__ int next() {
    while (r < rounds) {
      const int rr = r++;
      const int w = rr * G + ((rr & 1) ? G - 1 - g : g);
      if (w < num_items) return w;
    }
    return -1;
  }
};

__device__ __forceinline__ void named_barrier_slot(int slot) {
  asm volatile("bar.sync %0, 128;" ::"r"(slot + 1) : "memory");
}

// Phase timers of CTA 0 (cycles, summed), compiled in with -DSFL_ATTN_TRACE and read back
// with sfl_attn_trace_read: softmax warp 0 of slot 0 - [0] waiting for scores, [1] loading
// them, [2] row maximum and rescale, [3] exponentials and P store, [4] epilogue, [5] tiles;
// [6] waiting for the previous P V product; MMA warp of slot 0 - [8] waiting for P and V,
// [9] issuing a P V product, [10] waiting for the score tile to be free and for K (and Q),
// [11] issuing a score product, [12] tiles.
// Backward (sfl_attn_bwd_trace_read; 16 entries for the dQ kernel, then 16 for the dK/dV
// kernel; CTA (0, 0), the heaviest one under a causal mask): compute warp 2 - [0] tile set-up,
// [1] waiting for a score half, [3] loading scores and dP, [4] exponentials, dS and the stores
// to tensor memory, [2] waiting for those stores and publishing, [5] halves, [6] epilogue;
// MMA warp - [8] waiting for the streamed tile and issuing scores, [9] waiting for P / dS,
// [10] issuing the accumulations, [12] halves; [13] cycles and [15] nanoseconds in the kernel;
// with -DSFL_ATTN_TRACE_SERIAL the MMA warp also waits for each batch it issued and adds up
// [11] issue-to-completion cycles of the score batches and [14] of the accumulation batches.
#ifdef SFL_ATTN_TRACE
__device__ unsigned long long g_attn_trace[48];
__device__ unsigned long long g_attn_stamps[64];  // globaltimer of CTA 0: see SFL_STAMP uses
__device__ __forceinline__ void attn_stamp(int at) {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  if (at < 64) g_attn_stamps[at] = t;
}
#define SFL_STAMP(cond, at) if (cond) attn_stamp(at);
#define SFL_TRACE_DECL(cond)      \
  const bool tracing_ = (cond);   \
  long long trace_t_ = clock64();
#define SFL_TRACE_MARK(slot)                                                          \
  if (tracing_) {                                                                     \
    const long long now_ = clock64();                                                 \
    atomicAdd(&g_attn_trace[slot], static_cast<unsigned long long>(now_ - trace_t_)); \
    trace_t_ = now_;                                                                  \
  }
#define SFL_TRACE_COUNT(slot) \
  if (tracing_) atomicAdd(&g_attn_trace[slot], 1ull);
#define SFL_TRACE_TOTAL(cond, base)                                                            \
  if (cond) {                                                                                  \
    unsigned long long ns1_;                                                                   \
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(ns1_));                                    \
    atomicAdd(&g_attn_trace[(base) + 13], static_cast<unsigned long long>(clock64() - t0_));   \
    atomicAdd(&g_attn_trace[(base) + 15], ns1_ - ns0_);                                        \
  }
#define SFL_TRACE_BEGIN()                                  \
  const long long t0_ = clock64();                         \
  unsigned long long ns0_;                                 \
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(ns0_));
#else
#define SFL_TRACE_DECL(cond)
#define SFL_TRACE_MARK(slot)
#define SFL_TRACE_COUNT(slot)
#define SFL_TRACE_TOTAL(cond, base)
#define SFL_TRACE_BEGIN()
#define SFL_STAMP(cond, at)
#endif

template <bool FP16, bool P_TMEM>
__global__ void __launch_bounds__(kFwd2Threads, 1)
attn_fwd2_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                 const __grid_constant__ CUtensorMap tmV, const AttnParams p) {
#ifdef SFL_ATTN_TRACE
  const long long kernel_t0 = clock64();
  unsigned long long kernel_ns0;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(kernel_ns0));
#endif
  SFL_STAMP(blockIdx.x == 0 && threadIdx.x == 0, 0)
  constexpr int D = 64;
  using L = Fwd2Smem<P_TMEM>;
  constexpr int QB = L::kQBufs;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  Fwd2Shared* sh = reinterpret_cast<Fwd2Shared*>(smem + 2 * L::kSlotBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // warps 0, 1: TMA and MMA of slot 0; warps 2, 3: of slot 1; warps 4-7 and 8-11: softmax
  const int w = warp < 4 ? (warp >> 1) : ((warp - 4) >> 2);
  uint8_t* slot_base = smem + w * L::kSlotBytes;
  uint8_t* sQ = slot_base;                        // QB tiles
  uint8_t* sK = slot_base + QB * L::kTileBytes;   // kStages tiles
  uint8_t* sV = sK + L::kStages * L::kTileBytes;  // kStages tiles
  uint8_t* sP = sV + L::kStages * L::kTileBytes;  // only when !P_TMEM
  Fwd2SlotBars& bar = sh->slot[w];

  const int num_q_tiles = (p.N + kTile - 1) / kTile;
  const int BH = p.B * p.H;
  const int num_items = num_q_tiles * BH;
  const int G = 2 * static_cast<int>(gridDim.x);
  const int rounds = (num_items + G - 1) / G;
  SlotWalk walk{G, 2 * static_cast<int>(blockIdx.x) + w, rounds, num_items, 0};
  auto item_tile = [&](int item) { return num_q_tiles - 1 - item / BH; };

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      Fwd2SlotBars& b = sh->slot[i];
      for (int s = 0; s < 2; ++s) {
        mbar_init(&b.q_full[s], 1);
        mbar_init(&b.q_empty[s], 1);
        mbar_init(&b.k_full[s], 1);
        mbar_init(&b.k_empty[s], 1);
        mbar_init(&b.v_full[s], 1);
        mbar_init(&b.v_empty[s], 1);
      }
      mbar_init(&b.s_full, 1);
      mbar_init(&b.s_free, 128);
      mbar_init(&b.p_ready, 128);
      mbar_init(&b.pv_done, 1);
      mbar_init(&b.o_free, 128);
    }
    sh->abort = 0;
    mbar_fence_init();
    prefetch_tensormap(&tmQ);
    prefetch_tensormap(&tmK);
    prefetch_tensormap(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(&sh->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = sh->tmem_base;
  SFL_STAMP(blockIdx.x == 0 && threadIdx.x == 0, 1)
  pdl_launch_dependents();
  pdl_wait();
  SFL_STAMP(blockIdx.x == 0 && threadIdx.x == 0, 2)
  volatile int* abort = &sh->abort;
  // tensor memory of a slot: scores [0,128), P as 16-bit pairs [128,192), output [192,256)
  const uint32_t tS = tmem + static_cast<uint32_t>(w * 256);
  const uint32_t tP = tS + 128;
  const uint32_t tO = tS + 192;

  if (warp == 0 || warp == 2) {
    // ---------------------------------------------------- TMA producer ----
    if (lane == 0) {
      uint32_t it = 0, qi = 0;
      int item;
      bool ok = true;
      while (ok && (item = walk.next()) >= 0) {
        const int q_tile = item_tile(item), bh = item % BH;
        const int b = bh / p.H, h = bh % p.H;
        const TileRange range = tile_range(p.sched, q_tile, p.N, false);
        const int n_tiles = range.end - range.begin;
        if (n_tiles <= 0) continue;
        const int qb = qi % QB;
        if (!bounded_wait(&bar.q_empty[qb], ((qi / QB) & 1) ^ 1, abort, p.status,
                          kStatusTimeoutEmpty))
          break;
        mbar_expect_tx(&bar.q_full[qb], L::kTileBytes);
        load_rows<D>(sQ + qb * L::kTileBytes, &tmQ, &bar.q_full[qb], q_tile * kTile, h, b);
        ++qi;
        for (int j = 0; j < n_tiles; ++j, ++it) {
          const int other = tile_info(p.sched, range, j).other;
          const int s = it & 1;
          const uint32_t ph = ((it >> 1) & 1) ^ 1;
          if (!bounded_wait(&bar.k_empty[s], ph, abort, p.status, kStatusTimeoutEmpty)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&bar.k_full[s], L::kTileBytes);
          load_rows<D>(sK + s * L::kTileBytes, &tmK, &bar.k_full[s], other * kTile, h, b);
          if (!bounded_wait(&bar.v_empty[s], ph, abort, p.status, kStatusTimeoutEmpty)) {
            ok = false;
            break;
          }
          mbar_expect_tx(&bar.v_full[s], L::kTileBytes);
          load_rows<D>(sV + s * L::kTileBytes, &tmV, &bar.v_full[s], other * kTile, h, b);
        }
      }
    }
  } else if (warp == 1 || warp == 3) {
    // ------------------------------------------------------ MMA issuer ----
    // The whole warp walks the loop and waits on the barriers together; one elected
    // lane issues.  With warp-uniform control flow the descriptors, tensor-memory
    // addresses and loop counters live in uniform registers, which is where
    // tcgen05.mma takes its operands from: issuing from inside a single-lane branch
    // costs a register-to-uniform move per operand and made the issue of a 128 x 64 x 16
    // product slower than its execution.
    {
      constexpr uint32_t idesc_qk = idesc_16bit(FP16, kTile, kTile, false, false);
      constexpr uint32_t idesc_pv = idesc_16bit(FP16, kTile, D, false, true);
      // descriptors of the first reduction step of every buffer; the others follow by
      // constant offsets
      const uint64_t q_desc0 = desc_kmajor(smem_u32(sQ), kTile, 0);
      const uint64_t k_desc0 = desc_kmajor(smem_u32(sK), kTile, 0);
      const uint64_t v_desc0 = desc_mnmajor(smem_u32(sV), 0);
      const uint64_t p_desc0 = desc_kmajor(smem_u32(sP), kTile, 0);
      (void)p_desc0;
      // The score products run one tile ahead of the P V products: a second cursor over
      // the same item sequence.
      SlotWalk qk_walk = walk;
      int qk_n = 0, qk_j = 0;
      bool qk_done = false;
      auto qk_advance = [&]() {
        qk_n = qk_j = 0;
        int next_item;
        while ((next_item = qk_walk.next()) >= 0) {
          const TileRange t = tile_range(p.sched, item_tile(next_item), p.N, false);
          if (t.end - t.begin > 0) {
            qk_n = t.end - t.begin;
            return;
          }
        }
        qk_done = true;
      };
      uint32_t qk_it = 0, q_qi = 0;
      SFL_TRACE_DECL(blockIdx.x == 0 && warp == 1 && lane == 0)
      auto issue_qk = [&](bool after_tile, uint32_t prev) -> bool {
        if (qk_done) return true;
        const int qb = q_qi % QB;
        const int s = qk_it & 1;
        if (after_tile &&
            !bounded_wait(&bar.s_free, prev & 1, abort, p.status, kStatusTimeoutTmemEmpty))
          return false;
        if (qk_j == 0 && !bounded_wait(&bar.q_full[qb], (q_qi / QB) & 1, abort, p.status,
                                       kStatusTimeoutFull))
          return false;
        if (!bounded_wait(&bar.k_full[s], (qk_it >> 1) & 1, abort, p.status, kStatusTimeoutFull))
          return false;
        tc_fence_after();
        SFL_TRACE_MARK(10)
        const uint64_t qd = umma_desc_advance(q_desc0, qb * L::kTileBytes);
        const uint64_t kd = umma_desc_advance(k_desc0, s * L::kTileBytes);
        const bool last = qk_j + 1 == qk_n;
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < D / 16; ++k)
            umma_bf16_ss(tS, umma_desc_advance(qd, k * 32), umma_desc_advance(kd, k * 32),
                         idesc_qk, k != 0);
          umma_commit(&bar.s_full);
          if (last) umma_commit(&bar.q_empty[qb]);
        }
        __syncwarp();
        ++qk_it;
        if (++qk_j == qk_n) {
          ++q_qi;
          qk_advance();
        }
        SFL_TRACE_MARK(11)
        return true;
      };
      qk_advance();
      bool ok = issue_qk(false, 0);
      uint32_t it = 0, items = 0;
      int item;
      while (ok && (item = walk.next()) >= 0) {
        const TileRange range = tile_range(p.sched, item_tile(item), p.N, false);
        const int n_tiles = range.end - range.begin;
        if (n_tiles <= 0) continue;
        for (int j = 0; j < n_tiles && ok; ++j, ++it) {
          // scores of the next tile as soon as the softmax warps have copied this one
          ok = issue_qk(true, it);
          if (!ok) break;
          const int s = it & 1;
          if (!bounded_wait(&bar.p_ready, it & 1, abort, p.status, kStatusTimeoutTmemFull) ||
              !bounded_wait(&bar.v_full[s], (it >> 1) & 1, abort, p.status, kStatusTimeoutFull) ||
              (j == 0 && items > 0 &&
               !bounded_wait(&bar.o_free, (items - 1) & 1, abort, p.status,
                             kStatusTimeoutTmemEmpty))) {
            ok = false;
            break;
          }
          tc_fence_after();
          SFL_TRACE_MARK(8)
          const uint64_t vd = umma_desc_advance(v_desc0, s * L::kTileBytes);
          if (elect_one()) {
            if constexpr (P_TMEM) {
#pragma unroll
              for (int k = 0; k < kTile / 16; ++k)
                umma_bf16_ts(tO, tP + k * 8, umma_desc_advance(vd, k * 2048), idesc_pv,
                             (j | k) != 0);
            } else {
#pragma unroll
              for (int k = 0; k < kTile / 16; ++k)
                umma_bf16_ss(tO,
                             umma_desc_advance(p_desc0, (k >> 2) * (kTile * 128) + (k & 3) * 32),
                             umma_desc_advance(vd, k * 2048), idesc_pv, (j | k) != 0);
            }
            umma_commit(&bar.pv_done);
          }
          __syncwarp();
          if (j == n_tiles - 1) ++items;
          SFL_TRACE_MARK(9)
          SFL_TRACE_COUNT(12)
        }
      }
    }
  } else {
    // ------------------------------------------------ softmax + epilogue ----
    const int quarter = warp & 3;  // tensor-memory lane quarter this warp may access
    const int row = quarter * 32 + lane;
    const bool leader = (warp & 3) == 0 && lane == 0;  // hands K/V stages back
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float scale_log2 = p.scale * kLog2e;
    uint32_t it = 0;     // key tiles processed by this slot
    uint32_t items = 0;  // items with key tiles finished by this slot
    bool ok = true;
    int item;
    SFL_TRACE_DECL(blockIdx.x == 0 && warp == 4 && lane == 0)
    while (ok && (item = walk.next()) >= 0) {
      const int q_tile = item_tile(item), bh = item % BH;
      const int b = bh / p.H, h = bh % p.H;
      const TileRange range = tile_range(p.sched, q_tile, p.N, false);
      const int n_tiles = range.end - range.begin;
      const int q = q_tile * kTile + row;
      float m_used = -INFINITY;
      float l = 0.f;
      for (int j = 0; j < n_tiles && ok; ++j, ++it) {
        const TileInfo t = tile_info(p.sched, range, j);
        if (!bounded_wait(&bar.s_full, it & 1, abort, p.status, kStatusTimeoutTmemFull)) {
          ok = false;
          break;
        }
        tc_fence_after();
        if (leader) mbar_arrive(&bar.k_empty[it & 1]);  // the score product has read K(j)
        SFL_STAMP(blockIdx.x == 0 && warp == 4 && lane == 0, 8 + 2 * static_cast<int>(it))
        SFL_TRACE_MARK(0)
        float x[kTile];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_32x32f(tS + lane_base + c * 32, x + c * 32);
        tmem_ld_wait();
        tc_fence_before();
        mbar_arrive(&bar.s_free);  // the next scores may overwrite the tile
        SFL_TRACE_MARK(1)
        const int k0 = t.other * kTile;
        const bool ragged = (k0 + kTile > p.N) || (q_tile * kTile + kTile > p.N);
        if (!t.full || ragged) {
          const RowMask rm = row_mask_for_query(p.sched, q, k0, p.N);
          apply_mask(x, rm, static_cast<uint32_t>(t.bitmap >> ((row >> 4) * 8)) & 0xffu);
          if (p.sched.doc != nullptr) {
            named_barrier_slot(w);  // previous readers of the label tile are done
            bar.col_doc[row] = k0 + row < p.N ? p.sched.doc[k0 + row] : -1;
            named_barrier_slot(w);
            apply_doc_mask(x, bar.col_doc, q < p.N ? p.sched.doc[q] : -2);
          }
        }
        // three-input maxima: 64 instructions instead of 127, in eight independent chains
        float mx8[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) mx8[c] = fmaxf(x[2 * c], x[2 * c + 1]);
#pragma unroll
        for (int c = 16; c < kTile; c += 2) mx8[(c >> 1) & 7] = fmax3(mx8[(c >> 1) & 7], x[c], x[c + 1]);
        float mx = fmax3(fmax3(mx8[0], mx8[1], mx8[2]), fmax3(mx8[3], mx8[4], mx8[5]),
                         fmaxf(mx8[6], mx8[7]));
        mx *= scale_log2;
        SFL_TRACE_MARK(2)
        // P and the accumulator belong to the previous P V product until it is done.
        if (j > 0) {
          if (!bounded_wait(&bar.pv_done, (it - 1) & 1, abort, p.status, kStatusTimeoutTmemFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (leader) mbar_arrive(&bar.v_empty[(it - 1) & 1]);
        }
        SFL_TRACE_MARK(6)
        // Lazy rescale: keep a stale maximum until it is off by more than 2^8.
        const bool grow = mx > m_used + 8.0f;
        if (__any_sync(0xffffffffu, grow)) {
          if (j > 0) {
            const float alpha = grow ? fast_exp2(m_used - mx) : 1.0f;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              float o[32];
              tmem_ld_32x32f(tO + lane_base + c * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] *= alpha;
              tmem_st_32x32(tO + lane_base + c * 32, o);
            }
            l *= alpha;
          }
          if (grow) m_used = mx;
        }
        const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        if constexpr (P_TMEM) {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint32_t packed[16];
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float p0 = fast_exp2(fmaf(x[c * 32 + i], scale_log2, neg_m));
              const float p1 = fast_exp2(fmaf(x[c * 32 + i + 1], scale_log2, neg_m));
              sum4[(i >> 1) & 3] += p0 + p1;
              packed[i >> 1] = pack2<FP16>(p0, p1);
            }
            // 16-bit pairs: 16 columns of tensor memory per 32 probabilities
            tmem_st_32x16(tP + lane_base + c * 16, packed);
          }
          tmem_st_wait();
        } else {
          uint32_t packed[64];
#pragma unroll
          for (int c = 0; c < kTile; c += 2) {
            const float p0 = fast_exp2(fmaf(x[c], scale_log2, neg_m));
            const float p1 = fast_exp2(fmaf(x[c + 1], scale_log2, neg_m));
            sum4[(c >> 1) & 3] += p0 + p1;
            packed[c >> 1] = pack2<FP16>(p0, p1);
          }
          store_row_swizzled(sP, row, packed);
          fence_proxy_async_smem();
          tmem_st_wait();  // a rescale's stores, if any
        }
        l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
        tc_fence_before();
        mbar_arrive(&bar.p_ready);
        SFL_STAMP(blockIdx.x == 0 && warp == 4 && lane == 0, 9 + 2 * static_cast<int>(it))
        SFL_TRACE_MARK(3)
        SFL_TRACE_COUNT(5)
      }
      if (!ok) break;
      if (n_tiles > 0) {  // the item's last P V product
        if (!bounded_wait(&bar.pv_done, (it - 1) & 1, abort, p.status, kStatusTimeoutTmemFull))
          break;
        tc_fence_after();
        if (leader) mbar_arrive(&bar.v_empty[(it - 1) & 1]);
      }
      const float inv = l > 0.f ? 1.0f / l : 0.f;
      uint8_t* orow = static_cast<uint8_t*>(p.o) +
                      2 * (b * p.o_sb + h * p.o_sh + static_cast<long>(q) * p.o_st);
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        float o[32];
        if (n_tiles > 0) {
          tmem_ld_32x32f(tO + lane_base + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0.f;
        }
        if (q < p.N && SFL_BOUNDS_OK(q >= 0 && b >= 0 && b < p.B && h >= 0 && h < p.H, p.status)) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack2<FP16>(o[8 * i + 0] * inv, o[8 * i + 1] * inv);
            v.y = pack2<FP16>(o[8 * i + 2] * inv, o[8 * i + 3] * inv);
            v.z = pack2<FP16>(o[8 * i + 4] * inv, o[8 * i + 5] * inv);
            v.w = pack2<FP16>(o[8 * i + 6] * inv, o[8 * i + 7] * inv);
            *reinterpret_cast<uint4*>(orow + (c * 32 + i * 8) * 2) = v;
          }
        }
      }
      if (n_tiles > 0) {  // the accumulator may be overwritten by the next item
        tc_fence_before();
        mbar_arrive(&bar.o_free);
        ++items;
      }
      if (q < p.N && p.lse != nullptr)
        p.lse[(static_cast<long>(b) * p.H + h) * p.N + q] =
            l > 0.f ? (m_used + log2f(l)) * kLn2 : -INFINITY;
      SFL_STAMP(blockIdx.x == 0 && warp == 4 && lane == 0, 40 + static_cast<int>(items))
      SFL_TRACE_MARK(4)
    }
  }
  tc_fence_before();
  __syncthreads();
  SFL_STAMP(blockIdx.x == 0 && threadIdx.x == 0, 3)
#ifdef SFL_ATTN_TRACE
  if (threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1)) {
    unsigned long long ns1;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(ns1));
    const int at = blockIdx.x == 0 ? 13 : 14;   // [13] CTA 0, [14] last CTA: cycles in the kernel
    atomicAdd(&g_attn_trace[at], static_cast<unsigned long long>(clock64() - kernel_t0));
    if (blockIdx.x == 0) atomicAdd(&g_attn_trace[15], ns1 - kernel_ns0);  // [15] nanoseconds, CTA 0
  }
#endif
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// ====================================================== decode on tensor cores ====
// Single-token attention over a KV cache with grouped queries, split over the cache.
// The scores of one (batch, KV head) are a [cached tokens] x [query heads of the group]
// matrix product and the output a [heads] x [tokens] x [D] one: K and V tiles of 128
// tokens stream in through TMA, S^T = K Q^T and O += P^T V run on tcgen05 with the
// accumulators in tensor memory.  Scalar-FMA decode needs about 125 warp instructions per
// cached token for eight heads at D = 128 and is bound by the issue rate at a quarter of
// the memory bandwidth; here the arithmetic per token is a handful of instructions and the
// kernel is bound by the K/V stream.
//
// A CTA handles one (batch, KV head, split) and leaves (m, l, u) in the log-2 domain for
// the merge, which the last CTA of a (batch, KV head) to finish performs (decode.cu has the
// same protocol).  Partitioning follows the reference (attention_lab/cuda_decode/
// decode.cu:50-52): split s covers tokens [s chunk, min(length, (s + 1) chunk)) with
// chunk = ceil(capacity / splits); empty partitions contribute (-inf, 0, 0).
//
// The score product has the 128 cached tokens of a tile as its rows and the (padded) head
// group as its N = 16 columns, so a softmax thread owns one token and touches G <= 8 scores
// per tile.  (With the head group as the rows of a 128-row query tile every thread owns a
// row of which all but G are padding and pays 128 exponentials per tile: that layout was
// built first and measured 15 % slower on every shape.)  The per-head maximum over the tile's tokens is a warp
// redux.sync on order-preserving integer keys plus one exchange through shared memory; the
// running maximum is the same in every thread.  P goes to shared memory transposed (heads
// as rows of a K-major tile of which only 16 rows exist; the product reads 128 and the
// rows beyond the group produce values nobody reads) and O[heads, D] += P^T V accumulates
// in tensor memory.
struct DecParams {
  const void* q;       // [B, Hq, D]
  const int* lengths;  // [B]
  float* part_m;       // [B, Hq, S]  (log2 domain)
  float* part_l;       // [B, Hq, S]
  float* part_u;       // [B, Hq, S, D]
  int* counters;       // [B, Hkv], zero between launches
  void* out;           // [B, Hq, D]
  int B, Hq, Hkv, N, splits, G;
  float scale;
  int* status;
};

__device__ __forceinline__ float dec_merge_exp2(float x) { return fast_exp2(x); }

constexpr int kDec2Threads = 192;  // TMA warp, MMA warp, four softmax warps (thread = token)

template <int D>
struct Dec2Smem {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kStages = D == 64 ? 5 : 3;
  static constexpr int kQBytes = 16 * D * 2;        // [D / 64 atoms][16 heads][128 B]
  static constexpr int kPBytes = 2 * 16 * 128;      // one buffer: [2 atoms][16 heads][128 B]
  // the A operand of P^T V is read as 128 rows: 16 KB past each atom must be mapped, which
  // the K/V ring behind the P buffers provides
  static constexpr int kBytes = kQBytes + 2 * kPBytes + 2 * kStages * kTileBytes + 1024 + 1024;
};

struct Dec2Barriers {
  uint64_t q_ready;  // 128 arrivals: the query tile is written
  uint64_t k_full[5], k_empty[5], v_full[5], v_empty[5];
  uint64_t s_full[2], s_free[2], p_ready[2], pv_done[2];
  uint32_t tmem_base;
  int abort;
  int is_last;
  alignas(16) int tile_max[2][4][8];  // order-preserving keys of the per-warp maxima, by tile parity
  alignas(16) float row_sum[4][8];
};

__device__ __forceinline__ int float_key(float x) {  // signed-integer order == float order
  const int i = __float_as_int(x);
  return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float key_float(int k) {
  return __int_as_float(k ^ ((k >> 31) & 0x7fffffff));
}
__device__ __forceinline__ int warp_max_s32(int v) {
  int r;
  asm volatile("redux.sync.max.s32 %0, %1, 0xffffffff;" : "=r"(r) : "r"(v));
  return r;
}
__device__ __forceinline__ void tmem_ld_32x8(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]),
                 "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}

template <int D, bool FP16>
__global__ void __launch_bounds__(kDec2Threads, 1)
decode_mma2_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV,
                   const DecParams p) {
  using L = Dec2Smem<D>;
  constexpr int ST = L::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = smem;
  uint8_t* sP = sQ + L::kQBytes;
  uint8_t* sK = sP + 2 * L::kPBytes;
  uint8_t* sV = sK + ST * L::kTileBytes;
  Dec2Barriers* bars = reinterpret_cast<Dec2Barriers*>(sV + ST * L::kTileBytes);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  int len = p.lengths[b];
  len = len < 0 ? 0 : (len > p.N ? p.N : len);
  const int chunk = (p.N + p.splits - 1) / p.splits;
  const int begin = split * chunk;
  const int end = min(len, begin + chunk);
  const int n_tiles = end > begin ? (end - begin + kTile - 1) / kTile : 0;

  if (threadIdx.x == 0) {
    mbar_init(&bars->q_ready, 128);
    for (int s = 0; s < ST; ++s) {
      mbar_init(&bars->k_full[s], 1);
      mbar_init(&bars->k_empty[s], 1);
      mbar_init(&bars->v_full[s], 1);
      mbar_init(&bars->v_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&bars->s_full[s], 1);
      mbar_init(&bars->s_free[s], 128);
      mbar_init(&bars->p_ready[s], 128);
      mbar_init(&bars->pv_done[s], 1);
    }
    bars->abort = 0;
    mbar_fence_init();
    prefetch_tensormap(&tmK);
    prefetch_tensormap(&tmV);
  }
  // columns: two score buffers of 16, then the output [heads, D]
  constexpr uint32_t kTmemCols = D == 64 ? 128 : 256;
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  volatile int* abort = &bars->abort;
  const uint32_t tO = tmem + 32;

  if (warp == 0) {
    // ---------------------------------------------------- TMA producer ----
    if (lane == 0) {
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % ST;
        const uint32_t ph = ((j / ST) & 1) ^ 1;
        const int row0 = begin + j * kTile;
        if (!bounded_wait(&bars->k_empty[s], ph, abort, p.status, kStatusTimeoutEmpty)) break;
        mbar_expect_tx(&bars->k_full[s], L::kTileBytes);
        load_rows<D>(sK + s * L::kTileBytes, &tmK, &bars->k_full[s], row0, kvh, b);
        if (!bounded_wait(&bars->v_empty[s], ph, abort, p.status, kStatusTimeoutEmpty)) break;
        mbar_expect_tx(&bars->v_full[s], L::kTileBytes);
        load_rows<D>(sV + s * L::kTileBytes, &tmV, &bars->v_full[s], row0, kvh, b);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------ MMA issuer ----
    if (n_tiles > 0) {
      constexpr uint32_t idesc_qk = idesc_16bit(FP16, kTile, 16, false, false);
      constexpr uint32_t idesc_pv = idesc_16bit(FP16, kTile, D, false, true);
      const uint64_t q_desc0 = desc_kmajor(smem_u32(sQ), 16, 0);
      const uint64_t k_desc0 = desc_kmajor(smem_u32(sK), kTile, 0);
      const uint64_t p_desc0 = desc_kmajor(smem_u32(sP), 16, 0);
      const uint64_t v_desc0 = desc_mnmajor(smem_u32(sV), 0);
      bool ok = bounded_wait(&bars->q_ready, 0, abort, p.status, kStatusTimeoutFull);
      for (int j = 0; j <= n_tiles && ok; ++j) {
        if (j < n_tiles) {  // S^T(j) = K(j) Q^T into score buffer j & 1
          const int s = j % ST, sb = j & 1;
          if (j >= 2 && !bounded_wait(&bars->s_free[sb], ((j >> 1) - 1) & 1, abort, p.status,
                                      kStatusTimeoutTmemEmpty)) {
            ok = false;
            break;
          }
          if (!bounded_wait(&bars->k_full[s], (j / ST) & 1, abort, p.status, kStatusTimeoutFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t kd = umma_desc_advance(k_desc0, s * L::kTileBytes);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < D / 16; ++k)
              umma_bf16_ss(tmem + sb * 16,
                           umma_desc_advance(kd, (k >> 2) * (kTile * 128) + (k & 3) * 32),
                           umma_desc_advance(q_desc0, (k >> 2) * (16 * 128) + (k & 3) * 32), idesc_qk,
                           k != 0);
            umma_commit(&bars->s_full[sb]);
            umma_commit(&bars->k_empty[s]);
          }
          __syncwarp();
        }
        if (j >= 1) {  // O += P^T(j - 1) V(j - 1)
          const int i = j - 1, s = i % ST, pb = i & 1;
          if (!bounded_wait(&bars->p_ready[pb], (i >> 1) & 1, abort, p.status, kStatusTimeoutTmemFull) ||
              !bounded_wait(&bars->v_full[s], (i / ST) & 1, abort, p.status, kStatusTimeoutFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t pd = umma_desc_advance(p_desc0, pb * L::kPBytes);
          const uint64_t vd = umma_desc_advance(v_desc0, s * L::kTileBytes);
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < kTile / 16; ++k)
              umma_bf16_ss(tO, umma_desc_advance(pd, (k >> 2) * (16 * 128) + (k & 3) * 32),
                           umma_desc_advance(vd, k * 2048), idesc_pv, (i | k) != 0);
            umma_commit(&bars->pv_done[pb]);
            umma_commit(&bars->v_empty[s]);
          }
          __syncwarp();
        }
      }
    }
  } else {
    // ------------------------------------------------ softmax + partials ----
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;  // token of the tile
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float scale_log2 = p.scale * kLog2e;
    const long head0 = static_cast<long>(b) * p.Hq + static_cast<long>(kvh) * p.G;
    // The query tile [16 heads][D], K-major and swizzled; rows beyond the group are zero.
    for (int idx = threadIdx.x - 64; idx < 16 * (D / 8); idx += 128) {
      const int g = idx / (D / 8), c = idx % (D / 8);  // head, 16-byte chunk of its row
      uint4 v = make_uint4(0, 0, 0, 0);
      if (g < p.G)
        v = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.q) +
                                            (head0 + g) * D * 2 + c * 16);
      *reinterpret_cast<uint4*>(sQ + (c >> 3) * (16 * 128) + g * 128 + (((c & 7) ^ (g & 7)) << 4)) = v;
    }
    fence_proxy_async_smem();
    mbar_arrive(&bars->q_ready);

    float m[8], l_part[8];
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      m[g] = -INFINITY;
      l_part[g] = 0.f;
    }
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int sb = j & 1;
      if (!bounded_wait(&bars->s_full[sb], (j >> 1) & 1, abort, p.status, kStatusTimeoutTmemFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      uint32_t raw[8];
      tmem_ld_32x8(tmem + lane_base + sb * 16, raw);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(&bars->s_free[sb]);
      const bool live = begin + j * kTile + row < end;  // token inside the partition
      float x[8];
      int key[8];
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        x[g] = live && g < p.G ? __uint_as_float(raw[g]) * scale_log2 : -INFINITY;
        key[g] = warp_max_s32(float_key(x[g]));
      }
      if (lane == 0) {
        *reinterpret_cast<int4*>(&bars->tile_max[sb][quarter][0]) = make_int4(key[0], key[1], key[2], key[3]);
        *reinterpret_cast<int4*>(&bars->tile_max[sb][quarter][4]) = make_int4(key[4], key[5], key[6], key[7]);
      }
      named_barrier_128();
      bool grow = false;
      float alpha[8];
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        int k = bars->tile_max[sb][0][g];
        k = max(k, bars->tile_max[sb][1][g]);
        k = max(k, bars->tile_max[sb][2][g]);
        k = max(k, bars->tile_max[sb][3][g]);
        const float mx = key_float(k);
        alpha[g] = 1.0f;
        if (mx > m[g] + 8.0f) {  // a stale maximum is kept until it is off by 2^8
          alpha[g] = fast_exp2(m[g] - mx);  // 0 for the first tile
          m[g] = mx;
          grow = true;
        }
      }
      // the P buffer of this parity was last read by the product of tile j - 2
      if (j >= 2 && !bounded_wait(&bars->pv_done[sb], ((j >> 1) - 1) & 1, abort, p.status,
                                  kStatusTimeoutTmemFull)) {
        ok = false;
        break;
      }
      if (grow) {  // the same decision in every thread: the maxima are CTA-wide
#pragma unroll
        for (int g = 0; g < 8; ++g) l_part[g] *= alpha[g];
        if (j >= 1) {
          if (!bounded_wait(&bars->pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort, p.status,
                            kStatusTimeoutTmemFull)) {
            ok = false;
            break;
          }
          tc_fence_after();
          if (quarter == 0) {  // output rows (heads) live in lanes 0 .. G-1
            float a = 1.0f;
#pragma unroll
            for (int g = 0; g < 8; ++g) a = lane == g ? alpha[g] : a;
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              float o[32];
              tmem_ld_32x32f(tO + c * 32, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] *= a;
              tmem_st_32x32(tO + c * 32, o);
            }
            tmem_st_wait();
          }
        }
      }
      // P^T: head g is row g of a K-major tile whose 128 columns are this tile's tokens
      uint8_t* pt = sP + sb * L::kPBytes + (row >> 6) * (16 * 128);
      const int chunk16 = (row & 63) >> 3, within = (row & 7) * 2;
#pragma unroll
      for (int g = 0; g < 8; ++g) {
        const float neg_m = m[g] == -INFINITY ? 0.f : -m[g];
        const float pr = fast_exp2(x[g] + neg_m);
        l_part[g] += pr;
        uint16_t bits;
        if constexpr (FP16)
          bits = __half_as_ushort(__float2half_rn(pr));
        else
          bits = __bfloat16_as_ushort(__float2bfloat16_rn(pr));
        *reinterpret_cast<uint16_t*>(pt + g * 128 + ((chunk16 ^ g) << 4) + within) = bits;
      }
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(&bars->p_ready[sb]);
    }
    if (ok && n_tiles > 0)
      ok = bounded_wait(&bars->pv_done[(n_tiles - 1) & 1], ((n_tiles - 1) >> 1) & 1, abort, p.status,
                        kStatusTimeoutTmemFull);
    // row sums: lanes, then the four warps in a fixed order
#pragma unroll
    for (int g = 0; g < 8; ++g) {
      float v = l_part[g];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      if (lane == 0) bars->row_sum[quarter][g] = v;
    }
    named_barrier_128();
    if (ok && quarter == 0) {
      // tcgen05.ld is a warp-wide instruction: every lane loads its row, only the lanes
      // that hold a head store it
      tc_fence_after();
      const int g = lane;
      const bool real = g < p.G;
      float l = 0.f, mg = -INFINITY;
      if (g < 8) {
        l = (bars->row_sum[0][g] + bars->row_sum[1][g]) + (bars->row_sum[2][g] + bars->row_sum[3][g]);
#pragma unroll
        for (int i = 0; i < 8; ++i) mg = g == i ? m[i] : mg;
      }
      const long head = head0 + (real ? g : 0);
      const long slot = head * p.splits + split;
      const bool direct = p.splits == 1;
      const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        float o[32];
        if (n_tiles > 0) {
          tmem_ld_32x32f(tO + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0.f;
        }
        if (!real) continue;
        if (direct) {
          uint8_t* orow = static_cast<uint8_t*>(p.out) + head * D * 2;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack2<FP16>(o[8 * i + 0] * inv, o[8 * i + 1] * inv);
            v.y = pack2<FP16>(o[8 * i + 2] * inv, o[8 * i + 3] * inv);
            v.z = pack2<FP16>(o[8 * i + 4] * inv, o[8 * i + 5] * inv);
            v.w = pack2<FP16>(o[8 * i + 6] * inv, o[8 * i + 7] * inv);
            *reinterpret_cast<uint4*>(orow + (c * 32 + i * 8) * 2) = v;
          }
        } else {
          float* urow = p.part_u + slot * D + c * 32;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<float4*>(urow + 4 * i) =
                make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        }
      }
      if (!direct && real) {
        p.part_m[slot] = l > 0.f ? mg : -INFINITY;
        p.part_l[slot] = l;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, kTmemCols);
  }
  if (p.splits == 1) return;

  // ---- the last CTA of this (batch, kv head) merges the splits ------------------
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(&p.counters[b * p.Hkv + kvh], 1);
    bars->is_last = ticket == p.splits - 1;
    if (bars->is_last) p.counters[b * p.Hkv + kvh] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!bars->is_last) return;
  __threadfence();
  const long head0 = static_cast<long>(b) * p.Hq + static_cast<long>(kvh) * p.G;
  for (int idx = threadIdx.x; idx < p.G * D; idx += blockDim.x) {
    const int gg = idx / D, d = idx % D;
    const long base = (head0 + gg) * p.splits;
    float mm = -INFINITY;
    for (int s = 0; s < p.splits; ++s) mm = fmaxf(mm, __ldcg(p.part_m + base + s));
    float ll = 0.f, uu = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float ms = __ldcg(p.part_m + base + s);
      const float a = (ms == -INFINITY || mm == -INFINITY) ? 0.f : dec_merge_exp2(ms - mm);
      ll += __ldcg(p.part_l + base + s) * a;
      uu += __ldcg(p.part_u + (base + s) * D + d) * a;
    }
    const float r = ll > 0.f ? uu / ll : 0.f;
    if constexpr (FP16)
      static_cast<__half*>(p.out)[(head0 + gg) * D + d] = __float2half_rn(r);
    else
      static_cast<__nv_bfloat16*>(p.out)[(head0 + gg) * D + d] = __float2bfloat16_rn(r);
  }
}

// ============================================================= backward ====
// Shared layout of the two backward kernels: an "owned" pair of resident tiles and a
// ring of streamed tile pairs, each stage with the per-column statistics (and document
// labels) of its streamed tile.  Probabilities and dS never touch shared memory: the
// compute warps write them back into tensor memory, over the scores they were made
// from, and the accumulation MMAs read them from there as their A operand.
template <int D>
struct BwdSmem {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kStages = (D == 64) ? 4 : 2;
  static constexpr int kStatBytes = kStages * (2 * kTile * 4 + kTile * 4);
  static constexpr int kBytes = 2 * kTileBytes + kStages * 2 * kTileBytes + kStatBytes + 1024 + 256;
};

struct BwdBarriers {
  uint64_t own_full;
  uint64_t in_full[4], in_empty[4];
  // Each streamed tile is processed as two halves of 64 columns, one per compute
  // warpgroup; the halves rotate through up to three score buffers; index = buffer.
  uint64_t sp_full[3];    // score and dP accumulator halves ready
  uint64_t pds_ready[3];  // P and dS of the half written to tensor memory (128 arrivals)
  uint64_t acc_done;      // every accumulation MMA finished
  uint64_t probe;         // -DSFL_ATTN_TRACE_SERIAL only: completion of one batch of MMAs
  uint32_t tmem_base;
  int abort;
};

// dK/dV kernel (KV_OWNED = true): CTA owns a key tile; streams (Q, dO) tiles.
//   S^T = K Q^T, dP^T = V dO^T, P^T = exp(S^T - lse_q), dS^T = P^T (dP^T - delta_q)
//   dV += P^T dO,  dK += dS^T Q
// dQ kernel (KV_OWNED = false): CTA owns a query tile; streams (K, V) tiles.
//   S = Q K^T, dP = dO V^T, P = exp(S - lse_q), dS = P (dP - delta_q)
//   dQ += dS K
//
// Roles: warp 0 streams tiles (TMA) and stages the statistics of their columns, warp 1
// issues the MMAs, warps 2-5 and 6-9 are two compute warpgroups.  Warpgroup g owns
// columns [64 g, 64 g + 64) of every streamed tile: it waits for that half of S and dP,
// turns it into P and dS, stores them as packed 16-bit pairs over the first 32 columns
// of the half it just read, and signals the MMA warp, which accumulates from tensor
// memory.  The stream of halves rotates through kBufs score buffers in tensor memory
// (three where 3 x 128 columns fit beside the accumulators, else two): the scores of
// half h + kBufs are issued right after the accumulation of half h, so with three
// buffers a warpgroup finds its next half computed when it finishes one and the
// exponentials, not the hand-overs, set the pace.  A 128 x 64 x 16 product with both
// operands in shared memory is bound by the 6 KB it reads (48 cycles measured); with A
// in tensor memory it runs at the pipe's 32 cycles.
template <int D, bool FP16, bool KV_OWNED>
__global__ void __launch_bounds__(kBwdThreads, 1)
attn_bwd_kernel(const __grid_constant__ CUtensorMap tmOwnA,  // K (kv-owned) or Q
                const __grid_constant__ CUtensorMap tmOwnB,  // V (kv-owned) or dO
                const __grid_constant__ CUtensorMap tmInA,   // Q (kv-owned) or K
                const __grid_constant__ CUtensorMap tmInB,   // dO (kv-owned) or V
                const AttnParams p) {
  using L = BwdSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr int ST = L::kStages;
  uint8_t* sOwnA = smem;
  uint8_t* sOwnB = sOwnA + L::kTileBytes;
  uint8_t* sIn = sOwnB + L::kTileBytes;  // stages x (A, B)
  float* sStats = reinterpret_cast<float*>(sIn + ST * 2 * L::kTileBytes);  // stages x (-lse[128], delta[128])
  int* sDoc = reinterpret_cast<int*>(sStats + ST * 2 * kTile);             // stages x labels[128]
  BwdBarriers* bars = reinterpret_cast<BwdBarriers*>(sDoc + ST * kTile);

  SFL_TRACE_BEGIN()
  constexpr int kTr = KV_OWNED ? 32 : 16;  // base of this kernel's phase timers
  (void)kTr;  // referenced only by the timers
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_tiles = (p.N + kTile - 1) / kTile;
  const int own_tile = KV_OWNED ? blockIdx.x : num_tiles - 1 - blockIdx.x;
  const int bh = blockIdx.y;
  const int b = bh / p.H, h = bh % p.H;
  const TileRange range = tile_range(p.sched, own_tile, p.N, KV_OWNED);
  const int n_tiles = range.end - range.begin;
  const long stat_base = (static_cast<long>(b) * p.H + h) * p.N;
  const bool have_doc = p.sched.doc != nullptr;

  if (threadIdx.x == 0) {
    mbar_init(&bars->own_full, 1);
    for (int s = 0; s < ST; ++s) {
      mbar_init(&bars->in_full[s], 1 + 32);  // the TMA transaction and the 32 staging lanes
      mbar_init(&bars->in_empty[s], 1);
    }
    for (int s = 0; s < 3; ++s) {
      mbar_init(&bars->sp_full[s], 1);
      mbar_init(&bars->pds_ready[s], 128);
    }
    mbar_init(&bars->acc_done, 1);
    mbar_init(&bars->probe, 1);
    bars->abort = 0;
    mbar_fence_init();
  }
  if (warp == 1) {
    tmem_alloc(&bars->tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = bars->tmem_base;
  pdl_launch_dependents();
  pdl_wait();
  // Score buffer i: S in columns [128 i, 128 i + 64), dP in the next 64; P and dS are
  // written over the first 32 columns of each.  The accumulators follow the buffers.
  constexpr int kBufs = (KV_OWNED && D == 128) ? 2 : 3;
  const uint32_t tAcc0 = tmem + kBufs * 128;      // dV (kv-owned) or dQ
  const uint32_t tAcc1 = tmem + kBufs * 128 + D;  // dK (kv-owned)
  volatile int* abort = &bars->abort;

  if (warp == 0) {
    // ------------------------------------------------------ producer ----
    if (n_tiles > 0) {
      if (lane == 0) {
        mbar_expect_tx(&bars->own_full, 2 * L::kTileBytes);
        load_rows<D>(sOwnA, &tmOwnA, &bars->own_full, own_tile * kTile, h, b);
        load_rows<D>(sOwnB, &tmOwnB, &bars->own_full, own_tile * kTile, h, b);
      }
      for (int j = 0; j < n_tiles; ++j) {
        const TileInfo t = tile_info(p.sched, range, j);
        const int s = j % ST;
        if (!bounded_wait(&bars->in_empty[s], ((j / ST) & 1) ^ 1, abort, p.status,
                          kStatusTimeoutEmpty))
          break;
        if (lane == 0) {
          mbar_expect_tx(&bars->in_full[s], 2 * L::kTileBytes);
          uint8_t* dst = sIn + s * 2 * L::kTileBytes;
          load_rows<D>(dst, &tmInA, &bars->in_full[s], t.other * kTile, h, b);
          load_rows<D>(dst + L::kTileBytes, &tmInB, &bars->in_full[s], t.other * kTile, h, b);
        }
        // Per-column data of the streamed tile, four columns per lane: (negated, log-2)
        // log-sum-exp and delta of the query columns for the key-owned kernel, document
        // labels for both.  They travel with the tile: the lanes arrive on its barrier.
        if (KV_OWNED || have_doc) {
          float* stats = sStats + s * (2 * kTile);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = lane * 4 + e;
            const int ci = t.other * kTile + col;
            if constexpr (KV_OWNED) {
              float ls = ci < p.N ? p.lse[stat_base + ci] * kLog2e : INFINITY;
              if (ls == -INFINITY) ls = INFINITY;  // query without keys: P = 0
              stats[col] = -ls;
              stats[kTile + col] = ci < p.N ? p.delta[stat_base + ci] : 0.f;
            }
            if (have_doc) sDoc[s * kTile + col] = ci < p.N ? p.sched.doc[ci] : -1;
          }
        }
        mbar_arrive(&bars->in_full[s]);
      }
    }
  } else if (warp == 1) {
    // ---------------------------------------------------- MMA issuer ----
    // The whole warp walks the loop; one elected lane issues, so that descriptors and
    // tensor-memory addresses stay in uniform registers (see attn_fwd2_kernel).
    if (n_tiles > 0) {
      constexpr uint32_t idesc_s = idesc_16bit(FP16, kTile, 64, false, false);
      constexpr uint32_t idesc_acc = idesc_16bit(FP16, kTile, D, false, true);
      // Descriptors are built once and stepped by constant offsets (see
      // umma_desc_advance): per MMA the issuing thread then only adds and issues.
      uint64_t own_a[D / 16], own_b[D / 16];
#pragma unroll
      for (int k = 0; k < D / 16; ++k) {
        own_a[k] = desc_kmajor(smem_u32(sOwnA), kTile, k);
        own_b[k] = desc_kmajor(smem_u32(sOwnB), kTile, k);
      }
      const uint64_t in_k0 = desc_kmajor(smem_u32(sIn), kTile, 0);   // streamed tile, K-major view
      const uint64_t in_mn0 = desc_mnmajor(smem_u32(sIn), 0);        // same tile, MN-major view
      // scores and dP of half h of the stream (tile h / 2, columns 64 (h % 2) ...)
      const int halves = 2 * n_tiles;
      auto issue_scores = [&](int h) -> bool {
        const int j = h >> 1, g = h & 1, s = j % ST, buf = h % kBufs;
        if (g == 0 &&
            !bounded_wait(&bars->in_full[s], (j / ST) & 1, abort, p.status, kStatusTimeoutFull))
          return false;
        tc_fence_after();
        // rows [64 g, 64 g + 64) of the streamed pair (A then B, kTileBytes apart)
        const uint64_t in_a = umma_desc_advance(in_k0, s * 2 * L::kTileBytes + g * 64 * 128);
        const uint64_t in_b = umma_desc_advance(in_a, L::kTileBytes);
        const uint32_t tS = tmem + buf * 128, tDP = tS + 64;
#ifdef SFL_ATTN_TRACE_SERIAL
        const long long issue_t0 = clock64();
#endif
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < D / 16; ++k)  // S^T = K Q^T   or   S = Q K^T
            umma_bf16_ss(tS, own_a[k],
                         umma_desc_advance(in_a, (k >> 2) * (kTile * 128) + (k & 3) * 32), idesc_s,
                         k != 0);
#pragma unroll
          for (int k = 0; k < D / 16; ++k)  // dP^T = V dO^T  or  dP = dO V^T
            umma_bf16_ss(tDP, own_b[k],
                         umma_desc_advance(in_b, (k >> 2) * (kTile * 128) + (k & 3) * 32), idesc_s,
                         k != 0);
          umma_commit(&bars->sp_full[buf]);
        }
        __syncwarp();
#ifdef SFL_ATTN_TRACE_SERIAL
        {  // [7] cycles spent issuing a score batch into an idle pipe, [11] from then to its completion
          const long long t0 = clock64();
          if (blockIdx.x == 0 && blockIdx.y == 0 && lane == 0)
            atomicAdd(&g_attn_trace[kTr + 7], static_cast<unsigned long long>(t0 - issue_t0));
          bounded_wait(&bars->sp_full[buf], (h / kBufs) & 1, abort, p.status, kStatusTimeoutTmemFull);
          if (blockIdx.x == 0 && blockIdx.y == 0 && lane == 0)
            atomicAdd(&g_attn_trace[kTr + 11], static_cast<unsigned long long>(clock64() - t0));
        }
#endif
        return true;
      };
      bool ok = bounded_wait(&bars->own_full, 0, abort, p.status, kStatusTimeoutFull);
      for (int h = 0; h < kBufs && h < halves && ok; ++h) ok = issue_scores(h);
      SFL_TRACE_DECL(blockIdx.x == 0 && blockIdx.y == 0 && lane == 0)
      for (int h = 0; h < halves && ok; ++h) {
        const int j = h >> 1, g = h & 1, s = j % ST, buf = h % kBufs;
        if (!bounded_wait(&bars->pds_ready[buf], (h / kBufs) & 1, abort, p.status,
                          kStatusTimeoutTmemFull))
          break;
        tc_fence_after();
        SFL_TRACE_MARK(kTr + 9)
        // MN-major views of the streamed pair: 16 reduction rows per step, 2048 B apart
        const uint64_t mn_a = umma_desc_advance(in_mn0, s * 2 * L::kTileBytes + g * 4 * 2048);
        const uint64_t mn_b = umma_desc_advance(mn_a, L::kTileBytes);
        const uint32_t a_p = tmem + buf * 128, a_ds = a_p + 64;  // 16 reduction columns = 8 words
        if (elect_one()) {
          if constexpr (KV_OWNED) {
#pragma unroll
            for (int k = 0; k < 4; ++k)  // dV += P^T dO
              umma_bf16_ts(tAcc0, a_p + k * 8, umma_desc_advance(mn_b, k * 2048), idesc_acc,
                           (h | k) != 0);
#pragma unroll
            for (int k = 0; k < 4; ++k)  // dK += dS^T Q
              umma_bf16_ts(tAcc1, a_ds + k * 8, umma_desc_advance(mn_a, k * 2048), idesc_acc,
                           (h | k) != 0);
          } else {
#pragma unroll
            for (int k = 0; k < 4; ++k)  // dQ += dS K
              umma_bf16_ts(tAcc0, a_ds + k * 8, umma_desc_advance(mn_a, k * 2048), idesc_acc,
                           (h | k) != 0);
          }
          if (g == 1) umma_commit(&bars->in_empty[s]);
          if (h + 1 == halves) umma_commit(&bars->acc_done);
#ifdef SFL_ATTN_TRACE_SERIAL
          umma_commit(&bars->probe);
#endif
        }
        __syncwarp();
#ifdef SFL_ATTN_TRACE_SERIAL
        {  // [14] the same for a batch of accumulation products
          const long long t0 = clock64();
          bounded_wait(&bars->probe, h & 1, abort, p.status, kStatusTimeoutTmemFull);
          if (blockIdx.x == 0 && blockIdx.y == 0 && lane == 0)
            atomicAdd(&g_attn_trace[kTr + 14], static_cast<unsigned long long>(clock64() - t0));
        }
#endif
        SFL_TRACE_MARK(kTr + 10)
        SFL_TRACE_COUNT(kTr + 12)
        // The buffer's next half: the tensor pipe is in order, so it overwrites this
        // half's P and dS only after the products above have read them.
        if (h + kBufs < halves && !issue_scores(h + kBufs)) break;
        SFL_TRACE_MARK(kTr + 8)
      }
    }
  } else {
    // ------------------------------------------------ compute warpgroups ----
    const int quarter = warp & 3;
    const int wg = (warp - 2) >> 2;  // the 64-column half of every streamed tile this warp works on
    const int row = quarter * 32 + lane;
    const int own_pos = own_tile * kTile + row;  // key index (kv-owned) or query index
    const uint32_t lane_base = static_cast<uint32_t>(quarter * 32) << 16;
    const float scale_log2 = p.scale * kLog2e;
    float my_lse = 0.f, my_delta = 0.f;
    if constexpr (!KV_OWNED) {
      // lse in log2 units; +inf for padding rows makes P vanish.
      my_lse = own_pos < p.N ? p.lse[stat_base + own_pos] * kLog2e : INFINITY;
      if (my_lse == -INFINITY) my_lse = INFINITY;  // row without keys: P = 0
      // delta = sum_d O * dO of this query row; published for the key-owned kernel,
      // which runs after this one.
      if (own_pos < p.N) {
        const long off = 2 * (b * p.o_sb + h * p.o_sh + static_cast<long>(own_pos) * p.o_st);
        const uint4* po = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.o) + off);
        const uint4* pg = reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(p.d_o) + off);
#pragma unroll
        for (int i = 0; i < D / 8; ++i) {
          const uint4 a = po[i], g = pg[i];
          const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
          const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 x = unpack2<FP16>(aw[e]);
            const float2 y = unpack2<FP16>(gw[e]);
            my_delta = fmaf(x.x, y.x, my_delta);
            my_delta = fmaf(x.y, y.y, my_delta);
          }
        }
        if (wg == 0) p.delta[stat_base + own_pos] = my_delta;
      }
    }
    const float neg_lse = -my_lse;
    bool ok = true;
    SFL_TRACE_DECL(blockIdx.x == 0 && blockIdx.y == 0 && warp == 2 && lane == 0)
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int s = j % ST;
      const TileInfo t = tile_info(p.sched, range, j);
      const int other0 = t.other * kTile;
      const bool ragged = (other0 + kTile > p.N) || (own_tile * kTile + kTile > p.N);
      const bool masked = !t.full || ragged;
      const bool use_doc = masked && have_doc;
      RowMask rm{0, 0u};
      uint32_t group_bits = 0xffu;
      int my_doc = -2;
      if (masked) {
        // The bitmap is indexed (query sub-block, key sub-block).
        if constexpr (KV_OWNED) {
          rm = row_mask_for_key(p.sched, own_pos, other0, p.N);
          group_bits = 0;
#pragma unroll
          for (int g = 0; g < 8; ++g)
            group_bits |= static_cast<uint32_t>((t.bitmap >> (g * 8 + (row >> 4))) & 1ull) << g;
        } else {
          rm = row_mask_for_query(p.sched, own_pos, other0, p.N);
          group_bits = static_cast<uint32_t>(t.bitmap >> ((row >> 4) * 8)) & 0xffu;
        }
        if (use_doc && own_pos < p.N) my_doc = p.sched.doc[own_pos];
      }
      const int hs = 2 * j + wg;  // position in the stream of halves
      const int buf = hs % kBufs;
      const uint32_t tS = tmem + buf * 128, tDP = tS + 64;
      SFL_TRACE_MARK(kTr + 0)
      if (!bounded_wait(&bars->sp_full[buf], (hs / kBufs) & 1, abort, p.status,
                        kStatusTimeoutTmemFull)) {
        ok = false;
        break;
      }
      // The staged statistics were published on the tile's own barrier, which completed
      // before the scores were issued: this wait returns at once and orders the reads.
      if ((KV_OWNED || use_doc) &&
          !bounded_wait(&bars->in_full[s], (j / ST) & 1, abort, p.status, kStatusTimeoutFull)) {
        ok = false;
        break;
      }
      tc_fence_after();
      SFL_TRACE_MARK(kTr + 1)
      const float* stats = sStats + s * (2 * kTile);
      const int* docs = sDoc + s * kTile;
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int c = 2 * wg + cc;  // 32-column chunk of the tile
        float sv[32], dp[32];
        uint32_t pp[16], dd[16];
        tmem_ld_32x32f(tS + lane_base + cc * 32, sv);
        tmem_ld_32x32f(tDP + lane_base + cc * 32, dp);
        tmem_ld_wait();
        SFL_TRACE_MARK(kTr + 3)
        if (masked) {
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            const uint32_t len = (group_bits >> (c * 2 + g)) & 1u ? rm.len : 0u;
#pragma unroll
            for (int i = g * 16; i < g * 16 + 16; ++i)
              sv[i] = static_cast<uint32_t>(c * 32 + i - rm.rel_lo) < len ? sv[i] : -INFINITY;
          }
          if (use_doc) {
#pragma unroll
            for (int i = 0; i < 32; ++i) sv[i] = docs[c * 32 + i] == my_doc ? sv[i] : -INFINITY;
          }
        }
        // Statistics of the 32 columns: the key-owned kernel reads them from the staged
        // table (the same address for every lane, so 16-byte loads), the query-owned
        // kernel has them in registers.
        const float* col_ls = stats + c * 32;
        const float* col_dl = col_ls + kTile;
#pragma unroll
        for (int i = 0; i < 32; i += 4) {
          float nl[4], dl[4];
          if constexpr (KV_OWNED) {
            const float4 a = *reinterpret_cast<const float4*>(col_ls + i);
            const float4 b4 = *reinterpret_cast<const float4*>(col_dl + i);
            nl[0] = a.x; nl[1] = a.y; nl[2] = a.z; nl[3] = a.w;
            dl[0] = b4.x; dl[1] = b4.y; dl[2] = b4.z; dl[3] = b4.w;
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              nl[e] = neg_lse;
              dl[e] = my_delta;
            }
          }
          float pr[4], ds[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            // exp2(-inf) = 0 covers both masked scores and rows without keys.
            pr[e] = fast_exp2(fmaf(sv[i + e], scale_log2, nl[e]));
            ds[e] = pr[e] * (dp[i + e] - dl[e]);
          }
          pp[i >> 1] = pack2<FP16>(pr[0], pr[1]);
          pp[(i >> 1) + 1] = pack2<FP16>(pr[2], pr[3]);
          dd[i >> 1] = pack2<FP16>(ds[0], ds[1]);
          dd[(i >> 1) + 1] = pack2<FP16>(ds[2], ds[3]);
        }
        // 32 columns of 16-bit values are 16 words: chunk cc of the half lands in
        // columns [16 cc, 16 cc + 16) of the half, all of which this warp has read.
        if constexpr (KV_OWNED) tmem_st_32x16(tS + lane_base + cc * 16, pp);
        tmem_st_32x16(tDP + lane_base + cc * 16, dd);
        SFL_TRACE_MARK(kTr + 4)
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&bars->pds_ready[buf]);
      SFL_TRACE_MARK(kTr + 2)
      SFL_TRACE_COUNT(kTr + 5)
    }
    if (ok && n_tiles > 0)
      ok = bounded_wait(&bars->acc_done, 0, abort, p.status, kStatusTimeoutTmemFull);
    if (ok) {
      tc_fence_after();
      const long goff = 2 * (b * p.g_sb + h * p.g_sh + static_cast<long>(own_pos) * p.g_st);
      auto write_acc = [&](uint32_t taddr, void* dst_base, float mul, bool rotate) {
        uint8_t* dst = static_cast<uint8_t*>(dst_base) + goff;
#pragma unroll
        for (int c0 = 0; c0 < D / 32; c0 += 2) {
          const int c = c0 + wg;
          float a[32];
          if (n_tiles > 0) {
            tmem_ld_32x32f(taddr + lane_base + c * 32, a);
            tmem_ld_wait();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) a[i] = 0.f;
          }
          float out_mul = mul;
          if (rotate && own_pos < p.N) {
            // gradient of the rotary embedding: rotate each (even, odd) pair back by
            // its angle, starting from the value rounded to the storage type
            const long tab = static_cast<long>(own_pos) * (D / 2) + c * 16;
            const float4* cs = reinterpret_cast<const float4*>(p.rope_cos + tab);
            const float4* sn = reinterpret_cast<const float4*>(p.rope_sin + tab);
#pragma unroll
            for (int q4 = 0; q4 < 4; ++q4) {
              const float4 c4 = cs[q4], s4 = sn[q4];
              const float cc[4] = {c4.x, c4.y, c4.z, c4.w};
              const float ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const int i = 8 * q4 + 2 * e;
                const float ge = round_elem<FP16>(a[i] * mul);
                const float go = round_elem<FP16>(a[i + 1] * mul);
                a[i] = ge * cc[e] + go * ss[e];
                a[i + 1] = go * cc[e] - ge * ss[e];
              }
            }
            out_mul = 1.0f;
          }
          if (own_pos < p.N &&
              SFL_BOUNDS_OK(own_pos >= 0 && b < p.B && h < p.H && c * 32 + 32 <= D, p.status)) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 v;
              v.x = pack2<FP16>(a[8 * i + 0] * out_mul, a[8 * i + 1] * out_mul);
              v.y = pack2<FP16>(a[8 * i + 2] * out_mul, a[8 * i + 3] * out_mul);
              v.z = pack2<FP16>(a[8 * i + 4] * out_mul, a[8 * i + 5] * out_mul);
              v.w = pack2<FP16>(a[8 * i + 6] * out_mul, a[8 * i + 7] * out_mul);
              *reinterpret_cast<uint4*>(dst + (c * 32 + i * 8) * 2) = v;
            }
          }
        }
      };
      const bool rotate = p.rope_cos != nullptr;
      if constexpr (KV_OWNED) {
        write_acc(tAcc0, p.dv, 1.0f, false);
        write_acc(tAcc1, p.dk, p.scale, rotate);
      } else {
        write_acc(tAcc0, p.dq, p.scale, rotate);
      }
    }
    SFL_TRACE_MARK(kTr + 6)
  }
  tc_fence_before();
  __syncthreads();
  SFL_TRACE_TOTAL(blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0, kTr)
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem, 512);
  }
}

// Rotate (even, odd) pairs by -angle in place: the gradient of the rotary
// embedding applied in the q|k|v projection epilogue.  x is [rows, ld] with the
// first `cols` columns rotated; position = row % T.
__global__ void rope_bwd_kernel(__nv_bfloat16* __restrict__ x, long ld, const float* __restrict__ cos,
                                const float* __restrict__ sin, long rows, int cols, int T,
                                int head_dim) {
  const long pairs = rows * (cols >> 1);
  const int half = head_dim >> 1;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < pairs;
       i += static_cast<long>(gridDim.x) * blockDim.x) {
    const long r = i / (cols >> 1);
    const int c = static_cast<int>(i % (cols >> 1)) * 2;
    const int pos = static_cast<int>(r % T);
    const int pi = (c % head_dim) >> 1;
    const float cs = cos[static_cast<long>(pos) * half + pi];
    const float sn = sin[static_cast<long>(pos) * half + pi];
    __nv_bfloat162* ptr = reinterpret_cast<__nv_bfloat162*>(x + r * ld + c);
    const float2 g = __bfloat1622float2(*ptr);
    *ptr = __floats2bfloat162_rn(g.x * cs + g.y * sn, -g.x * sn + g.y * cs);
  }
}

// ------------------------------------------------------------------ host ----
namespace {

int make_map(CUtensorMap* map, const void* base, const SflAttnTensor& t, int B, int H, int N, int D) {
  uint64_t dims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(N),
                      static_cast<uint64_t>(H), static_cast<uint64_t>(B)};
  uint64_t strides[4] = {0, static_cast<uint64_t>(t.stride_t) * 2,
                         static_cast<uint64_t>(t.stride_h) * 2,
                         static_cast<uint64_t>(t.stride_b) * 2};
  uint32_t box[4] = {64, kTile, 1, 1};
  return make_tensormap_nd_b16(map, base, 4, dims, strides, box, 3);
}

int attn_sm_count() {
  static int count = 0;
  if (count == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
    if (count <= 0) count = 148;
  }
  return count;
}

bool strides_ok(const SflAttnTensor& t) {
  return t.ptr != nullptr && (reinterpret_cast<uintptr_t>(t.ptr) & 15) == 0 &&
         t.stride_t % 8 == 0 && t.stride_h % 8 == 0 && t.stride_b % 8 == 0;
}

AttnSchedule to_sched(const SflAttnMask* m, bool transposed) {
  AttnSchedule s{};
  s.mode = m->mode;
  s.row_ptr = transposed ? m->t_row_ptr : m->row_ptr;
  s.col_idx = transposed ? m->t_col_idx : m->col_idx;
  s.full = transposed ? m->t_full : m->full;
  s.bitmap = reinterpret_cast<const unsigned long long*>(transposed ? m->t_bitmap : m->bitmap);
  s.causal = m->causal;
  s.window_left = m->window_left;
  s.window_right = m->window_right;
  s.doc = m->doc;
  return s;
}

template <typename Kernel>
int set_smem(Kernel kernel, int bytes) {
  return static_cast<int>(
      cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
}

}  // namespace
}  // namespace sfl

using namespace sfl;

extern "C" int sfl_attn_fwd(const SflAttnTensor* q, const SflAttnTensor* k, const SflAttnTensor* v,
                            const SflAttnTensor* o, float* lse, int B, int H, int N, int D,
                            float scale, const SflAttnMask* mask, int is_fp16, int* status,
                            void* stream_) {
  return sfl_attn_fwd_pipeline(q, k, v, o, lse, B, H, N, D, scale, mask, is_fp16, 0, status,
                               stream_);
}

// pipeline: 0 = default (for head dimension 64 two work streams per CTA with P in tensor
// memory, unless the pairs would not fill the GPU and rows are long; one stream for 128;
// SFL_ATTN_FWD=1|2|3 overrides the default for A/B runs), 1 = one
// stream per CTA, 2 = two streams, P in tensor memory, 3 = two streams, P in shared memory.
// Head dimension 128 always runs the one-stream kernel.
extern "C" int sfl_attn_fwd_pipeline(const SflAttnTensor* q, const SflAttnTensor* k,
                                     const SflAttnTensor* v, const SflAttnTensor* o, float* lse,
                                     int B, int H, int N, int D, float scale,
                                     const SflAttnMask* mask, int is_fp16, int pipeline,
                                     int* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (pipeline < 0 || pipeline > 3) return -2;
  if ((D != 64 && D != 128) || B <= 0 || H <= 0 || N <= 0 || mask == nullptr) return -2;
  if (!strides_ok(*q) || !strides_ok(*k) || !strides_ok(*v) || !strides_ok(*o)) return -2;
  CUtensorMap tq, tk, tv;
  if (make_map(&tq, q->ptr, *q, B, H, N, D) || make_map(&tk, k->ptr, *k, B, H, N, D) ||
      make_map(&tv, v->ptr, *v, B, H, N, D))
    return -3;
  AttnParams p{};
  p.B = B; p.H = H; p.N = N; p.scale = scale;
  p.sched = to_sched(mask, false);
  p.o = o->ptr; p.o_sb = o->stride_b; p.o_sh = o->stride_h; p.o_st = o->stride_t;
  p.lse = lse; p.is_fp16 = is_fp16; p.status = status;
  const int items = ((N + kTile - 1) / kTile) * B * H;
  static const int env_variant = [] {
    const char* v = getenv("SFL_ATTN_FWD");
    const int chosen = v == nullptr ? 0 : atoi(v);
    return chosen >= 1 && chosen <= 3 ? chosen : 0;
  }();
  int variant = pipeline != 0 ? pipeline : env_variant;
  if (variant == 0) {
    // Two streams per CTA halve the number of work items.  When the pairs no longer fill
    // the GPU and the rows are long (an unbounded causal mask: the heaviest pair is twice
    // the average), one query tile per CTA balances better - 1.49x at B1 H8 N4096.
    variant = 2;
    const int q_tiles = (N + kTile - 1) / kTile;
    const bool long_rows = mask->mode == 1 && mask->window_left < 0 && q_tiles >= 16;
    if (long_rows && (items + 1) / 2 <= attn_sm_count()) variant = 1;
  }
  if (D == 64 && variant != 1) {
    const int slots = (items + 1) / 2;
    dim3 grid2(slots < attn_sm_count() ? slots : attn_sm_count());
    auto go = [&](auto kern, int bytes) -> int {
      int rc = set_smem(kern, bytes);
      if (rc) return rc;
      return launch_pdl(kern, grid2, dim3(kFwd2Threads), bytes, stream, tq, tk, tv, p);
    };
    int rc;
    if (variant == 3)
      rc = is_fp16 ? go(attn_fwd2_kernel<true, false>, Fwd2Smem<false>::kBytes)
                   : go(attn_fwd2_kernel<false, false>, Fwd2Smem<false>::kBytes);
    else
      rc = is_fp16 ? go(attn_fwd2_kernel<true, true>, Fwd2Smem<true>::kBytes)
                   : go(attn_fwd2_kernel<false, true>, Fwd2Smem<true>::kBytes);
    if (rc) return rc;
    return static_cast<int>(cudaGetLastError());
  }
  dim3 grid(items < attn_sm_count() ? items : attn_sm_count());
#define SFL_FWD(D_, F_)                                                                   \
  {                                                                                       \
    auto kern = attn_fwd_kernel<D_, F_>;                                                  \
    int rc = set_smem(kern, FwdSmem<D_>::kBytes);                                         \
    if (rc) return rc;                                                                    \
    rc = launch_pdl(kern, grid, dim3(kAttnThreads), FwdSmem<D_>::kBytes, stream, tq, tk, tv, p); \
    if (rc) return rc;                                                                    \
  }
  if (D == 64) { if (is_fp16) SFL_FWD(64, true) else SFL_FWD(64, false) }
  else { if (is_fp16) SFL_FWD(128, true) else SFL_FWD(128, false) }
#undef SFL_FWD
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sfl_attn_bwd(const SflAttnTensor* q, const SflAttnTensor* k, const SflAttnTensor* v,
                            const SflAttnTensor* o, const SflAttnTensor* d_o, const float* lse,
                            float* delta, const SflAttnTensor* dq, const SflAttnTensor* dk,
                            const SflAttnTensor* dv, int B, int H, int N, int D, float scale,
                            const SflAttnMask* mask, int is_fp16, int* status,
                            const float* rope_cos, const float* rope_sin, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if ((D != 64 && D != 128) || B <= 0 || H <= 0 || N <= 0 || mask == nullptr) return -2;
  for (const SflAttnTensor* t : {q, k, v, o, d_o, dq, dk, dv})
    if (!strides_ok(*t)) return -2;
  // dO must share O's strides; dq/dk/dv share one stride triple.
  if (o->stride_b != d_o->stride_b || o->stride_h != d_o->stride_h || o->stride_t != d_o->stride_t)
    return -2;
  if (dq->stride_b != dk->stride_b || dq->stride_b != dv->stride_b || dq->stride_h != dk->stride_h ||
      dq->stride_h != dv->stride_h || dq->stride_t != dk->stride_t || dq->stride_t != dv->stride_t)
    return -2;
  if (mask->mode == 0 && (mask->t_row_ptr == nullptr || mask->t_col_idx == nullptr)) return -2;
  if ((rope_cos == nullptr) != (rope_sin == nullptr)) return -2;
  if (rope_cos != nullptr && ((reinterpret_cast<uintptr_t>(rope_cos) & 15) ||
                              (reinterpret_cast<uintptr_t>(rope_sin) & 15)))
    return -2;
  CUtensorMap tq, tk, tv, tdo;
  {
    // -3000 - 100 * operand - driver code tells which map was refused and why
    const SflAttnTensor* operands[4] = {q, k, v, d_o};
    CUtensorMap* maps[4] = {&tq, &tk, &tv, &tdo};
    for (int i = 0; i < 4; ++i) {
      const int rc = make_map(maps[i], operands[i]->ptr, *operands[i], B, H, N, D);
      if (rc) return -3000 - 100 * i - (rc > 0 && rc < 100 ? rc : 99);
    }
  }
  AttnParams p{};
  p.B = B; p.H = H; p.N = N; p.scale = scale;
  p.lse = const_cast<float*>(lse); p.delta = delta;
  p.o = o->ptr; p.d_o = d_o->ptr;
  p.o_sb = o->stride_b; p.o_sh = o->stride_h; p.o_st = o->stride_t;
  p.rope_cos = rope_cos; p.rope_sin = rope_sin;
  p.dq = dq->ptr; p.dk = dk->ptr; p.dv = dv->ptr;
  p.g_sb = dq->stride_b; p.g_sh = dq->stride_h; p.g_st = dq->stride_t;
  p.is_fp16 = is_fp16; p.status = status;
  dim3 grid((N + kTile - 1) / kTile, B * H);
#define SFL_BWD(D_, F_)                                                                       \
  {                                                                                           \
    auto kq = attn_bwd_kernel<D_, F_, false>;                                                 \
    auto kkv = attn_bwd_kernel<D_, F_, true>;                                                 \
    int rc = set_smem(kq, BwdSmem<D_>::kBytes);                                               \
    if (rc) return rc;                                                                        \
    rc = set_smem(kkv, BwdSmem<D_>::kBytes);                                                  \
    if (rc) return rc;                                                                        \
    p.sched = to_sched(mask, false);                                                          \
    rc = launch_pdl(kq, grid, dim3(kBwdThreads), BwdSmem<D_>::kBytes, stream, tq, tdo, tk, tv, p); \
    if (rc) return rc;                                                                        \
    p.sched = to_sched(mask, true);                                                           \
    rc = launch_pdl(kkv, grid, dim3(kBwdThreads), BwdSmem<D_>::kBytes, stream, tk, tv, tq, tdo, p); \
    if (rc) return rc;                                                                        \
  }
  if (D == 64) { if (is_fp16) SFL_BWD(64, true) else SFL_BWD(64, false) }
  else { if (is_fp16) SFL_BWD(128, true) else SFL_BWD(128, false) }
#undef SFL_BWD
  return static_cast<int>(cudaGetLastError());
}

// Copies and clears the phase timers of the two-stream forward kernel; returns -1 when the
// library was built without -DSFL_ATTN_TRACE.
extern "C" int sfl_attn_trace_read(unsigned long long* out16) {
#ifdef SFL_ATTN_TRACE
  unsigned long long zero[16] = {};
  cudaError_t e = cudaMemcpyFromSymbol(out16, g_attn_trace, sizeof(zero));
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaMemcpyToSymbol(g_attn_trace, zero, sizeof(zero)));
#else
  (void)out16;
  return -1;
#endif
}

// The same for the two backward kernels: 16 entries of the dQ kernel, then 16 of dK/dV.
extern "C" int sfl_attn_bwd_trace_read(unsigned long long* out32) {
#ifdef SFL_ATTN_TRACE
  unsigned long long zero[32] = {};
  const size_t at = 16 * sizeof(unsigned long long);
  cudaError_t e = cudaMemcpyFromSymbol(out32, g_attn_trace, sizeof(zero), at);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaMemcpyToSymbol(g_attn_trace, zero, sizeof(zero), at));
#else
  (void)out32;
  return -1;
#endif
}

// The raw time stamps (nanoseconds) of the last traced launch; -1 without -DSFL_ATTN_TRACE.
extern "C" int sfl_attn_stamps_read(unsigned long long* out64) {
#ifdef SFL_ATTN_TRACE
  return static_cast<int>(cudaMemcpyFromSymbol(out64, g_attn_stamps, 64 * sizeof(unsigned long long)));
#else
  (void)out64;
  return -1;
#endif
}

// Tensor-core split-KV decode (decode_mma2_kernel).  Same contract as sfl_decode: q
// [B, Hq, D], k / v [B, Hkv, N, D] contiguous, lengths [B], scratch for splits > 1, counters
// zero between launches; Hq / Hkv in {1, 2, 4, 8}; D in {64, 128}.
extern "C" int sfl_decode_mma(const void* q, const void* k, const void* v, const int* lengths,
                              float* part_m, float* part_l, float* part_u, int* counters,
                              void* out, int B, int Hq, int Hkv, int N, int D, int splits,
                              float scale, int is_fp16, int* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (q == nullptr || k == nullptr || v == nullptr || lengths == nullptr || out == nullptr)
    return -2;
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || N <= 0 || Hq % Hkv || splits < 1 || splits > 128 ||
      (D != 64 && D != 128))
    return -2;
  const int G = Hq / Hkv;
  if (G != 1 && G != 2 && G != 4 && G != 8) return -2;
  if (splits > 1 && (part_m == nullptr || part_l == nullptr || part_u == nullptr ||
                     counters == nullptr))
    return -2;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) |
       reinterpret_cast<uintptr_t>(part_u)) & 15)
    return -2;
  SflAttnTensor kt{const_cast<void*>(k), static_cast<long>(Hkv) * N * D, static_cast<long>(N) * D, D};
  SflAttnTensor vt{const_cast<void*>(v), static_cast<long>(Hkv) * N * D, static_cast<long>(N) * D, D};
  if (!strides_ok(kt) || !strides_ok(vt)) return -2;
  CUtensorMap tk, tv;
  if (make_map(&tk, k, kt, B, Hkv, N, D) || make_map(&tv, v, vt, B, Hkv, N, D)) return -3;
  DecParams p{};
  p.q = q; p.lengths = lengths; p.part_m = part_m; p.part_l = part_l; p.part_u = part_u;
  p.counters = counters; p.out = out;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.N = N; p.splits = splits; p.G = G;
  p.scale = scale; p.status = status;
  dim3 grid(B, Hkv, splits);
#define SFL_DEC(D_, F_)                                                                \
  {                                                                                    \
    auto kern = decode_mma2_kernel<D_, F_>;                                            \
    int rc = set_smem(kern, Dec2Smem<D_>::kBytes);                                     \
    if (rc) return rc;                                                                 \
    kern<<<grid, kDec2Threads, Dec2Smem<D_>::kBytes, stream>>>(tk, tv, p);             \
  }
  if (D == 64) { if (is_fp16) SFL_DEC(64, true) else SFL_DEC(64, false) }
  else { if (is_fp16) SFL_DEC(128, true) else SFL_DEC(128, false) }
#undef SFL_DEC
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sfl_rope_bwd(void* x_bf16, long ld, const float* cos, const float* sin, long rows,
                            int cols, int T, int head_dim, void* stream_) {
  if (rows <= 0 || cols <= 0) return 0;
  const long pairs = rows * (cols / 2);
  long blocks = (pairs + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  rope_bwd_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream_)>>>(
      static_cast<__nv_bfloat16*>(x_bf16), ld, cos, sin, rows, cols, T, head_dim);
  return static_cast<int>(cudaGetLastError());
}
