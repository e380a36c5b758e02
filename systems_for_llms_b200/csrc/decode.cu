// Single-token attention over a contiguous KV cache (split-KV, grouped queries).
//
// Decode is bound by reading the cache once from HBM, so the kernel is built
// around wide loads and many of them in flight rather than tensor cores: a CTA
// owns (batch, kv head, split); its 8 warps walk the split's tokens, 16 bytes of
// a K or V row per lane (D/8 lanes per token, so a warp covers 2 or 4 tokens per
// instruction) with several rows in flight per lane; all query heads of the GQA
// group are evaluated against every loaded row, so K and V are read exactly once
// per group.  Softmax state (m, l, accumulator) is kept per lane group and
// merged across lanes, warps and finally splits with the exact log-sum-exp
// algebra; the cross-split merge runs in the last CTA to finish for its
// (batch, kv head) - found with an arrival counter - so no second launch and no
// host round trip is needed.
//
// Semantics follow the reference kernel (attention_lab/cuda_decode/decode.cu:
// 27-184): lengths clamp to the cache capacity, splits partition the capacity
// (chunk = ceil(N / splits)) so empty partitions contribute (m=-inf, l=0),
// scores are scaled after the dot product, zero-length rows return zeros,
// "token" rescales the running state after every token and "tile" once per
// group of tokens.
#include <atomic>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>

#include <type_traits>

#include "sfl.h"

namespace sfl {

constexpr int kDecodeWarps = 8;
constexpr float kDecLog2e = 1.4426950408889634f;

template <typename T>
__device__ __forceinline__ void unpack8(const uint4& raw, float (&out)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (sizeof(T) == 2 && std::is_same<T, __half>::value) {
      const __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      const float2 f = __half22float2(h);
      out[2 * i] = f.x;
      out[2 * i + 1] = f.y;
    } else {
      const __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
      const float2 f = __bfloat1622float2(h);
      out[2 * i] = f.x;
      out[2 * i + 1] = f.y;
    }
  }
}

__device__ __forceinline__ float dec_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

struct DecodeParams {
  const void* q;  // [B, Hq, D]
  const void* k;  // [B, Hkv, N, D]
  const void* v;
  const int* lengths;  // [B]
  float* part_m;       // [B, Hq, S]  (log2 domain)
  float* part_l;       // [B, Hq, S]
  float* part_u;       // [B, Hq, S, D]
  int* counters;       // [B, Hkv], zero between launches
  void* out;           // [B, Hq, D]
  int B, Hq, Hkv, N, splits;
  float scale;
};

// Merge (m, l, acc) pairs: a <- a (+) b.
template <int D8>
__device__ __forceinline__ void merge_state(float& m, float& l, float (&acc)[D8], float m2, float l2,
                                            const float (&acc2)[D8]) {
  const float mn = fmaxf(m, m2);
  const float a = m == -INFINITY ? 0.f : dec_exp2(m - mn);
  const float b = m2 == -INFINITY ? 0.f : dec_exp2(m2 - mn);
  l = l * a + l2 * b;
#pragma unroll
  for (int i = 0; i < D8; ++i) acc[i] = acc[i] * a + acc2[i] * b;
  m = mn;
}

// UNROLL tokens per lane group are scored before the running state is rescaled
// (1 = "token" variant, 4 = "tile" variant).
template <typename T, int D, int G, int UNROLL>
__global__ void __launch_bounds__(kDecodeWarps * 32)
decode_kernel(const DecodeParams p) {
  constexpr int LPT = D / 8;    // lanes per token (16 bytes each)
  constexpr int TPW = 32 / LPT; // tokens per warp per load instruction
  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane / LPT;   // which token of the warp's TPW this lane serves
  const int dl = lane % LPT;    // which 8-element slice of the head dimension
  int len = p.lengths[b];
  len = len < 0 ? 0 : (len > p.N ? p.N : len);
  const int chunk = (p.N + p.splits - 1) / p.splits;
  const int begin = split * chunk;
  const int end = min(len, begin + chunk);

  // Query slices for the group's heads, pre-multiplied by scale * log2(e).
  float q[G][8];
  const float qs = p.scale * kDecLog2e;
#pragma unroll
  for (int g = 0; g < G; ++g) {
    const T* qp = static_cast<const T*>(p.q) + (static_cast<long>(b) * p.Hq + kvh * G + g) * D + dl * 8;
    const uint4 raw = *reinterpret_cast<const uint4*>(qp);
    unpack8<T>(raw, q[g]);
#pragma unroll
    for (int i = 0; i < 8; ++i) q[g][i] *= qs;
  }
  float m[G], l[G], acc[G][8];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[g][i] = 0.f;
  }
  const long kv_base = (static_cast<long>(b) * p.Hkv + kvh) * p.N;
  const T* kbase = static_cast<const T*>(p.k) + kv_base * D + dl * 8;
  const T* vbase = static_cast<const T*>(p.v) + kv_base * D + dl * 8;
  constexpr int STEP = kDecodeWarps * TPW;  // tokens covered by the CTA per instruction

  for (int t0 = begin + warp * TPW + sub; t0 < end + STEP * UNROLL; t0 += STEP * UNROLL) {
    if (t0 - (warp * TPW + sub) >= end) break;  // warp-uniform: nothing left for anyone
    uint4 kr[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int t = t0 + u * STEP;
      kr[u] = t < end ? *reinterpret_cast<const uint4*>(kbase + static_cast<long>(t) * D)
                      : make_uint4(0, 0, 0, 0);
    }
    uint4 vr[UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int t = t0 + u * STEP;
      vr[u] = t < end ? *reinterpret_cast<const uint4*>(vbase + static_cast<long>(t) * D)
                      : make_uint4(0, 0, 0, 0);
    }
    float s[G][UNROLL];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      float kf[8];
      unpack8<T>(kr[u], kf);
      const bool valid = t0 + u * STEP < end;
#pragma unroll
      for (int g = 0; g < G; ++g) {
        float d = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) d = fmaf(q[g][i], kf[i], d);
#pragma unroll
        for (int o = LPT / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
        s[g][u] = valid ? d : -INFINITY;
      }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float mx = s[g][0];
#pragma unroll
      for (int u = 1; u < UNROLL; ++u) mx = fmaxf(mx, s[g][u]);
      const float mn = fmaxf(m[g], mx);
      if (mn > m[g]) {
        const float a = m[g] == -INFINITY ? 0.f : dec_exp2(m[g] - mn);
        l[g] *= a;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] *= a;
        m[g] = mn;
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      float vf[8];
      unpack8<T>(vr[u], vf);
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pr = m[g] == -INFINITY ? 0.f : dec_exp2(s[g][u] - m[g]);
        l[g] += pr;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[g][i] = fmaf(pr, vf[i], acc[g][i]);
      }
    }
  }

  // ---- merge the TPW lane groups of the warp --------------------------------
#pragma unroll
  for (int g = 0; g < G; ++g) {
#pragma unroll
    for (int o = LPT; o < 32; o <<= 1) {
      const float m2 = __shfl_xor_sync(0xffffffffu, m[g], o);
      const float l2 = __shfl_xor_sync(0xffffffffu, l[g], o);
      float a2[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) a2[i] = __shfl_xor_sync(0xffffffffu, acc[g][i], o);
      merge_state<8>(m[g], l[g], acc[g], m2, l2, a2);
    }
  }
  // ---- merge the warps through shared memory ----------------------------------
  __shared__ float sm_m[kDecodeWarps][G];
  __shared__ float sm_l[kDecodeWarps][G];
  __shared__ float sm_u[kDecodeWarps][G][D];
  if (sub == 0) {
#pragma unroll
    for (int g = 0; g < G; ++g) {
      if (dl == 0) {
        sm_m[warp][g] = m[g];
        sm_l[warp][g] = l[g];
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) sm_u[warp][g][dl * 8 + i] = acc[g][i];
    }
  }
  __syncthreads();
  const long head0 = static_cast<long>(b) * p.Hq + kvh * G;
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) mm = fmaxf(mm, sm_m[w][g]);
    float ll = 0.f, uu = 0.f;
#pragma unroll
    for (int w = 0; w < kDecodeWarps; ++w) {
      const float a = sm_m[w][g] == -INFINITY ? 0.f : dec_exp2(sm_m[w][g] - mm);
      ll += sm_l[w][g] * a;
      uu += sm_u[w][g][d] * a;
    }
    if (p.splits == 1) {
      static_cast<T*>(p.out)[(head0 + g) * D + d] = from_float<T>(ll > 0.f ? uu / ll : 0.f);
    } else {
      const long slot = (head0 + g) * p.splits + split;
      p.part_u[slot * D + d] = uu;
      if (d == 0) {
        p.part_m[slot] = mm;
        p.part_l[slot] = ll;
      }
    }
  }
  if (p.splits == 1) return;

  // ---- the last CTA of this (batch, kv head) merges the splits ------------------
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(&p.counters[b * p.Hkv + kvh], 1);
    is_last = ticket == p.splits - 1;
    if (is_last) p.counters[b * p.Hkv + kvh] = 0;  // ready for the next launch
  }
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int g = idx / D, d = idx % D;
    const long base = (head0 + g) * p.splits;
    float mm = -INFINITY;
    for (int s = 0; s < p.splits; ++s) mm = fmaxf(mm, __ldcg(p.part_m + base + s));
    float ll = 0.f, uu = 0.f;
    for (int s = 0; s < p.splits; ++s) {
      const float ms = __ldcg(p.part_m + base + s);
      const float a = (ms == -INFINITY || mm == -INFINITY) ? 0.f : dec_exp2(ms - mm);
      ll += __ldcg(p.part_l + base + s) * a;
      uu += __ldcg(p.part_u + (base + s) * D + d) * a;
    }
    static_cast<T*>(p.out)[(head0 + g) * D + d] = from_float<T>(ll > 0.f ? uu / ll : 0.f);
  }
}

template <typename T, int D, int G>
int launch_decode(const DecodeParams& p, bool tile, cudaStream_t stream) {
  dim3 grid(p.B, p.Hkv, p.splits);
  if (tile)
    decode_kernel<T, D, G, 4><<<grid, kDecodeWarps * 32, 0, stream>>>(p);
  else
    decode_kernel<T, D, G, 1><<<grid, kDecodeWarps * 32, 0, stream>>>(p);
  return static_cast<int>(cudaGetLastError());
}

template <typename T, int D>
int dispatch_group(const DecodeParams& p, int groups, bool tile, cudaStream_t stream) {
  switch (groups) {
    case 1: return launch_decode<T, D, 1>(p, tile, stream);
    case 2: return launch_decode<T, D, 2>(p, tile, stream);
    case 4: return launch_decode<T, D, 4>(p, tile, stream);
    case 8: return launch_decode<T, D, 8>(p, tile, stream);
    default: return -2;
  }
}

}  // namespace sfl

using namespace sfl;

extern "C" int sfl_decode(const void* q, const void* k, const void* v, const int* lengths,
                          float* part_m, float* part_l, float* part_u, int* counters, void* out,
                          int B, int Hq, int Hkv, int N, int D, int splits, float scale,
                          int tile_variant, int is_fp16, void* stream_) {
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || N <= 0 || Hq % Hkv) return -2;
  if (splits < 1 || splits > 128 || (D != 64 && D != 128)) return -2;
  if (splits > 1 && (part_m == nullptr || part_l == nullptr || part_u == nullptr ||
                     counters == nullptr))
    return -2;
  DecodeParams p{q, k, v, lengths, part_m, part_l, part_u, counters, out,
                 B, Hq, Hkv, N, splits, scale};
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int groups = Hq / Hkv;
  const bool tile = tile_variant != 0;
  if (is_fp16) {
    return D == 64 ? dispatch_group<__half, 64>(p, groups, tile, stream)
                   : dispatch_group<__half, 128>(p, groups, tile, stream);
  }
  return D == 64 ? dispatch_group<__nv_bfloat16, 64>(p, groups, tile, stream)
                 : dispatch_group<__nv_bfloat16, 128>(p, groups, tile, stream);
}

// ------------------------------------------------------------------------------
// Allocation-free variant of sfl_decode (declared in sfl.h as sfl_decode_static).
//
// Some callers cannot reach a device allocator at the moment they need to decode:
// code running inside a CUDA-graph capture or between the nodes of a latency
// critical serving loop (cudaMalloc synchronises the device and is illegal during
// capture), plug-ins loaded into a host process whose memory pool they may not
// touch, and C callers that link this library without PyTorch and therefore have
// no caching allocator to lean on.  For them the split-KV scratch (per-split
// maxima, normalisers, partial outputs and the arrival counters) lives in one
// fixed array inside the library image.  Every GPU that loads the library holds
// those bytes until the process exits, which is why the capacity is modest.
namespace sfl {

constexpr long kStaticSlots = 8192;     // max batch * query_heads * splits
constexpr long kStaticCounters = 1024;  // max batch * kv_heads
constexpr long kStaticFloats = kStaticSlots * 2 + kStaticSlots * 128;
constexpr long kStaticBytes = kStaticFloats * 4 + kStaticCounters * 4;

// Layout: part_m[kStaticSlots] | part_l[kStaticSlots] | part_u[kStaticSlots * 128] | counters.
static __device__ __align__(256) unsigned char g_decode_scratch[kStaticBytes];

// In host code `g_decode_scratch` is only a handle for the runtime, not an
// address a kernel may dereference; the real device address is looked up once
// per device and remembered here.
constexpr int kMaxDevices = 64;
// (atomic: two host threads may make their first call on a device at the same time; both
// resolve the same address)
static std::atomic<void*> g_scratch_address[kMaxDevices] = {};
static thread_local char g_static_error[256] = "";

int fail_static(int code, const char* message) {
  snprintf(g_static_error, sizeof(g_static_error), "%s", message);
  return code;
}

}  // namespace sfl

extern "C" const char* sfl_decode_static_error(void) { return sfl::g_static_error; }

extern "C" long sfl_decode_static_capacity_slots(void) { return sfl::kStaticSlots; }

extern "C" int sfl_decode_static(const void* q, const void* k, const void* v, const int* lengths,
                                 void* out, int B, int Hq, int Hkv, int N, int D, int splits,
                                 float scale, int tile_variant, int is_fp16, void* stream_) {
  using namespace sfl;
  // Everything is checked before anything is queued on the stream: plain C callers are
  // the audience of this entry point, and a null pointer would reach the kernel.
  if (q == nullptr || k == nullptr || v == nullptr || lengths == nullptr || out == nullptr)
    return fail_static(-2, "sfl_decode_static: q, k, v, lengths and out must not be null");
  if (B <= 0 || Hq <= 0 || Hkv <= 0 || N <= 0 || Hq % Hkv || splits < 1 || splits > 128 ||
      (D != 64 && D != 128))
    return fail_static(-2, "sfl_decode_static: unsupported shape (see sfl_decode)");
  {
    const int ratio = Hq / Hkv;
    if (ratio != 1 && ratio != 2 && ratio != 4 && ratio != 8)
      return fail_static(-2, "sfl_decode_static: query heads per KV head must be 1, 2, 4 or 8");
  }
  if (!(scale > 0.0f) || !isfinite(scale))
    return fail_static(-2, "sfl_decode_static: scale must be finite and positive");
  const long slots = static_cast<long>(B) * Hq * splits;
  if (slots > kStaticSlots || static_cast<long>(B) * Hkv > kStaticCounters) {
    char text[200];
    snprintf(text, sizeof(text),
             "sfl_decode_static: batch*query_heads*splits = %ld exceeds the built-in scratch "
             "capacity of %ld (or batch*kv_heads > %ld); use sfl_decode with caller scratch",
             slots, kStaticSlots, kStaticCounters);
    return fail_static(-10, text);
  }
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess || device < 0 || device >= kMaxDevices)
    return fail_static(-11, "sfl_decode_static: cannot identify the current device");
  void* resolved = g_scratch_address[device].load(std::memory_order_acquire);
  if (resolved == nullptr) {
    // First call on this device: resolve the array's device address.  This is a
    // runtime query, not an allocation, but it may not be issued while a stream
    // is capturing, so make the first call before any capture.
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, g_decode_scratch);
    if (err != cudaSuccess || address == nullptr)
      return fail_static(-12, "sfl_decode_static: cudaGetSymbolAddress failed");
    g_scratch_address[device].store(address, std::memory_order_release);
    resolved = address;
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  float* base = static_cast<float*>(resolved);
  float* part_m = base;
  float* part_l = base + kStaticSlots;
  float* part_u = base + 2 * kStaticSlots;
  int* counters = reinterpret_cast<int*>(base + kStaticFloats);
  // The array keeps whatever the previous call left.  Partials are fully
  // rewritten before they are read; the arrival counters must start at zero, so
  // clear the ones this call uses (a stale count from an interrupted launch would
  // otherwise pick the wrong "last" CTA).
  err = cudaMemsetAsync(counters, 0, sizeof(int) * static_cast<size_t>(B) * Hkv, stream);
  if (err != cudaSuccess) return fail_static(-13, "sfl_decode_static: clearing counters failed");
  const int rc = sfl_decode(q, k, v, lengths, part_m, part_l, part_u, counters, out, B, Hq, Hkv,
                            N, D, splits, scale, tile_variant, is_fp16, stream_);
  if (rc != 0) return fail_static(rc, "sfl_decode_static: kernel launch failed");
  g_static_error[0] = '\0';
  return 0;
}
