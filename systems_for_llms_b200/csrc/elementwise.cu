// Bandwidth-bound kernels of the training step: RMSNorm forward/backward, fused
// cross-entropy (loss + logit gradient in one pass), gradient norm, fused AdamW
// over flat buffers, casts and the embedding gather.  Each replaces a chain of
// eager PyTorch kernels in the reference (src/llmlab/model/layers.py:133-141,
// src/llmlab/training/loss.py:4-22, src/llmlab/train.py:77-79) with one pass
// over HBM.  All math is fp32; reductions are tree-shaped and order-fixed so the
// results are bitwise reproducible from run to run.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "launch.cuh"
#include "ptx.cuh"
#include "sfl.h"

namespace sfl {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum; result valid in every thread.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x >> 5) ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x >> 5) ? scratch[lane] : -INFINITY;
    t = warp_max(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// ---------------------------------------------------------------- RMSNorm ---
// One warp per row.
__global__ void rmsnorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                   __nv_bfloat16* __restrict__ y, float* __restrict__ rstd,
                                   int rows, int dim, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  if (!SFL_BOUNDS_OK(row >= 0 && dim > 0, nullptr)) return;
  const float* xr = x + static_cast<long>(row) * dim;
  __nv_bfloat16* yr = y + static_cast<long>(row) * dim;
  float ss = 0.f;
  if ((dim & 3) == 0) {
    for (int i = lane * 4; i < dim; i += 128) {
      const float4 v = *reinterpret_cast<const float4*>(xr + i);
      ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
  } else {
    for (int i = lane; i < dim; i += 32) ss += xr[i] * xr[i];
  }
  ss = warp_sum(ss);
  // Same operation order as the reference: x / sqrt(mean + eps) * w.
  const float rms = sqrtf(ss / static_cast<float>(dim) + eps);
  const float inv = 1.0f / rms;
  if (lane == 0 && rstd != nullptr) rstd[row] = inv;
  if ((dim & 3) == 0) {
    for (int i = lane * 4; i < dim; i += 128) {
      const float4 v = *reinterpret_cast<const float4*>(xr + i);
      const float4 g = *reinterpret_cast<const float4*>(w + i);
      uint2 o;
      o.x = pack_bf16(v.x / rms * g.x, v.y / rms * g.y);
      o.y = pack_bf16(v.z / rms * g.z, v.w / rms * g.w);
      *reinterpret_cast<uint2*>(yr + i) = o;
    }
  } else {
    for (int i = lane; i < dim; i += 32) yr[i] = __float2bfloat16_rn(xr[i] / rms * w[i]);
  }
}

// The same with the row held in registers (dim = 128 NCH): every load of the row is in
// flight at once and x is read a single time.
template <int NCH>
__global__ void __launch_bounds__(128)
rmsnorm_fwd_vec_kernel(const float* __restrict__ x, const float* __restrict__ w,
                       __nv_bfloat16* __restrict__ y, float* __restrict__ rstd, int rows,
                       float eps) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int dim = NCH * 128;
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  if (!SFL_BOUNDS_OK(row >= 0, nullptr)) return;
  const float* xr = x + static_cast<long>(row) * dim;
  __nv_bfloat16* yr = y + static_cast<long>(row) * dim;
  float4 xv[NCH], g[NCH];
#pragma unroll
  for (int c = 0; c < NCH; ++c) xv[c] = *reinterpret_cast<const float4*>(xr + c * 128 + lane * 4);
#pragma unroll
  for (int c = 0; c < NCH; ++c) g[c] = *reinterpret_cast<const float4*>(w + c * 128 + lane * 4);
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < NCH; ++c)
    ss += xv[c].x * xv[c].x + xv[c].y * xv[c].y + xv[c].z * xv[c].z + xv[c].w * xv[c].w;
  ss = warp_sum(ss);
  // One division per row: the quotient x / rms of the portable path differs from x * (1 / rms)
  // by at most an ulp of fp32, far below the bf16 rounding of the result, and a division per
  // element kept the special-function unit busier than the memory system (36 % against 21 %).
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(dim) + eps);
  if (lane == 0 && rstd != nullptr) rstd[row] = inv;
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    uint2 o;
    o.x = pack_bf16(xv[c].x * inv * g[c].x, xv[c].y * inv * g[c].y);
    o.y = pack_bf16(xv[c].z * inv * g[c].z, xv[c].w * inv * g[c].w);
    *reinterpret_cast<uint2*>(yr + c * 128 + lane * 4) = o;
  }
}

constexpr int kNormBwdBlocks = 296;  // two CTAs per SM on a 148-SM part
constexpr int kNormBwdThreads = 256;

// Each block owns a strided set of rows, one warp per row at a time.  A lane
// always touches the same columns (4 consecutive elements every 128), so the
// weight-gradient partial lives in registers across rows; the row itself is
// read once and kept in registers between the dot-product and the update.
// NCH = dim / 128 (dim must be a multiple of 128 and at most 1024 here).
template <int NCH>
__global__ void __launch_bounds__(kNormBwdThreads)
rmsnorm_bwd_vec_kernel(const __nv_bfloat16* __restrict__ dy, const float* __restrict__ x,
                       const float* __restrict__ w, const float* __restrict__ rstd,
                       const float* __restrict__ dres_in, float* __restrict__ dx_out,
                       __nv_bfloat16* __restrict__ dx_bf16, float* __restrict__ dw_partial,
                       int rows) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int dim = NCH * 128;
  extern __shared__ float dw_smem[];  // [warps, dim]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = blockDim.x >> 5;
  float4 wv[NCH], dwv[NCH];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    wv[c] = *reinterpret_cast<const float4*>(w + c * 128 + lane * 4);
    dwv[c] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  for (int row = blockIdx.x * warps + warp; row < rows; row += gridDim.x * warps) {
    const long off = static_cast<long>(row) * dim;
    const float inv = rstd[row];
    float4 xh[NCH], g[NCH], res[NCH];
    float dot = 0.f;
    // every load of the row is issued before the first use, so one round trip to
    // memory covers x, dy and the incoming residual gradient
#pragma unroll
    for (int c = 0; c < NCH; ++c)
      res[c] = dres_in != nullptr
                   ? *reinterpret_cast<const float4*>(dres_in + off + c * 128 + lane * 4)
                   : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = c * 128 + lane * 4;
      const float4 xv = *reinterpret_cast<const float4*>(x + off + col);
      const uint2 dq = *reinterpret_cast<const uint2*>(dy + off + col);
      const float2 d01 = unpack_bf16(dq.x), d23 = unpack_bf16(dq.y);
      xh[c] = make_float4(xv.x * inv, xv.y * inv, xv.z * inv, xv.w * inv);
      g[c] = make_float4(d01.x, d01.y, d23.x, d23.y);
      dot += g[c].x * wv[c].x * xh[c].x + g[c].y * wv[c].y * xh[c].y +
             g[c].z * wv[c].z * xh[c].z + g[c].w * wv[c].w * xh[c].w;
    }
    dot = warp_sum(dot) / static_cast<float>(dim);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int col = c * 128 + lane * 4;
      float4 d;
      d.x = inv * (g[c].x * wv[c].x - xh[c].x * dot);
      d.y = inv * (g[c].y * wv[c].y - xh[c].y * dot);
      d.z = inv * (g[c].z * wv[c].z - xh[c].z * dot);
      d.w = inv * (g[c].w * wv[c].w - xh[c].w * dot);
      d.x += res[c].x; d.y += res[c].y; d.z += res[c].z; d.w += res[c].w;
      *reinterpret_cast<float4*>(dx_out + off + col) = d;
      if (dx_bf16 != nullptr) {
        uint2 o;
        o.x = pack_bf16(d.x, d.y);
        o.y = pack_bf16(d.z, d.w);
        *reinterpret_cast<uint2*>(dx_bf16 + off + col) = o;
      }
      dwv[c].x += g[c].x * xh[c].x;
      dwv[c].y += g[c].y * xh[c].y;
      dwv[c].z += g[c].z * xh[c].z;
      dwv[c].w += g[c].w * xh[c].w;
    }
  }
#pragma unroll
  for (int c = 0; c < NCH; ++c)
    *reinterpret_cast<float4*>(dw_smem + static_cast<long>(warp) * dim + c * 128 + lane * 4) = dwv[c];
  __syncthreads();
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < warps; ++k) s += dw_smem[static_cast<long>(k) * dim + i];
    dw_partial[static_cast<long>(blockIdx.x) * dim + i] = s;
  }
}

// The same with a row shared by two warps (NCH even): each warp holds half as many
// registers, so two CTAs fit on an SM and twice as many rows are in flight; the two
// halves of the row's dot product meet in shared memory and are added in a fixed order.
template <int NCH>
__global__ void __launch_bounds__(kNormBwdThreads, 2)
rmsnorm_bwd_pair_kernel(const __nv_bfloat16* __restrict__ dy, const float* __restrict__ x,
                        const float* __restrict__ w, const float* __restrict__ rstd,
                        const float* __restrict__ dres_in, float* __restrict__ dx_out,
                        __nv_bfloat16* __restrict__ dx_bf16, float* __restrict__ dw_partial,
                        int rows) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int dim = NCH * 128;
  constexpr int HC = NCH / 2;
  constexpr int kPairs = kNormBwdThreads / 64;
  extern __shared__ float dw_smem[];  // [pairs, dim]
  __shared__ float pair_dot[2][kPairs][2];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pair = warp >> 1, half = warp & 1;
  const int col0 = half * HC * 128 + lane * 4;
  float4 wv[HC], dwv[HC];
#pragma unroll
  for (int c = 0; c < HC; ++c) {
    wv[c] = *reinterpret_cast<const float4*>(w + col0 + c * 128);
    dwv[c] = make_float4(0.f, 0.f, 0.f, 0.f);
  }
  int parity = 0;
  for (int row = blockIdx.x * kPairs + pair; row < rows; row += gridDim.x * kPairs, parity ^= 1) {
    const long off = static_cast<long>(row) * dim + col0;
    const float inv = rstd[row];
    float4 xh[HC], g[HC], res[HC];
    float dot = 0.f;
#pragma unroll
    for (int c = 0; c < HC; ++c)
      res[c] = dres_in != nullptr ? *reinterpret_cast<const float4*>(dres_in + off + c * 128)
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int c = 0; c < HC; ++c) {
      const float4 xv = *reinterpret_cast<const float4*>(x + off + c * 128);
      const uint2 dq = *reinterpret_cast<const uint2*>(dy + off + c * 128);
      const float2 d01 = unpack_bf16(dq.x), d23 = unpack_bf16(dq.y);
      xh[c] = make_float4(xv.x * inv, xv.y * inv, xv.z * inv, xv.w * inv);
      g[c] = make_float4(d01.x, d01.y, d23.x, d23.y);
      dot += g[c].x * wv[c].x * xh[c].x + g[c].y * wv[c].y * xh[c].y +
             g[c].z * wv[c].z * xh[c].z + g[c].w * wv[c].w * xh[c].w;
    }
    dot = warp_sum(dot);
    if (lane == 0) pair_dot[parity][pair][half] = dot;
    // the two warps of the pair meet; buffers alternate, so a slot is rewritten only after
    // both warps have passed the barrier that follows their last read of it
    asm volatile("bar.sync %0, 64;" ::"r"(1 + pair) : "memory");
    dot = (pair_dot[parity][pair][0] + pair_dot[parity][pair][1]) / static_cast<float>(dim);
#pragma unroll
    for (int c = 0; c < HC; ++c) {
      float4 d;
      d.x = inv * (g[c].x * wv[c].x - xh[c].x * dot);
      d.y = inv * (g[c].y * wv[c].y - xh[c].y * dot);
      d.z = inv * (g[c].z * wv[c].z - xh[c].z * dot);
      d.w = inv * (g[c].w * wv[c].w - xh[c].w * dot);
      d.x += res[c].x; d.y += res[c].y; d.z += res[c].z; d.w += res[c].w;
      *reinterpret_cast<float4*>(dx_out + off + c * 128) = d;
      if (dx_bf16 != nullptr) {
        uint2 o;
        o.x = pack_bf16(d.x, d.y);
        o.y = pack_bf16(d.z, d.w);
        *reinterpret_cast<uint2*>(dx_bf16 + off + c * 128) = o;
      }
      dwv[c].x += g[c].x * xh[c].x;
      dwv[c].y += g[c].y * xh[c].y;
      dwv[c].z += g[c].z * xh[c].z;
      dwv[c].w += g[c].w * xh[c].w;
    }
  }
#pragma unroll
  for (int c = 0; c < HC; ++c)
    *reinterpret_cast<float4*>(dw_smem + static_cast<long>(pair) * dim + col0 + c * 128) = dwv[c];
  __syncthreads();
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kPairs; ++k) s += dw_smem[static_cast<long>(k) * dim + i];
    dw_partial[static_cast<long>(blockIdx.x) * dim + i] = s;
  }
}

// Generic fallback for any row width.
__global__ void __launch_bounds__(kNormBwdThreads)
rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ dy, const float* __restrict__ x,
                   const float* __restrict__ w, const float* __restrict__ rstd,
                   const float* __restrict__ dres_in, float* __restrict__ dx_out,
                   __nv_bfloat16* __restrict__ dx_bf16, float* __restrict__ dw_partial, int rows,
                   int dim) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float dw_smem[];  // [warps, dim]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int warps = blockDim.x >> 5;
  float* my_dw = dw_smem + static_cast<long>(warp) * dim;
  for (int i = lane; i < dim; i += 32) my_dw[i] = 0.f;
  __syncwarp();
  for (int row = blockIdx.x * warps + warp; row < rows; row += gridDim.x * warps) {
    const long off = static_cast<long>(row) * dim;
    const float inv = rstd[row];
    float dot = 0.f;
    for (int i = lane; i < dim; i += 32) {
      const float g = __bfloat162float(dy[off + i]) * w[i];
      dot += g * x[off + i] * inv;
    }
    dot = warp_sum(dot) / static_cast<float>(dim);
    for (int i = lane; i < dim; i += 32) {
      const float dyi = __bfloat162float(dy[off + i]);
      const float xhat = x[off + i] * inv;
      float dxi = inv * (dyi * w[i] - xhat * dot);
      if (dres_in != nullptr) dxi += dres_in[off + i];
      dx_out[off + i] = dxi;
      if (dx_bf16 != nullptr) dx_bf16[off + i] = __float2bfloat16_rn(dxi);
      my_dw[i] += dyi * xhat;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float s = 0.f;
    for (int k = 0; k < warps; ++k) s += dw_smem[static_cast<long>(k) * dim + i];
    dw_partial[static_cast<long>(blockIdx.x) * dim + i] = s;
  }
}

// Each CTA folds 32 columns over all partial rows: 32 warps take every 32nd row
// (independent loads in flight: about ten rows per warp for 296 partials, so the whole
// fold is three round trips to L2), then one warp adds the 32 sums in a fixed order,
// so the result does not depend on scheduling.
constexpr int kDwReduceWarps = 32;
// blockIdx.y selects one of up to two folds done by the same launch (the two norms of a
// transformer block).
__global__ void __launch_bounds__(32 * kDwReduceWarps)
rmsnorm_dw_reduce_kernel(const float* __restrict__ partial, int blocks, float* __restrict__ dw,
                         int dim, int accumulate, const float* __restrict__ partial_b,
                         float* __restrict__ dw_b, int accumulate_b) {
  pdl_launch_dependents();
  pdl_wait();
  if (blockIdx.y == 1) {
    partial = partial_b;
    dw = dw_b;
    accumulate = accumulate_b;
  }
  __shared__ float part[kDwReduceWarps][32];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int i = blockIdx.x * 32 + lane;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  if (i < dim) {
    int b = warp;
    for (; b + 3 * kDwReduceWarps < blocks; b += 4 * kDwReduceWarps) {
      s0 += partial[static_cast<long>(b) * dim + i];
      s1 += partial[static_cast<long>(b + kDwReduceWarps) * dim + i];
      s2 += partial[static_cast<long>(b + 2 * kDwReduceWarps) * dim + i];
      s3 += partial[static_cast<long>(b + 3 * kDwReduceWarps) * dim + i];
    }
    for (; b < blocks; b += kDwReduceWarps) s0 += partial[static_cast<long>(b) * dim + i];
  }
  part[warp][lane] = (s0 + s1) + (s2 + s3);
  __syncthreads();
  if (warp == 0 && i < dim) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kDwReduceWarps; ++k) s += part[k][lane];
    dw[i] = accumulate ? dw[i] + s : s;
  }
}

// ---------------------------------------------------------- cross entropy ---
// One CTA per row.  The row (vocab * 2 bytes) is read twice from L1/L2 and the
// gradient written once; logits never exist in fp32 in memory.
__global__ void __launch_bounds__(256)
cross_entropy_kernel(const __nv_bfloat16* __restrict__ logits, long ld,
                     const int64_t* __restrict__ targets, float* __restrict__ row_loss,
                     __nv_bfloat16* __restrict__ dlogits, float grad_scale, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int row = blockIdx.x;
  const __nv_bfloat16* lr = logits + static_cast<long>(row) * ld;
  // The gradient may overwrite the logits in place: fetch the target's logit before
  // any thread of the block can have stored anything.
  const int64_t tgt = targets[row];
  const bool tgt_ok = tgt >= 0 && tgt < vocab;
  const float target_logit = (threadIdx.x == 0 && tgt_ok) ? __bfloat162float(lr[tgt]) : 0.f;
  float mx = -INFINITY;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) mx = fmaxf(mx, __bfloat162float(lr[i]));
  mx = block_max(mx, scratch);
  float sum = 0.f;
  for (int i = threadIdx.x; i < vocab; i += blockDim.x) sum += expf(__bfloat162float(lr[i]) - mx);
  sum = block_sum(sum, scratch);
  if (threadIdx.x == 0) row_loss[row] = logf(sum) - (tgt_ok ? target_logit - mx : 0.f);
  if (dlogits != nullptr) {
    __nv_bfloat16* dr = dlogits + static_cast<long>(row) * ld;
    const float inv = 1.0f / sum;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
      float p = expf(__bfloat162float(lr[i]) - mx) * inv;
      if (i == tgt) p -= 1.0f;
      dr[i] = __float2bfloat16_rn(p * grad_scale);
    }
  }
}

// The same for rows that fit in registers (vocab a multiple of 8 and at most
// 256 x 8 x 8 = 16384, 16-byte aligned rows): the row is read once with 16-byte
// loads, exp is evaluated once per element and the gradient leaves as 16-byte
// stores.
constexpr int kCeVecs = 8;  // 16-byte vectors per thread
__global__ void __launch_bounds__(256)
cross_entropy_vec_kernel(const __nv_bfloat16* __restrict__ logits, long ld,
                         const int64_t* __restrict__ targets, float* __restrict__ row_loss,
                         __nv_bfloat16* __restrict__ dlogits, float grad_scale, int vocab) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[33];
  const int row = blockIdx.x;
  const __nv_bfloat16* lr = logits + static_cast<long>(row) * ld;
  const int nvec = vocab >> 3;
  const int64_t tgt = targets[row];
  const bool tgt_ok = tgt >= 0 && tgt < vocab;
  const float target_logit = (threadIdx.x == 0 && tgt_ok) ? __bfloat162float(lr[tgt]) : 0.f;
  float e[kCeVecs][8];
  float mx = -INFINITY;
#pragma unroll
  for (int k = 0; k < kCeVecs; ++k) {
    const int idx = threadIdx.x + k * 256;
    if (idx < nvec) {
      const uint4 q = *reinterpret_cast<const uint4*>(lr + idx * 8);
      const float2 a = unpack_bf16(q.x), b = unpack_bf16(q.y), c = unpack_bf16(q.z),
                   d = unpack_bf16(q.w);
      e[k][0] = a.x; e[k][1] = a.y; e[k][2] = b.x; e[k][3] = b.y;
      e[k][4] = c.x; e[k][5] = c.y; e[k][6] = d.x; e[k][7] = d.y;
#pragma unroll
      for (int j = 0; j < 8; ++j) mx = fmaxf(mx, e[k][j]);
    }
  }
  mx = block_max(mx, scratch);
  float sum = 0.f;
#pragma unroll
  for (int k = 0; k < kCeVecs; ++k) {
    if (threadIdx.x + k * 256 < nvec) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        e[k][j] = expf(e[k][j] - mx);
        sum += e[k][j];
      }
    }
  }
  sum = block_sum(sum, scratch);
  if (threadIdx.x == 0) row_loss[row] = logf(sum) - (tgt_ok ? target_logit - mx : 0.f);
  if (dlogits != nullptr) {
    __nv_bfloat16* dr = dlogits + static_cast<long>(row) * ld;
    const float inv = 1.0f / sum;
#pragma unroll
    for (int k = 0; k < kCeVecs; ++k) {
      const int idx = threadIdx.x + k * 256;
      if (idx < nvec) {
        float p[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          p[j] = e[k][j] * inv;
          if (idx * 8 + j == tgt) p[j] -= 1.0f;
          p[j] *= grad_scale;
        }
        uint4 o;
        o.x = pack_bf16(p[0], p[1]);
        o.y = pack_bf16(p[2], p[3]);
        o.z = pack_bf16(p[4], p[5]);
        o.w = pack_bf16(p[6], p[7]);
        *reinterpret_cast<uint4*>(dr + idx * 8) = o;
      }
    }
  }
}

// -------------------------------------------------------------- optimizer ---
constexpr int kSqnormThreads = 512;
constexpr long kSqnormChunk = 1 << 16;  // elements per block

__global__ void __launch_bounds__(kSqnormThreads)
sqnorm_partial_kernel(const float* __restrict__ x, long n, float* __restrict__ partial) {
  __shared__ float scratch[33];
  const long begin = static_cast<long>(blockIdx.x) * kSqnormChunk;
  const long end = begin + kSqnormChunk < n ? begin + kSqnormChunk : n;
  float s = 0.f;
  // begin is a multiple of 4 elements, so float4 loads are aligned when x is.
  const long vec_end = begin + ((end - begin) & ~3L);
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    for (long i = begin + threadIdx.x * 4L; i < vec_end; i += kSqnormThreads * 4L) {
      const float4 v = *reinterpret_cast<const float4*>(x + i);
      s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    for (long i = vec_end + threadIdx.x; i < end; i += kSqnormThreads) s += x[i] * x[i];
  } else {
    for (long i = begin + threadIdx.x; i < end; i += kSqnormThreads) s += x[i] * x[i];
  }
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

__global__ void norm_finalize_kernel(const float* __restrict__ partial, int n, float sum_scale,
                                     float max_norm, float* __restrict__ out) {
  // Double accumulation in a fixed order keeps the total independent of n's split.
  double s = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += static_cast<double>(partial[i]);
  __shared__ double dsum[256];
  dsum[threadIdx.x] = s;
  __syncthreads();
  for (int o = blockDim.x >> 1; o > 0; o >>= 1) {
    if (threadIdx.x < o) dsum[threadIdx.x] += dsum[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    const float norm = sqrtf(static_cast<float>(dsum[0] * static_cast<double>(sum_scale)));
    out[0] = norm;
    const float coef = max_norm / (norm + 1e-6f);
    out[1] = coef < 1.0f ? coef : 1.0f;
    out[2] = isfinite(norm) ? 1.0f : 0.0f;
  }
}

// One AdamW update, in the operation order of torch.optim.AdamW (single-tensor path).
__device__ __forceinline__ void adamw_one(float& pi, float gi, float& mi, float& vi, float lr,
                                          float beta1, float beta2, float eps, float wd,
                                          float step_size, float bias2_sqrt, float grad_scale,
                                          bool has_coef, float coef) {
  if (grad_scale != 1.0f) gi *= grad_scale;
  if (has_coef) gi *= coef;
  pi = pi * (1.0f - lr * wd);
  mi = mi + (gi - mi) * (1.0f - beta1);
  vi = vi * beta2 + (1.0f - beta2) * gi * gi;
  const float denom = sqrtf(vi) / bias2_sqrt + eps;
  pi = pi - step_size * (mi / denom);
}

// Four elements per thread and trip (16-byte loads and stores on every stream) when
// the arrays allow it; 34 bytes move per element, so the kernel is pure bandwidth.
__global__ void __launch_bounds__(256)
adamw_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m,
             float* __restrict__ v, __nv_bfloat16* __restrict__ shadow, long n, float lr,
             float beta1, float beta2, float eps, float wd, float bias1, float bias2_sqrt,
             const float* __restrict__ grad_coef, float grad_scale,
             const float* __restrict__ ok_flag, int vectorized) {
  if (ok_flag != nullptr && *ok_flag == 0.0f) return;
  const bool has_coef = grad_coef != nullptr;
  const float coef = has_coef ? *grad_coef : 1.0f;
  const float step_size = lr / bias1;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  const long i0 = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  long done = 0;
  if (vectorized) {
    const long n4 = n >> 2;
    for (long i = i0; i < n4; i += stride) {
      float4 p4 = reinterpret_cast<float4*>(p)[i];
      const float4 g4 = reinterpret_cast<const float4*>(g)[i];
      float4 m4 = reinterpret_cast<float4*>(m)[i];
      float4 v4 = reinterpret_cast<float4*>(v)[i];
      adamw_one(p4.x, g4.x, m4.x, v4.x, lr, beta1, beta2, eps, wd, step_size, bias2_sqrt,
                grad_scale, has_coef, coef);
      adamw_one(p4.y, g4.y, m4.y, v4.y, lr, beta1, beta2, eps, wd, step_size, bias2_sqrt,
                grad_scale, has_coef, coef);
      adamw_one(p4.z, g4.z, m4.z, v4.z, lr, beta1, beta2, eps, wd, step_size, bias2_sqrt,
                grad_scale, has_coef, coef);
      adamw_one(p4.w, g4.w, m4.w, v4.w, lr, beta1, beta2, eps, wd, step_size, bias2_sqrt,
                grad_scale, has_coef, coef);
      reinterpret_cast<float4*>(p)[i] = p4;
      reinterpret_cast<float4*>(m)[i] = m4;
      reinterpret_cast<float4*>(v)[i] = v4;
      if (shadow != nullptr) {
        uint2 o;
        o.x = pack_bf16(p4.x, p4.y);
        o.y = pack_bf16(p4.z, p4.w);
        reinterpret_cast<uint2*>(shadow)[i] = o;
      }
    }
    done = n4 << 2;
  }
  for (long i = done + i0; i < n; i += stride) {
    float pi = p[i], mi = m[i], vi = v[i];
    adamw_one(pi, g[i], mi, vi, lr, beta1, beta2, eps, wd, step_size, bias2_sqrt, grad_scale,
              has_coef, coef);
    p[i] = pi;
    m[i] = mi;
    v[i] = vi;
    if (shadow != nullptr) shadow[i] = __float2bfloat16_rn(pi);
  }
}

// ------------------------------------------------------------------- misc ---
__global__ void cast_f32_bf16_kernel(const float* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                     long n) {
  pdl_launch_dependents();
  pdl_wait();
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  const long i0 = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const bool aligned = ((reinterpret_cast<uintptr_t>(x) & 15) | (reinterpret_cast<uintptr_t>(y) & 7)) == 0;
  if (aligned) {
    const long n4 = n >> 2;
    for (long i = i0; i < n4; i += stride) {
      const float4 v = reinterpret_cast<const float4*>(x)[i];
      uint2 o;
      o.x = pack_bf16(v.x, v.y);
      o.y = pack_bf16(v.z, v.w);
      reinterpret_cast<uint2*>(y)[i] = o;
    }
    for (long i = (n4 << 2) + i0; i < n; i += stride) y[i] = __float2bfloat16_rn(x[i]);
  } else {
    for (long i = i0; i < n; i += stride) y[i] = __float2bfloat16_rn(x[i]);
  }
}

__global__ void scale_f32_kernel(float* __restrict__ x, long n, const float* __restrict__ coef,
                                 float scale) {
  const float c = (coef != nullptr ? *coef : 1.0f) * scale;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    x[i] *= c;
}

// x *= *coef for bf16 data, and nothing at all when *coef is exactly 1: the gradient
// that arrives at a loss is almost always the constant one, known only on the device.
__global__ void scale_bf16_unless_one_kernel(__nv_bfloat16* __restrict__ x, long n,
                                             const float* __restrict__ coef) {
  const float c = *coef;
  if (c == 1.0f) return;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
    x[i] = __float2bfloat16_rn(__bfloat162float(x[i]) * c);
}

__global__ void embedding_fwd_kernel(const float* __restrict__ weight,
                                     const int64_t* __restrict__ ids, float* __restrict__ out,
                                     int rows, int dim, int vocab) {
  const int row = blockIdx.x;
  int64_t id = ids[row];
  if (id < 0 || id >= vocab) id = 0;  // validated on the host; never index out of range
  const float* src = weight + id * dim;
  float* dst = out + static_cast<long>(row) * dim;
  if ((dim & 3) == 0) {
    for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4)
      *reinterpret_cast<float4*>(dst + i) = *reinterpret_cast<const float4*>(src + i);
  } else {
    for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = src[i];
  }
}

// Embedding backward: dW[v] (+)= sum of dx[t] over the tokens t with ids[t] == v, added
// in token order so the result does not depend on scheduling (the reference relies
// on autograd's embedding backward, src/llmlab/model/layers.py:60-74).  Two kernels:
// the first links the tokens of each id into a chain (next[t] = next later token with
// the same id, found by scanning the ids in shared memory; head[v] = its first token,
// by atomicMin); the second walks one chain per vocabulary row.  No sort, no dense
// temporary.
constexpr int kNoToken = 0x7F7F7F7F;  // what a byte-wise memset of 0x7F leaves in head[]

__global__ void __launch_bounds__(64)
embedding_links_kernel(const int64_t* __restrict__ ids, int rows, int vocab,
                       int* __restrict__ next, int* __restrict__ head) {
  extern __shared__ __align__(16) int sid[];
  for (int i = threadIdx.x; i < rows; i += blockDim.x) {
    const int64_t v = ids[i];
    sid[i] = (v < 0 || v >= vocab) ? 0 : static_cast<int>(v);  // same clamp as the forward
  }
  __syncthreads();
  for (int t = blockIdx.x * blockDim.x + threadIdx.x; t < rows; t += gridDim.x * blockDim.x) {
    const int id = sid[t];
    atomicMin(head + id, t);  // the first token of the id, whatever the arrival order
    // next later token with the same id: scalar up to a 16-byte boundary, then four
    // ids per shared-memory load
    int nx = -1;
    int u = t + 1;
    for (; u < rows && (u & 3) != 0 && nx < 0; ++u)
      if (sid[u] == id) nx = u;
    if (nx < 0) {
      for (; u + 3 < rows; u += 4) {
        const int4 q = *reinterpret_cast<const int4*>(sid + u);
        if (q.x == id || q.y == id || q.z == id || q.w == id) {
          nx = q.x == id ? u : q.y == id ? u + 1 : q.z == id ? u + 2 : u + 3;
          break;
        }
      }
      if (nx < 0)
        for (; u < rows && nx < 0; ++u)
          if (sid[u] == id) nx = u;
    }
    next[t] = nx;
  }
}

__global__ void __launch_bounds__(128)
embedding_bwd_kernel(const float* __restrict__ dx, const int* __restrict__ next,
                     const int* __restrict__ head, float* __restrict__ dweight, int dim,
                     int accumulate) {
  const int v = blockIdx.x;
  float* dst = dweight + static_cast<long>(v) * dim;
  int t = head[v];
  if (t == kNoToken) {
    if (!accumulate)
      for (int i = threadIdx.x; i < dim; i += blockDim.x) dst[i] = 0.f;
    return;
  }
  if ((dim & 3) == 0) {
    for (int i = threadIdx.x * 4; i < dim; i += blockDim.x * 4) {
      float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
      for (int u = t; u >= 0; u = next[u]) {
        const float4 g = *reinterpret_cast<const float4*>(dx + static_cast<long>(u) * dim + i);
        sum.x += g.x; sum.y += g.y; sum.z += g.z; sum.w += g.w;
      }
      if (accumulate) {
        const float4 o = *reinterpret_cast<const float4*>(dst + i);
        sum.x += o.x; sum.y += o.y; sum.z += o.z; sum.w += o.w;
      }
      *reinterpret_cast<float4*>(dst + i) = sum;
    }
  } else {
    for (int i = threadIdx.x; i < dim; i += blockDim.x) {
      float sum = 0.f;
      for (int u = t; u >= 0; u = next[u]) sum += dx[static_cast<long>(u) * dim + i];
      dst[i] = accumulate ? dst[i] + sum : sum;
    }
  }
}

inline int grid_for(long n, int threads, int cap = 148 * 8) {
  long blocks = (n + threads - 1) / threads;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace sfl

using namespace sfl;
#define SFL_STREAM(s) static_cast<cudaStream_t>(s)
#define SFL_RET() return static_cast<int>(cudaGetLastError())

extern "C" int sfl_rmsnorm_fwd(const float* x, const float* w, void* y, float* rstd, int rows,
                               int dim, float eps, void* stream) {
  if (rows <= 0 || dim <= 0) return -2;
  static const bool plain = getenv("SFL_NORM_PLAIN") != nullptr;  // the one-warp-per-row loops
  if (!plain && dim % 128 == 0 && dim <= 1024) {
    const int vw = 4;
#define SFL_NORM_FWD(NCH)                                                                        \
  case NCH:                                                                                      \
    return launch_pdl(rmsnorm_fwd_vec_kernel<NCH>, dim3((rows + vw - 1) / vw), dim3(vw * 32), 0, \
                      SFL_STREAM(stream), x, w, static_cast<__nv_bfloat16*>(y), rstd, rows, eps);
    switch (dim / 128) {
      SFL_NORM_FWD(1) SFL_NORM_FWD(2) SFL_NORM_FWD(3) SFL_NORM_FWD(4)
      SFL_NORM_FWD(5) SFL_NORM_FWD(6) SFL_NORM_FWD(7) SFL_NORM_FWD(8)
    }
#undef SFL_NORM_FWD
  }
  const int warps = 8;
  return launch_pdl(rmsnorm_fwd_kernel, dim3((rows + warps - 1) / warps), dim3(warps * 32), 0,
                    SFL_STREAM(stream), x, w, static_cast<__nv_bfloat16*>(y), rstd, rows, dim, eps);
}

extern "C" int sfl_rmsnorm_bwd_blocks(int rows) {
  const int warps = kNormBwdThreads / 32;
  const int need = (rows + warps - 1) / warps;
  return need < kNormBwdBlocks ? (need < 1 ? 1 : need) : kNormBwdBlocks;
}

extern "C" int sfl_rmsnorm_bwd(const void* dy, const float* x, const float* w, const float* rstd,
                               const float* dres_in, float* dx_out, void* dx_bf16,
                               float* dw_partial, int rows, int dim, void* stream) {
  if (rows <= 0 || dim <= 0) return -2;
  const int blocks = sfl_rmsnorm_bwd_blocks(rows);
  const size_t smem = static_cast<size_t>(kNormBwdThreads / 32) * dim * sizeof(float);
  if (smem > 200 * 1024) return -2;
  static bool configured = false;
  if (!configured && smem > 48 * 1024) {
    cudaFuncSetAttribute(rmsnorm_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         200 * 1024);
    configured = true;
  }
  const __nv_bfloat16* dyp = static_cast<const __nv_bfloat16*>(dy);
  __nv_bfloat16* dxb = static_cast<__nv_bfloat16*>(dx_bf16);
  cudaStream_t st = SFL_STREAM(stream);
#define SFL_NORM_BWD(NCH)                                                                     \
  case NCH:                                                                                   \
    return launch_pdl(rmsnorm_bwd_vec_kernel<NCH>, dim3(blocks), dim3(kNormBwdThreads), smem, \
                      st, dyp, x, w, rstd, dres_in, dx_out, dxb, dw_partial, rows);
  static const bool plain = getenv("SFL_NORM_PLAIN") != nullptr;
#define SFL_NORM_PAIR(NCH)                                                                     \
  case NCH:                                                                                    \
    return launch_pdl(rmsnorm_bwd_pair_kernel<NCH>, dim3(blocks), dim3(kNormBwdThreads),       \
                      static_cast<size_t>(kNormBwdThreads / 64) * dim * sizeof(float), st, dyp, \
                      x, w, rstd, dres_in, dx_out, dxb, dw_partial, rows);
  if (!plain && dim % 256 == 0 && dim <= 1024) {
    switch (dim / 128) { SFL_NORM_PAIR(2) SFL_NORM_PAIR(4) SFL_NORM_PAIR(6) SFL_NORM_PAIR(8) }
  }
#undef SFL_NORM_PAIR
  if (dim % 128 == 0 && dim <= 1024) {
    switch (dim / 128) {
      SFL_NORM_BWD(1) SFL_NORM_BWD(2) SFL_NORM_BWD(3) SFL_NORM_BWD(4)
      SFL_NORM_BWD(5) SFL_NORM_BWD(6) SFL_NORM_BWD(7) SFL_NORM_BWD(8)
    }
  } else {
    return launch_pdl(rmsnorm_bwd_kernel, dim3(blocks), dim3(kNormBwdThreads), smem, st, dyp, x, w,
                      rstd, dres_in, dx_out, dxb, dw_partial, rows, dim);
  }
#undef SFL_NORM_BWD
  SFL_RET();
}

extern "C" int sfl_rmsnorm_dw_reduce(const float* partial, int blocks, float* dw, int dim,
                                     int accumulate, void* stream) {
  return launch_pdl(rmsnorm_dw_reduce_kernel, dim3((dim + 31) / 32), dim3(32 * kDwReduceWarps), 0,
                    SFL_STREAM(stream), partial, blocks, dw, dim, accumulate,
                    static_cast<const float*>(nullptr), static_cast<float*>(nullptr), 0);
}

// Two folds of the same shape in one launch.
extern "C" int sfl_rmsnorm_dw_reduce2(const float* partial_a, float* dw_a, int accumulate_a,
                                      const float* partial_b, float* dw_b, int accumulate_b,
                                      int blocks, int dim, void* stream) {
  if (partial_a == nullptr || partial_b == nullptr || dw_a == nullptr || dw_b == nullptr) return -2;
  return launch_pdl(rmsnorm_dw_reduce_kernel, dim3((dim + 31) / 32, 2), dim3(32 * kDwReduceWarps),
                    0, SFL_STREAM(stream), partial_a, blocks, dw_a, dim, accumulate_a, partial_b,
                    dw_b, accumulate_b);
}

extern "C" int sfl_cross_entropy(const void* logits, long ld, const int64_t* targets,
                                 float* row_loss, void* dlogits, float grad_scale, int rows,
                                 int vocab, void* stream) {
  if (rows <= 0 || vocab <= 0) return -2;
  const uintptr_t bases = reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(dlogits);
  if ((vocab & 7) == 0 && vocab <= 256 * kCeVecs * 8 && (ld & 7) == 0 && (bases & 15) == 0)
    return launch_pdl(cross_entropy_vec_kernel, dim3(rows), dim3(256), 0, SFL_STREAM(stream),
                      static_cast<const __nv_bfloat16*>(logits), ld, targets, row_loss,
                      static_cast<__nv_bfloat16*>(dlogits), grad_scale, vocab);
  return launch_pdl(cross_entropy_kernel, dim3(rows), dim3(256), 0, SFL_STREAM(stream),
                    static_cast<const __nv_bfloat16*>(logits), ld, targets, row_loss,
                    static_cast<__nv_bfloat16*>(dlogits), grad_scale, vocab);
}

extern "C" int sfl_sqnorm_blocks(long n) {
  return static_cast<int>((n + kSqnormChunk - 1) / kSqnormChunk);
}

extern "C" int sfl_sqnorm_partial(const float* x, long n, float* partial, void* stream) {
  if (n <= 0) return -2;
  sqnorm_partial_kernel<<<sfl_sqnorm_blocks(n), kSqnormThreads, 0, SFL_STREAM(stream)>>>(x, n,
                                                                                       partial);
  SFL_RET();
}

extern "C" int sfl_norm_finalize(const float* partial, int n, float sum_scale, float max_norm,
                                 float* out, void* stream) {
  norm_finalize_kernel<<<1, 256, 0, SFL_STREAM(stream)>>>(partial, n, sum_scale, max_norm, out);
  SFL_RET();
}

extern "C" int sfl_adamw(float* p, const float* g, float* m, float* v, void* shadow, long n,
                         float lr, float beta1, float beta2, float eps, float wd, float bias1,
                         float bias2, const float* grad_coef, float grad_scale,
                         const float* ok_flag, void* stream) {
  if (n <= 0) return 0;
  const uintptr_t all = reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) |
                        reinterpret_cast<uintptr_t>(m) | reinterpret_cast<uintptr_t>(v);
  const int vectorized = (all & 15) == 0 && (reinterpret_cast<uintptr_t>(shadow) & 7) == 0;
  adamw_kernel<<<grid_for(vectorized ? (n + 3) / 4 : n, 256, 148 * 16), 256, 0,
                 SFL_STREAM(stream)>>>(
      p, g, m, v, static_cast<__nv_bfloat16*>(shadow), n, lr, beta1, beta2, eps, wd, bias1,
      sqrtf(bias2), grad_coef, grad_scale, ok_flag, vectorized);
  SFL_RET();
}

extern "C" int sfl_cast_f32_to_bf16(const float* x, void* y, long n, void* stream) {
  if (n <= 0) return 0;
  return launch_pdl(cast_f32_bf16_kernel, dim3(grid_for((n + 3) / 4, 256)), dim3(256), 0,
                    SFL_STREAM(stream), x, static_cast<__nv_bfloat16*>(y), n);
}

extern "C" int sfl_scale_f32(float* x, long n, const float* coef, float scale, void* stream) {
  if (n <= 0) return 0;
  scale_f32_kernel<<<grid_for(n, 256), 256, 0, SFL_STREAM(stream)>>>(x, n, coef, scale);
  SFL_RET();
}

extern "C" int sfl_scale_bf16_unless_one(void* x_bf16, long n, const float* coef_dev,
                                         void* stream) {
  if (x_bf16 == nullptr || coef_dev == nullptr || n < 0) return -2;
  if (n == 0) return 0;
  scale_bf16_unless_one_kernel<<<grid_for(n, 256), 256, 0, SFL_STREAM(stream)>>>(
      static_cast<__nv_bfloat16*>(x_bf16), n, coef_dev);
  SFL_RET();
}

extern "C" int sfl_embedding_fwd(const float* weight, const int64_t* ids, float* out, int rows,
                                 int dim, int vocab, void* stream) {
  if (rows <= 0) return -2;
  embedding_fwd_kernel<<<rows, 128, 0, SFL_STREAM(stream)>>>(weight, ids, out, rows, dim, vocab);
  SFL_RET();
}

extern "C" int sfl_embedding_bwd(const float* dx, const int64_t* ids, float* dweight, int rows,
                                 int dim, int vocab, int accumulate, int* next_scratch,
                                 int* head_scratch, void* stream) {
  if (rows <= 0 || dim <= 0 || vocab <= 0 || dx == nullptr || ids == nullptr ||
      dweight == nullptr || next_scratch == nullptr || head_scratch == nullptr)
    return -2;
  const size_t smem = static_cast<size_t>(rows) * sizeof(int);
  if (smem > 200 * 1024) return -2;  // ids must fit in shared memory; callers fall back
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(embedding_links_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured = true;
  }
  cudaError_t e = cudaMemsetAsync(head_scratch, 0x7F, static_cast<size_t>(vocab) * sizeof(int),
                                  SFL_STREAM(stream));
  if (e != cudaSuccess) return static_cast<int>(e);
  const int ctas = grid_for(rows, 64, 148 * 2);
  embedding_links_kernel<<<ctas, 64, smem, SFL_STREAM(stream)>>>(ids, rows, vocab, next_scratch,
                                                                 head_scratch);
  embedding_bwd_kernel<<<vocab, 128, 0, SFL_STREAM(stream)>>>(dx, next_scratch, head_scratch,
                                                              dweight, dim, accumulate);
  SFL_RET();
}

extern "C" const char* sfl_version(void) { return "sfl_b200 sm_100a"; }

// sizeof of every structure that crosses the C interface, in the order of the
// enum below, so a binding can verify its mirrors field for field.
extern "C" int sfl_struct_sizes(int* sizes, int capacity) {
  const int values[] = {static_cast<int>(sizeof(SflGemmEpilogue)), static_cast<int>(sizeof(SflWgradProblem)),
                        static_cast<int>(sizeof(SflAttnTensor)), static_cast<int>(sizeof(SflAttnMask)),
                        static_cast<int>(sizeof(SflComm)), static_cast<int>(sizeof(SflBlockArgs)),
                        static_cast<int>(sizeof(SflTpFuse))};
  const int count = static_cast<int>(sizeof(values) / sizeof(values[0]));
  for (int i = 0; i < count && i < capacity; ++i) sizes[i] = values[i];
  return count;
}
