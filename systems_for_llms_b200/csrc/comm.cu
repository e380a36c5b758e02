// Collectives over NVLink peer memory, fused with the arithmetic around them.
//
// Every rank allocates the same "symmetric" buffers with cudaMalloc, exports
// them as CUDA IPC handles and maps its peers' buffers, so a kernel holds a table
// of up to 8 base pointers and reads or writes any peer with plain loads and
// stores that travel over NVLink / NVSwitch.  Synchronisation uses flag words in
// a second symmetric buffer: a rank publishes an epoch number into its slot of
// every peer's flag array (system-scope release) and waits for all slots of its
// own array to reach that epoch (system-scope acquire).  Every wait is bounded
// and reports through a status word.
//
// Kernels:
//   allreduce_f32      ready-barrier, reduce my 1/W slice from all peers in rank
//                      order, scale, write the result to every peer, emit
//                      squared-norm partials of the reduced slice to every peer,
//                      done-barrier.  Replaces the NCCL bucket all-reduce of the
//                      reference's DDP (distributed/llmdist/train.py:263-265) plus
//                      the separate averaging and gradient-norm passes.
//   reduce_scatter_f32 same without the write-back: the owner keeps its reduced
//                      slice (sharded-optimizer path).
//   adamw_allgather    AdamW on the owned slice (fp32 master, moments) and push
//                      of the updated fp32 parameters and their bf16 shadow to
//                      every peer.  Replaces the reference's local AdamW + one
//                      broadcast per parameter (distributed/llmdist/
//                      optim_shard.py:119-126).
//   allgather_bytes    pull every peer's slice into the local buffer (FSDP
//                      parameter gather) .
//   reduce_rows_resid  tensor-parallel epilogue: sum W partial activations,
//                      add the residual, write the fp32 result to every peer.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <string.h>

#include "comm.cuh"
#include "ptx.cuh"
#include "sfl.h"

namespace sfl {

// Polling budget of a peer wait (iterations of roughly 200 ns).  The default, about ten
// seconds, is sized for training: ranks of one job reach a collective at different times
// (a garbage-collection pause, a page fault in a memory-mapped data file, lazy module
// loading on the first step) and a budget near the skew would turn ordinary jitter into a
// failed step.  Tests of the timeout path set a millisecond budget
// (sfl_comm_set_spin_limit).  When the budget runs out the wait gives up and the kernel
// reports a status, which the trainers read back every step.
__device__ uint32_t g_peer_spin_limit = 48u << 20;

__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t epoch) {
  const uint32_t limit = g_peer_spin_limit;
  for (uint32_t spin = 0; spin < limit; ++spin) {
    if (reached(ld_acquire_sys(flag), epoch)) return true;
    if (spin > 64) __nanosleep(200);
  }
  return false;
}

// Block 0 tells every peer "my data for `slot` is ready"; every block then
// waits until all peers have said the same.  Returns false on timeout.
__device__ __forceinline__ bool ready_barrier(const CommView& c, int slot, uint32_t epoch,
                                              int* status) {
  __shared__ int failed;
  if (threadIdx.x == 0) failed = 0;
  __syncthreads();
  if (blockIdx.x == 0 && threadIdx.x < c.world) {
    __threadfence_system();
    st_release_sys(flag_ptr(c.flags[threadIdx.x], slot, 0, c.rank), epoch);
  }
  if (threadIdx.x < c.world) {
    if (!wait_flag(flag_ptr(c.flags[c.rank], slot, 0, threadIdx.x), epoch)) {
      failed = 1;
      report_status(status, kStatusTimeoutPeer);
    }
  }
  __syncthreads();
  return failed == 0;
}

// Every block calls this after its last peer write.  The last block to arrive
// publishes "done" to all peers and waits for theirs, so when the kernel ends
// every peer's writes into this rank's buffers have landed.
//
// A block whose ready-wait ran out still arrives here (`healthy` false) without having
// touched any peer: the arrival counter then returns to zero as usual, so the slot works
// again after the host has dealt with the reported status, and "done" is not traded by a
// launch in which any wait failed on this rank.
__device__ __forceinline__ void done_barrier(const CommView& c, int slot, uint32_t epoch,
                                             int* status, bool healthy = true) {
  __shared__ int last;
  // The block barrier orders every thread's stores before thread 0's fence, which
  // is cumulative: one system fence per block instead of one per thread (each
  // waits for the block's outstanding peer stores, and 256 of them queue up).
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const uint32_t arrived = atomicAdd(counter_ptr(c.flags[c.rank], slot), 1u);
    last = arrived == gridDim.x - 1;
  }
  __syncthreads();
  if (!last) return;
  if (threadIdx.x == 0) *counter_ptr(c.flags[c.rank], slot) = 0;
  if (!healthy || (status != nullptr && *static_cast<volatile int*>(status) != 0)) return;
  if (threadIdx.x < c.world) {
    st_release_sys(flag_ptr(c.flags[threadIdx.x], slot, 1, c.rank), epoch);
    if (!wait_flag(flag_ptr(c.flags[c.rank], slot, 1, threadIdx.x), epoch))
      report_status(status, kStatusTimeoutPeer);
  }
  __syncthreads();
}

__device__ __forceinline__ float block_sum_256(float v) {
  __shared__ float scratch[33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < (blockDim.x >> 5) ? scratch[lane] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// Slice of [0, count) owned by `rank`, in float4 units, 4-element aligned.
__device__ __forceinline__ void slice_of(long count, int world, int rank, long* begin, long* end) {
  const long vecs = count >> 2;
  const long per = (vecs + world - 1) / world;
  long b = per * rank, e = b + per;
  if (b > vecs) b = vecs;
  if (e > vecs) e = vecs;
  *begin = b;
  *end = e;
}

// count must be a multiple of 4 elements and offset 16-byte aligned.
// W = world size known at compile time (0 = runtime loop), U = vectors per thread
// per trip: all W*U peer loads are issued before the first add so that enough
// bytes are in flight to cover NVLink latency.
template <int W, int U, bool WRITE_BACK>
__global__ void __launch_bounds__(256)
reduce_kernel(const CommView c, long offset, long count, float scale, int slot, uint32_t epoch,
              float* __restrict__ local_out, int accumulate_partial, int accumulate_out,
              int* status) {
  if (!ready_barrier(c, slot, epoch, status)) {
    done_barrier(c, slot, epoch, status, false);
    return;
  }
  long begin, end;
  slice_of(count, c.world, c.rank, &begin, &end);
  float sq = 0.f;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  const int world = W > 0 ? W : c.world;
  for (long i0 = begin + static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < end;
       i0 += stride * U) {
    float4 v[W > 0 ? W : 1][U];
    float4 acc[U];
    if constexpr (W > 0) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const long i = i0 + u * stride;
        if (i < end) {
#pragma unroll
          for (int p = 0; p < W; ++p)
            v[p][u] = ld_peer_f4(reinterpret_cast<const float*>(c.data[p]) + offset + (i << 2));
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long i = i0 + u * stride;
      if (i >= end) continue;
      const long elem = offset + (i << 2);
      float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
      // Fixed rank order: the owner of a slice is the only one summing it, so all
      // replicas receive the same bits and reruns reproduce them.
      if constexpr (W > 0) {
#pragma unroll
        for (int p = 0; p < W; ++p) {
          a.x += v[p][u].x; a.y += v[p][u].y; a.z += v[p][u].z; a.w += v[p][u].w;
        }
      } else {
#pragma unroll 1
        for (int p = 0; p < world; ++p) {
          const float4 t = ld_peer_f4(reinterpret_cast<const float*>(c.data[p]) + elem);
          a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
        }
      }
      a.x *= scale; a.y *= scale; a.z *= scale; a.w *= scale;
      sq += a.x * a.x + a.y * a.y + a.z * a.z + a.w * a.w;
      acc[u] = a;
      if constexpr (WRITE_BACK) {
#pragma unroll 1
        for (int p = 0; p < world; ++p)
          st_peer_f4(reinterpret_cast<float*>(c.data[p]) + elem, acc[u]);
      } else {
        float* dst = local_out != nullptr ? local_out + ((i - begin) << 2)
                                          : reinterpret_cast<float*>(c.data[c.rank]) + elem;
        if (accumulate_out) {
          const float4 old = *reinterpret_cast<const float4*>(dst);
          acc[u].x += old.x; acc[u].y += old.y; acc[u].z += old.z; acc[u].w += old.w;
        }
        *reinterpret_cast<float4*>(dst) = acc[u];
      }
    }
  }
  sq = block_sum_256(sq);
  if (threadIdx.x == 0 && accumulate_partial)
    sq += *partial_ptr(c.flags[c.rank], slot, c.rank, blockIdx.x);
  __shared__ float total;
  if (threadIdx.x == 0) total = sq;
  __syncthreads();
  if (threadIdx.x < c.world)
    *partial_ptr(c.flags[threadIdx.x], slot, c.rank, blockIdx.x) = total;
  // Entries of CTAs this launch does not have: zero on every peer, so that the norm
  // may add up all kMaxCtas entries of a slot whatever grid its reductions ran on.
  if (blockIdx.x == 0 && !accumulate_partial)
    for (int i = gridDim.x + threadIdx.x; i < kMaxCtas; i += blockDim.x)
      for (int p = 0; p < c.world; ++p) *partial_ptr(c.flags[p], slot, c.rank, i) = 0.f;
  done_barrier(c, slot, epoch, status);
}

template <bool WRITE_BACK>
int launch_reduce(const CommView& v, long offset, long count, float scale, int slot,
                  uint32_t epoch, float* local_out, int accumulate, int ctas, int* status,
                  cudaStream_t stream, int accumulate_out = 0) {
  switch (v.world) {
    case 2:
      reduce_kernel<2, 8, WRITE_BACK><<<ctas, 256, 0, stream>>>(v, offset, count, scale, slot,
                                                               epoch, local_out, accumulate,
                                                               accumulate_out, status);
      break;
    case 4:
      reduce_kernel<4, 4, WRITE_BACK><<<ctas, 256, 0, stream>>>(v, offset, count, scale, slot,
                                                               epoch, local_out, accumulate,
                                                               accumulate_out, status);
      break;
    case 8:
      reduce_kernel<8, 2, WRITE_BACK><<<ctas, 256, 0, stream>>>(v, offset, count, scale, slot,
                                                               epoch, local_out, accumulate,
                                                               accumulate_out, status);
      break;
    default:
      reduce_kernel<0, 1, WRITE_BACK><<<ctas, 256, 0, stream>>>(v, offset, count, scale, slot,
                                                               epoch, local_out, accumulate,
                                                               accumulate_out, status);
  }
  return static_cast<int>(cudaGetLastError());
}

// out[0] = sqrt(sum of all partials of the given slots), out[1] = clip coef, out[2] = finite.
// One block: thread t adds entries t, t + 256, ... of the [slot][rank][CTA] table in that
// order, then the 256 sums are folded by a fixed tree - the same arithmetic in the same order
// on every rank, whatever the grid size of the reductions that left the partials (unused CTA
// entries of a slot are zero, see reduce_kernel).
__global__ void __launch_bounds__(256)
comm_norm_finalize_kernel(const uint32_t* flags, const int* slots, int n_slots, int world,
                          float max_norm, const float* extra_sq, float* out) {
  __shared__ double fold[256];
  const float* table = reinterpret_cast<const float*>(flags + kFlagWords);
  const int per_slot = world * kMaxCtas;
  const long entries = static_cast<long>(n_slots) * per_slot;
  double mine = 0.0;
  for (long i = threadIdx.x; i < entries; i += 256) {
    const int s = static_cast<int>(i / per_slot);
    const int within = static_cast<int>(i - static_cast<long>(s) * per_slot);
    const int r = within / kMaxCtas, k = within - r * kMaxCtas;
    mine += static_cast<double>(table[(slots[s] * kMaxPeers + r) * kMaxCtas + k]);
  }
  fold[threadIdx.x] = mine;
  __syncthreads();
  for (int width = 128; width > 0; width >>= 1) {
    if (threadIdx.x < width) fold[threadIdx.x] += fold[threadIdx.x + width];
    __syncthreads();
  }
  if (threadIdx.x != 0) return;
  const double total = fold[0] + (extra_sq != nullptr ? static_cast<double>(*extra_sq) : 0.0);
  const float norm = sqrtf(static_cast<float>(total));
  out[0] = norm;
  const float coef = max_norm / (norm + 1e-6f);
  out[1] = coef < 1.0f ? coef : 1.0f;
  out[2] = isfinite(norm) ? 1.0f : 0.0f;
}

// AdamW on this rank's slice of the flat range, then push parameters (fp32)
// and shadow (bf16) to every peer.  `grad` holds the already reduced slice,
// m/v cover only the slice.  param / shadow are symmetric buffers.
struct ShardedAdamParams {
  long offset, count;  // the flat range being sharded (elements)
  const float* grad;   // local, slice-relative
  float* m;
  float* v;
  float lr, beta1, beta2, eps, wd, bias1, bias2_sqrt;
  const float* coef;   // clip coefficient (device)
  const float* ok;     // skip update when 0
};

// AdamW on this rank's slice of one range, results stored into every peer.
__device__ __forceinline__ void adamw_allgather_range(const CommView& params,
                                                      const CommView& shadows,
                                                      const ShardedAdamParams& a) {
  long begin, end;
  slice_of(a.count, params.world, params.rank, &begin, &end);
  const bool apply = a.ok == nullptr || *a.ok != 0.0f;
  const float coef = a.coef != nullptr ? *a.coef : 1.0f;
  const float step_size = a.lr / a.bias1;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  float* my_param = reinterpret_cast<float*>(params.data[params.rank]);
  for (long i = begin + static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < end;
       i += stride) {
    const long rel = (i - begin) << 2;
    const long elem = a.offset + (i << 2);
    float4 p4 = *reinterpret_cast<const float4*>(my_param + elem);
    if (apply) {
      const float4 g4 = *reinterpret_cast<const float4*>(a.grad + rel);
      float4 m4 = *reinterpret_cast<const float4*>(a.m + rel);
      float4 v4 = *reinterpret_cast<const float4*>(a.v + rel);
      float* pp = reinterpret_cast<float*>(&p4);
      const float* gg = reinterpret_cast<const float*>(&g4);
      float* mm = reinterpret_cast<float*>(&m4);
      float* vv = reinterpret_cast<float*>(&v4);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float g = gg[k] * coef;
        float pk = pp[k] * (1.0f - a.lr * a.wd);
        mm[k] = mm[k] + (g - mm[k]) * (1.0f - a.beta1);
        vv[k] = vv[k] * a.beta2 + (1.0f - a.beta2) * g * g;
        const float denom = sqrtf(vv[k]) / a.bias2_sqrt + a.eps;
        pp[k] = pk - step_size * (mm[k] / denom);
      }
      *reinterpret_cast<float4*>(a.m + rel) = m4;
      *reinterpret_cast<float4*>(a.v + rel) = v4;
    }
    uint2 sh;
    sh.x = pack_bf16(p4.x, p4.y);
    sh.y = pack_bf16(p4.z, p4.w);
#pragma unroll 1
    for (int p = 0; p < params.world; ++p) {
      st_peer_f4(reinterpret_cast<float*>(params.data[p]) + elem, p4);
      st_peer_u2(reinterpret_cast<__nv_bfloat16*>(shadows.data[p]) + elem, sh);
    }
  }
}

__global__ void __launch_bounds__(256)
adamw_allgather_kernel(const CommView params, const CommView shadows, ShardedAdamParams a,
                       int slot, uint32_t epoch, int* status) {
  // Peers must have finished reading the old parameters (their forward/backward
  // is complete when they reach this kernel), hence the ready barrier.
  if (!ready_barrier(params, slot, epoch, status)) {
    done_barrier(params, slot, epoch, status, false);
    return;
  }
  adamw_allgather_range(params, shadows, a);
  done_barrier(params, slot, epoch, status);
}

// The same update over a table of ranges (one per gradient bucket) between a single
// pair of barriers: launching and synchronising once per bucket costs more than the
// update itself when eight GPUs each own an eighth of a 25 MB bucket.
// ranges[3 r .. 3 r + 2] = {element offset, element count, offset of this rank's
// slice inside grad / m / v}.
__global__ void __launch_bounds__(256)
adamw_allgather_ranges_kernel(const CommView params, const CommView shadows,
                              ShardedAdamParams a, const long* __restrict__ ranges, int num_ranges,
                              int slot, uint32_t epoch, int* status) {
  if (!ready_barrier(params, slot, epoch, status)) {
    done_barrier(params, slot, epoch, status, false);
    return;
  }
  const float* grad = a.grad;
  float* m = a.m;
  float* v = a.v;
  for (int r = 0; r < num_ranges; ++r) {
    a.offset = ranges[3 * r];
    a.count = ranges[3 * r + 1];
    const long shard = ranges[3 * r + 2];
    a.grad = grad + shard;
    a.m = m + shard;
    a.v = v + shard;
    adamw_allgather_range(params, shadows, a);
  }
  done_barrier(params, slot, epoch, status);
}

// Pull bytes [offset + r*chunk, offset + (r+1)*chunk) from peer r into the same
// place of the local buffer, for every r != rank.  chunk is a multiple of 16.
__global__ void __launch_bounds__(256)
allgather_kernel(const CommView c, long offset_bytes, long chunk_bytes, int slot, uint32_t epoch,
                 int* status) {
  if (!ready_barrier(c, slot, epoch, status)) {
    done_barrier(c, slot, epoch, status, false);
    return;
  }
  const long vecs = chunk_bytes >> 4;
  const long total = vecs * (c.world - 1);
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  constexpr int U = 8;  // loads in flight per thread
  for (long i0 = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total;
       i0 += stride * U) {
    uint4 v[U];
    long byte[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long i = i0 + u * stride;
      byte[u] = -1;
      if (i < total) {
        int peer = static_cast<int>(i / vecs);
        const long w = i - peer * vecs;
        if (peer >= c.rank) ++peer;
        byte[u] = offset_bytes + peer * chunk_bytes + (w << 4);
        v[u] = ld_peer_u4(c.data[peer] + byte[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (byte[u] >= 0) *reinterpret_cast<uint4*>(c.data[c.rank] + byte[u]) = v[u];
  }
  done_barrier(c, slot, epoch, status);
}

// dst[r * chunk .. (r+1) * chunk) <- peer r's bytes [src_off, src_off + chunk), for
// every rank r (own slice included); dst is ordinary local memory.
__global__ void __launch_bounds__(256)
allgather_into_kernel(const CommView c, long src_off, long chunk_bytes, char* __restrict__ dst,
                      int slot, uint32_t epoch, int* status) {
  if (!ready_barrier(c, slot, epoch, status)) {
    done_barrier(c, slot, epoch, status, false);
    return;
  }
  const long vecs = chunk_bytes >> 4;
  const long total = vecs * c.world;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  constexpr int U = 8;
  for (long i0 = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total;
       i0 += stride * U) {
    uint4 v[U];
    long at[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const long i = i0 + u * stride;
      at[u] = -1;
      if (i < total) {
        const int peer = static_cast<int>(i / vecs);
        const long w = i - peer * vecs;
        at[u] = peer * chunk_bytes + (w << 4);
        v[u] = ld_peer_u4(c.data[peer] + src_off + (w << 4));
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u)
      if (at[u] >= 0) *reinterpret_cast<uint4*>(dst + at[u]) = v[u];
  }
  done_barrier(c, slot, epoch, status);
}

// Tensor-parallel row reduction.  Each rank holds bf16 partial sums
// partial[rows, cols] in the symmetric buffer `c` at byte offset in_off; the
// result out = resid + bf16(sum of partials) (fp32) is written to every peer's
// symmetric buffer `o` at byte offset out_off.  Rows are split across ranks.
template <bool OUT_BF16>
__global__ void __launch_bounds__(256)
reduce_rows_resid_kernel(const CommView c, const CommView o, long in_off, long out_off,
                         const float* __restrict__ resid, long rows, int cols, int slot,
                         uint32_t epoch, int* status) {
  if (!ready_barrier(c, slot, epoch, status)) {
    done_barrier(c, slot, epoch, status, false);
    return;
  }
  const long per = (rows + c.world - 1) / c.world;
  const long r0 = per * c.rank;
  const long r1 = r0 + per < rows ? r0 + per : rows;
  const int vec_per_row = cols >> 3;  // 8 bf16 per 16-byte vector
  const long total = (r1 > r0 ? r1 - r0 : 0) * vec_per_row;
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  for (long i = static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
    const long row = r0 + i / vec_per_row;
    const int col = static_cast<int>(i % vec_per_row) << 3;
    const long elem = row * cols + col;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    // Issue every peer's load before the first add (predicated full unroll).
    uint4 qs[kMaxPeers];
#pragma unroll
    for (int p = 0; p < kMaxPeers; ++p)
      if (p < c.world) qs[p] = ld_peer_u4(c.data[p] + in_off + elem * 2);
#pragma unroll
    for (int p = 0; p < kMaxPeers; ++p) {
      if (p >= c.world) break;
      const uint4 q = qs[p];
      const float2 a = unpack_bf16(q.x), b = unpack_bf16(q.y), cc = unpack_bf16(q.z),
                   d = unpack_bf16(q.w);
      acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
      acc[4] += cc.x; acc[5] += cc.y; acc[6] += d.x; acc[7] += d.y;
    }
    float4 lo, hi;
    if (resid != nullptr) {
      lo = *reinterpret_cast<const float4*>(resid + elem);
      hi = *reinterpret_cast<const float4*>(resid + elem + 4);
    } else {
      lo = hi = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    lo.x += bf16_round(acc[0]); lo.y += bf16_round(acc[1]);
    lo.z += bf16_round(acc[2]); lo.w += bf16_round(acc[3]);
    hi.x += bf16_round(acc[4]); hi.y += bf16_round(acc[5]);
    hi.z += bf16_round(acc[6]); hi.w += bf16_round(acc[7]);
    if constexpr (OUT_BF16) {
      uint4 packed;
      packed.x = pack_bf16(lo.x, lo.y);
      packed.y = pack_bf16(lo.z, lo.w);
      packed.z = pack_bf16(hi.x, hi.y);
      packed.w = pack_bf16(hi.z, hi.w);
#pragma unroll 1
      for (int p = 0; p < o.world; ++p) st_peer_u4(o.data[p] + out_off + elem * 2, packed);
    } else {
#pragma unroll 1
      for (int p = 0; p < o.world; ++p) {
        float* dst = reinterpret_cast<float*>(o.data[p] + out_off) + elem;
        st_peer_f4(dst, lo);
        st_peer_f4(dst + 4, hi);
      }
    }
  }
  done_barrier(c, slot, epoch, status);
}

// Same for fp32 partials without a residual (tensor-parallel input gradients).
__global__ void __launch_bounds__(256)
allreduce_rows_f32_kernel(const CommView c, const CommView o, long in_off, long out_off,
                          long count, int slot, uint32_t epoch, int* status) {
  if (!ready_barrier(c, slot, epoch, status)) {
    done_barrier(c, slot, epoch, status, false);
    return;
  }
  long begin, end;
  slice_of(count, c.world, c.rank, &begin, &end);
  const long stride = static_cast<long>(gridDim.x) * blockDim.x;
  for (long i = begin + static_cast<long>(blockIdx.x) * blockDim.x + threadIdx.x; i < end;
       i += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 vs[kMaxPeers];
#pragma unroll
    for (int p = 0; p < kMaxPeers; ++p)
      if (p < c.world)
        vs[p] = ld_peer_f4(reinterpret_cast<const float*>(c.data[p] + in_off) + (i << 2));
#pragma unroll
    for (int p = 0; p < kMaxPeers; ++p) {
      if (p >= c.world) break;
      acc.x += vs[p].x; acc.y += vs[p].y; acc.z += vs[p].z; acc.w += vs[p].w;
    }
#pragma unroll 1
    for (int p = 0; p < o.world; ++p)
      st_peer_f4(reinterpret_cast<float*>(o.data[p] + out_off) + (i << 2), acc);
  }
  done_barrier(c, slot, epoch, status);
}

CommView to_view(const SflComm* c, int which) {
  CommView v{};
  v.rank = c->rank;
  v.world = c->world;
  for (int i = 0; i < c->world && i < kMaxPeers; ++i) {
    v.data[i] = static_cast<char*>(which == 0 ? c->data[i] : c->data2[i]);
    v.flags[i] = static_cast<uint32_t*>(c->flags[i]);
  }
  return v;
}

int clamp_ctas(int ctas) {
  if (ctas <= 0) ctas = 32;
  if (ctas > kMaxCtas) ctas = kMaxCtas;
  return ctas;
}

}  // namespace sfl

using namespace sfl;

// ------------------------------------------------------------------- IPC ----
extern "C" int sfl_ipc_alloc(void** ptr, size_t bytes) {
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  return static_cast<int>(cudaMemset(*ptr, 0, bytes));
}
extern "C" int sfl_ipc_free(void* ptr) { return static_cast<int>(cudaFree(ptr)); }
extern "C" int sfl_ipc_get_handle(void* ptr, void* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
  return static_cast<int>(cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(handle64), ptr));
}
extern "C" int sfl_ipc_open_handle(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  return static_cast<int>(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}
extern "C" int sfl_ipc_close_handle(void* ptr) {
  return static_cast<int>(cudaIpcCloseMemHandle(ptr));
}
extern "C" int sfl_comm_set_spin_limit(unsigned iterations) {
  const int rc = sfl_gemm_tp_set_spin_limit(iterations);  // the fused GEMM + all-reduce kernels
  if (rc != 0) return rc;
  return static_cast<int>(cudaMemcpyToSymbol(g_peer_spin_limit, &iterations, sizeof(iterations)));
}
extern "C" long sfl_comm_flag_bytes(void) { return static_cast<long>(kFlagBytes); }
extern "C" int sfl_comm_slots(void) { return kSlots; }
extern "C" int sfl_comm_max_ctas(void) { return kMaxCtas; }

// ----------------------------------------------------------- collectives ----
extern "C" int sfl_allreduce_f32(const SflComm* comm, long offset, long count, float scale,
                                 int slot, unsigned epoch, int accumulate_partial, int ctas,
                                 int* status, void* stream) {
  if (comm == nullptr || comm->world < 1 || comm->world > kMaxPeers) return -2;
  if ((count & 3) || (offset & 3) || slot < 0 || slot >= kSlots) return -2;
  return launch_reduce<true>(to_view(comm, 0), offset, count, scale, slot, epoch, nullptr,
                             accumulate_partial, clamp_ctas(ctas), status,
                             static_cast<cudaStream_t>(stream));
}

extern "C" int sfl_reduce_scatter_f32(const SflComm* comm, long offset, long count, float scale,
                                      float* local_out, int slot, unsigned epoch,
                                      int accumulate_partial, int ctas, int* status,
                                      void* stream) {
  if (comm == nullptr || comm->world < 1 || comm->world > kMaxPeers) return -2;
  if ((count & 3) || (offset & 3) || slot < 0 || slot >= kSlots) return -2;
  return launch_reduce<false>(to_view(comm, 0), offset, count, scale, slot, epoch, local_out,
                              accumulate_partial & 1, clamp_ctas(ctas), status,
                              static_cast<cudaStream_t>(stream), (accumulate_partial >> 1) & 1);
}

extern "C" int sfl_comm_norm_finalize(const SflComm* comm, const int* slots_dev, int n_slots,
                                      int ctas, float max_norm, const float* extra_sq, float* out,
                                      void* stream) {
  (void)ctas;  // every CTA entry of a slot is added; unused ones are zero
  comm_norm_finalize_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(comm->flags[comm->rank]), slots_dev, n_slots, comm->world,
      max_norm, extra_sq, out);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sfl_adamw_allgather(const SflComm* comm, long offset, long count, const float* grad,
                                   float* m, float* v, float lr, float beta1, float beta2,
                                   float eps, float wd, float bias1, float bias2,
                                   const float* coef, const float* ok, int slot, unsigned epoch,
                                   int ctas, int* status, void* stream) {
  if (comm == nullptr || comm->world < 1 || comm->world > kMaxPeers) return -2;
  if ((count & 3) || (offset & 3) || slot < 0 || slot >= kSlots) return -2;
  ShardedAdamParams a{offset, count, grad, m, v, lr, beta1, beta2, eps, wd, bias1, sqrtf(bias2),
                      coef, ok};
  ctas = clamp_ctas(ctas);
  adamw_allgather_kernel<<<ctas, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      to_view(comm, 0), to_view(comm, 1), a, slot, epoch, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sfl_adamw_allgather_ranges(const SflComm* comm, const long* ranges, int num_ranges,
                                          const float* grad, float* m, float* v, float lr,
                                          float beta1, float beta2, float eps, float wd,
                                          float bias1, float bias2, const float* coef,
                                          const float* ok, int slot, unsigned epoch, int ctas,
                                          int* status, void* stream) {
  if (comm == nullptr || comm->world < 1 || comm->world > kMaxPeers) return -2;
  if (ranges == nullptr || num_ranges <= 0 || slot < 0 || slot >= kSlots) return -2;
  ShardedAdamParams a{0, 0, grad, m, v, lr, beta1, beta2, eps, wd, bias1, sqrtf(bias2), coef, ok};
  ctas = clamp_ctas(ctas);
  adamw_allgather_ranges_kernel<<<ctas, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      to_view(comm, 0), to_view(comm, 1), a, ranges, num_ranges, slot, epoch, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sfl_allgather_bytes(const SflComm* comm, long offset_bytes, long chunk_bytes,
                                   int slot, unsigned epoch, int ctas, int* status, void* stream) {
  if (comm == nullptr || comm->world < 1 || comm->world > kMaxPeers) return -2;
  if ((chunk_bytes & 15) || (offset_bytes & 15) || slot < 0 || slot >= kSlots) return -2;
  ctas = clamp_ctas(ctas);
  allgather_kernel<<<ctas, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      to_view(comm, 0), offset_bytes, chunk_bytes, slot, epoch, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sfl_allgather_into(const SflComm* comm, long src_off_bytes, long chunk_bytes,
                                  void* dst, int slot, unsigned epoch, int ctas, int* status,
                                  void* stream) {
  if (comm == nullptr || comm->world < 1 || comm->world > kMaxPeers) return -2;
  if ((chunk_bytes & 15) || (src_off_bytes & 15) || slot < 0 || slot >= kSlots) return -2;
  if (reinterpret_cast<uintptr_t>(dst) & 15) return -2;
  ctas = clamp_ctas(ctas);
  allgather_into_kernel<<<ctas, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      to_view(comm, 0), src_off_bytes, chunk_bytes, static_cast<char*>(dst), slot, epoch, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sfl_reduce_rows_resid(const SflComm* comm, long in_off, long out_off,
                                     const float* resid, long rows, int cols, int slot,
                                     unsigned epoch, int ctas, int* status, void* stream) {
  if (comm == nullptr || comm->world < 1 || comm->world > kMaxPeers) return -2;
  if ((cols & 7) || (in_off & 15) || (out_off & 15) || slot < 0 || slot >= kSlots) return -2;
  ctas = clamp_ctas(ctas);
  reduce_rows_resid_kernel<false><<<ctas, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      to_view(comm, 0), to_view(comm, 1), in_off, out_off, resid, rows, cols, slot, epoch, status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sfl_reduce_rows_bf16(const SflComm* comm, long in_off, long out_off, long rows,
                                    int cols, int slot, unsigned epoch, int ctas, int* status,
                                    void* stream) {
  if (comm == nullptr || comm->world < 1 || comm->world > kMaxPeers) return -2;
  if ((cols & 7) || (in_off & 15) || (out_off & 15) || slot < 0 || slot >= kSlots) return -2;
  ctas = clamp_ctas(ctas);
  reduce_rows_resid_kernel<true><<<ctas, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      to_view(comm, 0), to_view(comm, 1), in_off, out_off, nullptr, rows, cols, slot, epoch,
      status);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int sfl_allreduce_rows_f32(const SflComm* comm, long in_off, long out_off, long count,
                                      int slot, unsigned epoch, int ctas, int* status,
                                      void* stream) {
  if (comm == nullptr || comm->world < 1 || comm->world > kMaxPeers) return -2;
  if ((count & 3) || (in_off & 15) || (out_off & 15) || slot < 0 || slot >= kSlots) return -2;
  ctas = clamp_ctas(ctas);
  allreduce_rows_f32_kernel<<<ctas, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      to_view(comm, 0), to_view(comm, 1), in_off, out_off, count, slot, epoch, status);
  return static_cast<int>(cudaGetLastError());
}
