// Issue rate of tcgen05.mma.cta_group::1.kind::f16 from one thread, and from two
// threads of different warps at once: one CTA, 1024 back-to-back 128 x N x 16
// products on zeroed shared memory, timed with clock64 from first issue to the last
// issue and to completion (tcgen05.commit + mbarrier).  Three ways of issuing: from
// inside a single-lane branch, from a converged warp with one elected lane, and the
// latter with the A operand in tensor memory (no 4 KB shared-memory read per product).
// Built and run by
//   python -m systems_for_llms_b200.ops.microbench mma
// It answers how small an MMA may be before the instruction, not the arithmetic,
// bounds the tensor pipe (attention with head dimension 64 issues N = 64 products).
#include <cstdio>
#include <cuda_runtime.h>
#include "ptx.cuh"
using namespace sfl;

// Background load for the contention rows: while warp 0 issues, warps 4.. (two per lane
// quarter) keep reading (BG 1) or reading and writing (BG 2) 32-column chunks of tensor
// memory, or (BG 3) reading shared memory with 16-byte loads.
template <int BG>
__device__ __forceinline__ void background(uint32_t tmem, const uint8_t* smem, volatile int* stop) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t base = tmem + (static_cast<uint32_t>((warp & 3) * 32) << 16) + 384 + ((warp >> 2) & 1) * 64;
  uint32_t r[32];
  uint32_t sink = 0;
  for (int it = 0; it < (1 << 20) && !*stop; ++it) {
    if (BG == 1 || BG == 2) {
      tmem_ld_32x32(base, r);
      tmem_ld_32x32(base + 32, r);
      tmem_ld_wait();
      if (BG == 2) {
        uint32_t a[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) a[i] = r[i] + it;
        tmem_st_32x16(base, a);
        tmem_st_32x16(base + 16, a);
        tmem_st_wait();
      }
      sink += r[0];
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        uint32_t x, y, z, w;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                     : "=r"(x), "=r"(y), "=r"(z), "=r"(w)
                     : "r"(smem_u32(smem) + 32768 + ((warp * 32 + lane) * 16 + i * 4096) % 32768));
        sink += x;
      }
    }
  }
  if (sink == 0x12345678u) *stop = 2;
}

// MODE 0 lane-0 branch, 1 elected lane of a converged warp, 2 = 1 + A in TMEM; MODE 3 / 4 are
// 1 / 2 with the B operand MN-major (N contiguous, as the V tile of an attention P V product)
template <int N, int MODE, int BG = 0>
__global__ void __launch_bounds__(384, 1) bench(long long* out, int iters, int two) {
  __shared__ int stop_flag;
  if (threadIdx.x == 0) stop_flag = 0;
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ uint64_t bar[2];
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) { mbar_init(&bar[0], 1); mbar_init(&bar[1], 1); mbar_fence_init(); }
  if (warp == 0) { tmem_alloc(&tmem_slot, 512); tmem_relinquish(); }
  for (int i = threadIdx.x; i < 64 * 1024 / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(smem)[i] = 0;
  fence_proxy_async_smem();
  tc_fence_before(); __syncthreads(); tc_fence_after();
  const uint32_t tmem = tmem_slot;
  constexpr bool kBmn = MODE >= 3;
  constexpr uint32_t idesc = umma_idesc_bf16(128, N, false, kBmn);
  if (MODE == 0) {
    if (lane == 0 && (warp == 0 || (two && warp == 1))) {
      const uint64_t a = umma_smem_desc(smem_u32(smem), 16, 1024);
      const uint64_t b = umma_smem_desc(smem_u32(smem) + 16384, 16, 1024);
      long long t0 = clock64();
      for (int i = 0; i < iters; ++i) {
#pragma unroll
        for (int k = 0; k < 4; ++k)
          umma_bf16_ss(tmem + warp * 256, umma_desc_advance(a, k * 32), umma_desc_advance(b, k * 32), idesc, (i | k) != 0);
      }
      long long t1 = clock64();
      umma_commit(&bar[warp]);
      mbar_wait(&bar[warp], 0);
      long long t2 = clock64();
      out[warp * 2] = t1 - t0; out[warp * 2 + 1] = t2 - t0;
    }
  } else if (BG != 0 && warp >= 4) {
    background<BG>(tmem, smem, &stop_flag);
  } else if (warp == 0 || (two && warp == 1)) {
    const uint64_t a = umma_smem_desc(smem_u32(smem), 16, 1024);
    // MN-major B: 16 reduction rows of 128 B per step (2 KB apart), 64-wide N blocks 16 KB apart
    const uint64_t b = kBmn ? umma_smem_desc(smem_u32(smem) + 16384, 16384, 1024)
                            : umma_smem_desc(smem_u32(smem) + 16384, 16, 1024);
    constexpr int kBStep = kBmn ? 2048 : 32;
    const uint32_t acc = tmem + warp * 256, a_tmem = tmem + warp * 256 + 192;
    long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (MODE == 2 || MODE == 4)
            umma_bf16_ts(acc, a_tmem + k * 8, umma_desc_advance(b, k * kBStep), idesc, (i | k) != 0);
          else
            umma_bf16_ss(acc, umma_desc_advance(a, k * 32), umma_desc_advance(b, k * kBStep), idesc, (i | k) != 0);
        }
      }
      __syncwarp();
    }
    long long t1 = clock64();
    if (elect_one()) umma_commit(&bar[warp]);
    __syncwarp();
    mbar_wait(&bar[warp], 0);
    long long t2 = clock64();
    if (lane == 0) { out[warp * 2] = t1 - t0; out[warp * 2 + 1] = t2 - t0; }
    if (BG != 0) *reinterpret_cast<volatile int*>(&stop_flag) = 1;
  }
  tc_fence_before(); __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

template <int N, int MODE = 0, int BG = 0> void run(int two) {
  long long* d; cudaMalloc(&d, 64); cudaMemset(d, 0, 64);
  cudaFuncSetAttribute(bench<N, MODE, BG>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  const int iters = 256;
  const int threads = BG != 0 ? 384 : 128;
  bench<N, MODE, BG><<<1, threads, 64 * 1024>>>(d, iters, two);
  bench<N, MODE, BG><<<1, threads, 64 * 1024>>>(d, iters, two);
  long long h[4]; cudaMemcpy(h, d, 32, cudaMemcpyDeviceToHost);
  cudaError_t e = cudaDeviceSynchronize();
  printf("%s%s N=%3d threads=%d: issue %.1f cyc/MMA, complete %.1f cyc/MMA (thread1: %.1f / %.1f) %s\n",
         MODE == 0 ? "lane-0 branch " : MODE == 1 ? "elected lane  " : MODE == 2 ? "elected, A TMEM"
         : MODE == 3 ? "elected, B MN-major" : "elected, A TMEM, B MN-major",
         BG == 0 ? "" : BG == 1 ? " + 8 warps tcgen05.ld" : BG == 2 ? " + 8 warps tcgen05.ld/st" : " + 8 warps ld.shared", N, two + 1,
         h[0] / (4.0 * iters), h[1] / (4.0 * iters), h[2] / (4.0 * iters), h[3] / (4.0 * iters), cudaGetErrorString(e));
  cudaFree(d);
}
int main() {
  run<64>(0); run<128>(0); run<256>(0);
  run<64>(1); run<128>(1); run<256>(1);
  run<64, 1>(0); run<128, 1>(0); run<256, 1>(0);
  run<64, 2>(0); run<128, 2>(0);
  run<64, 1>(1); run<64, 2>(1);
  run<64, 1, 1>(0); run<64, 1, 2>(0); run<64, 1, 3>(0);
  run<64, 2, 1>(0); run<64, 2, 2>(0); run<64, 2, 3>(0);
  run<128, 1, 2>(0);
  run<64, 3>(0); run<64, 4>(0); run<128, 3>(0); run<128, 4>(0);
  return 0;
}
