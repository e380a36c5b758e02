// Issue rate of tcgen05.mma.cta_group::1.kind::f16 from one thread, and from two
// threads of different warps at once: one CTA, 1024 back-to-back 128 x N x 16
// products on zeroed shared memory, timed with clock64 from first issue to the last
// issue and to completion (tcgen05.commit + mbarrier).  Built and run by
//   python -m systems_for_llms_b200.ops.microbench mma
// It answers how small an MMA may be before the instruction, not the arithmetic,
// bounds the tensor pipe (attention with head dimension 64 issues N = 64 products).
#include <cstdio>
#include <cuda_runtime.h>
#include "ptx.cuh"
using namespace sfl;

template <int N>
__global__ void __launch_bounds__(128, 1) bench(long long* out, int iters, int two) {
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
  constexpr uint32_t idesc = umma_idesc_bf16(128, N, false, false);
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
  tc_fence_before(); __syncthreads();
  if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem, 512); }
}

template <int N> void run(int two) {
  long long* d; cudaMalloc(&d, 64); cudaMemset(d, 0, 64);
  cudaFuncSetAttribute(bench<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
  const int iters = 256;
  bench<N><<<1, 128, 64 * 1024>>>(d, iters, two);
  bench<N><<<1, 128, 64 * 1024>>>(d, iters, two);
  long long h[4]; cudaMemcpy(h, d, 32, cudaMemcpyDeviceToHost);
  cudaError_t e = cudaDeviceSynchronize();
  printf("N=%3d threads=%d: issue %.1f cyc/MMA, complete %.1f cyc/MMA (thread1: %.1f / %.1f) %s\n", N, two + 1,
         h[0] / (4.0 * iters), h[1] / (4.0 * iters), h[2] / (4.0 * iters), h[3] / (4.0 * iters), cudaGetErrorString(e));
  cudaFree(d);
}
int main() {
  run<64>(0); run<128>(0); run<256>(0);
  run<64>(1); run<128>(1); run<256>(1);
  return 0;
}
