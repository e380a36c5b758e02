// Rate of the exponentials of an attention score tile: every thread turns a 128-element
// row into probabilities (scale, subtract, ex2, sum, pack to bf16), 148 CTAs, one or two
// warps per SM sub-partition, timed with clock64.  Built and run by
//   python -m systems_for_llms_b200.ops.microbench sfu
// Variants: fp32 ex2.approx (the kernels' form), with the row sum, with bf16 packing;
// half or a quarter of the exponentials evaluated as polynomials on the FMA pipes
// (Cody-Waite split and a cubic); packed half-precision ex2 (two results per
// instruction) converted back to fp32, or used as fp16 probabilities directly.
// It answers what the special-function unit allows per 128 x 128 tile (16,384
// exponentials per SM) and whether any of the usual ways around it pays on this part.
#include <cstdio>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
// 2^x for x <= 0 on the FMA pipes, accurate to bf16 precision
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -127.0f);
  const float whole = floorf(x);
  const float f = x - whole;  // in [0, 1)
  float p = fmaf(f, 0.0555041086648216f, 0.2402265069591007f);
  p = fmaf(p, f, 0.6931471805599453f);
  p = fmaf(p, f, 1.0f);
  return __int_as_float(__float_as_int(p) + (static_cast<int>(whole) << 23));
}
// two exponentials per special-function instruction: fp16 in, fp16 out
__device__ __forceinline__ uint32_t ex2_h2(float a, float b) {
  __half2 h = __floats2half2_rn(a, b);
  uint32_t y;
  asm("ex2.approx.f16x2 %0, %1;" : "=r"(y) : "r"(*reinterpret_cast<uint32_t*>(&h)));
  return y;
}

enum { kPlain = 0, kSum, kSumPack, kHalfPoly, kQuarterPoly, kPackedToF32, kPackedAsIs, kVariants };

template <int VARIANT>
__global__ void bench(const float* in, float* out, unsigned long long* cycles, int iters) {
  float x[128];
  const float scale = in[0], negm = in[1];
#pragma unroll
  for (int i = 0; i < 128; ++i) x[i] = in[2 + ((threadIdx.x + i) & 63)];
  float acc = 0.f;
  uint32_t keep = 0;
  __syncthreads();
  const long long t0 = clock64();
  for (int it = 0; it < iters; ++it) {
    float sum4[4] = {0, 0, 0, 0};
#pragma unroll
    for (int c = 0; c < 128; c += 2) {
      const float a = fmaf(x[c], scale, negm), b = fmaf(x[c + 1], scale, negm);
      float p0, p1;
      const bool poly = (VARIANT == kHalfPoly && ((c >> 1) & 1)) ||
                        (VARIANT == kQuarterPoly && ((c >> 1) & 3) == 3);
      if (poly) {
        p0 = ex2_poly(a);
        p1 = ex2_poly(b);
      } else if (VARIANT == kPackedToF32 || VARIANT == kPackedAsIs) {
        const uint32_t y = ex2_h2(a, b);
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&y));
        p0 = f.x;
        p1 = f.y;
        if (VARIANT == kPackedAsIs) keep ^= y;
      } else {
        p0 = ex2(a);
        p1 = ex2(b);
      }
      if (VARIANT == kPlain) sum4[(c >> 1) & 3] += p0 * p1;
      else sum4[(c >> 1) & 3] += p0 + p1;
      if (VARIANT >= kSumPack && VARIANT != kPackedAsIs) keep ^= pack_bf16(p0, p1);
    }
    acc += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]);
#pragma unroll
    for (int i = 0; i < 128; ++i) x[i] += acc * 1e-30f;  // loop-carried dependence, one FMA each
  }
  const long long t1 = clock64();
  if (threadIdx.x == 0 && blockIdx.x == 0) cycles[0] = static_cast<unsigned long long>(t1 - t0);
  out[blockIdx.x * blockDim.x + threadIdx.x] = acc + __uint_as_float(keep & 1);
}

template <int VARIANT>
void run(const char* name, const float* in, float* out, unsigned long long* cyc) {
  const int iters = 200;
  for (int warps : {4, 8}) {
    for (int rep = 0; rep < 2; ++rep) {
      bench<VARIANT><<<148, warps * 32>>>(in, out, cyc, iters);
      cudaDeviceSynchronize();
    }
    unsigned long long c = 0;
    cudaMemcpy(&c, cyc, 8, cudaMemcpyDeviceToHost);
    printf("%-44s %d warp(s) per sub-partition: %5.0f cycles per 128-element row, %5.0f per 128 x 128 tile and SM\n",
           name, warps / 4, double(c) / iters, double(c) / iters / (warps / 4));
  }
}

int main() {
  float h[66];
  h[0] = 0.18f;
  h[1] = -3.0f;
  for (int i = 0; i < 64; ++i) h[2 + i] = -0.1f * i;
  float *in, *out;
  unsigned long long* cyc;
  cudaMalloc(&in, sizeof(h));
  cudaMalloc(&out, 4 * 148 * 256);
  cudaMalloc(&cyc, 8);
  cudaMemcpy(in, h, sizeof(h), cudaMemcpyHostToDevice);
  run<kPlain>("ex2.approx.f32", in, out, cyc);
  run<kSum>("ex2.approx.f32 + row sum", in, out, cyc);
  run<kSumPack>("ex2.approx.f32 + row sum + bf16 pack", in, out, cyc);
  run<kHalfPoly>("half of them as polynomials", in, out, cyc);
  run<kQuarterPoly>("a quarter of them as polynomials", in, out, cyc);
  run<kPackedToF32>("ex2.approx.f16x2, back to fp32, bf16 pack", in, out, cyc);
  run<kPackedAsIs>("ex2.approx.f16x2 used as fp16 probabilities", in, out, cyc);
  printf("%s\n", cudaGetErrorString(cudaGetLastError()));
  return 0;
}
