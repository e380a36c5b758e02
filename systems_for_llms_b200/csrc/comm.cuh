// Shared pieces of the peer-memory collectives: the table of symmetric-buffer
// pointers a kernel receives, the layout of the flag buffer, and system-scope
// loads and stores that travel over NVLink.  Used by the collective kernels and by
// GEMM kernels whose epilogue talks to peers directly.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace sfl {

constexpr int kMaxPeers = 8;

struct CommView {
  int rank, world;
  char* data[kMaxPeers];       // symmetric payload buffers
  uint32_t* flags[kMaxPeers];  // symmetric flag + scratch buffers
};

// Layout of the flag buffer (uint32 words):
//   [slot][phase][rank]   phase 0 = ready, 1 = done      (kSlots * 2 * 8 words)
//   then float partials [slot][rank][kMaxCtas]
//   then a local arrival counter per slot
constexpr int kSlots = 64;
constexpr int kMaxCtas = 148;
constexpr int kFlagWords = kSlots * 2 * kMaxPeers;
constexpr int kPartialWords = kSlots * kMaxPeers * kMaxCtas;
constexpr int kCounterWords = kSlots;
constexpr size_t kFlagBytes = sizeof(uint32_t) * (kFlagWords + kPartialWords + kCounterWords);

__device__ __forceinline__ uint32_t* flag_ptr(uint32_t* base, int slot, int phase, int rank) {
  return base + (slot * 2 + phase) * kMaxPeers + rank;
}
__device__ __forceinline__ float* partial_ptr(uint32_t* base, int slot, int rank, int cta) {
  return reinterpret_cast<float*>(base + kFlagWords) + (slot * kMaxPeers + rank) * kMaxCtas + cta;
}
__device__ __forceinline__ uint32_t* counter_ptr(uint32_t* base, int slot) {
  return base + kFlagWords + kPartialWords + slot;
}

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_peer_f4(const float* p) {
  float4 v;
  asm volatile("ld.relaxed.sys.global.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_peer_f4(float* p, float4 v) {
  asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(p), "f"(v.x),
               "f"(v.y), "f"(v.z), "f"(v.w)
               : "memory");
}
__device__ __forceinline__ uint4 ld_peer_u4(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_peer_u2(void* p, uint2 v) {
  asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(v.x), "r"(v.y)
               : "memory");
}
__device__ __forceinline__ void st_peer_u4(void* p, uint4 v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Epochs only grow; compare with wrap-around tolerance.
__device__ __forceinline__ bool reached(uint32_t seen, uint32_t epoch) {
  return static_cast<int32_t>(seen - epoch) >= 0;
}

}  // namespace sfl
