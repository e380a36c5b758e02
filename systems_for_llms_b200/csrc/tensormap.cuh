// Host-side construction of TMA tensor maps.  The driver entry point
// cuTensorMapEncodeTiled is looked up once through the runtime so the library
// does not need to link against libcuda directly.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace sfl {

// Returns nullptr if the driver entry point cannot be resolved.
void* tensormap_encode_fn();

// 2-D bf16 (or any 2-byte type) tensor map with a 128-byte-swizzled box.
//   inner    : number of elements in the contiguous dimension
//   outer    : number of rows
//   ld_elems : row pitch in elements (must be a multiple of 8 -> 16 bytes)
//   box_inner must be 64 elements (128 bytes), box_outer <= 256.
// Returns 0 on success, a CUresult-style code otherwise.
int make_tensormap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                           uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer);

// 2-D map with a 128-byte-swizzled box for 2-byte (bf16/fp16) or 4-byte (fp32)
// elements; box_inner * elem_bytes must be 128.  Maps of 4-byte elements are
// typed fp32, which is what a TMA reduce-add on them accumulates in.
int make_tensormap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner,
                      uint64_t outer, uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer);

// General tiled map of rank <= 5; elem_bytes is 2 or 4.
int make_tensormap_nd(CUtensorMap* out, const void* base, int elem_bytes, int rank,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      int swizzle);

// General tiled map of rank <= 5 for 2-byte elements.  dims/strides are given
// innermost first; strides[0] is implied (contiguous) and strides_bytes[i] is the
// byte pitch of dimension i (i >= 1).  swizzle: 0 none, 1 32B, 2 64B, 3 128B.
int make_tensormap_nd_b16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box, int swizzle);

}  // namespace sfl
