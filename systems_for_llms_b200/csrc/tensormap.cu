#include "tensormap.cuh"

#include <mutex>

namespace sfl {

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                              const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                              const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                              CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

void* tensormap_encode_fn() {
  static void* fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    cudaDriverEntryPointQueryResult query;
    void* ptr = nullptr;
    cudaError_t err =
        cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &query);
    if (err == cudaSuccess && query == cudaDriverEntryPointSuccess) fn = ptr;
  });
  return fn;
}

int make_tensormap_nd(CUtensorMap* out, const void* base, int elem_bytes, int rank,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      int swizzle) {
  if (elem_bytes != 2 && elem_bytes != 4) return -2;
  const CUtensorMapDataType dtype =
      elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  auto encode = reinterpret_cast<EncodeFn>(tensormap_encode_fn());
  if (encode == nullptr) return -1;
  cuuint64_t gdim[5];
  cuuint64_t gstride[4];
  cuuint32_t bdim[5];
  cuuint32_t estride[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
    estride[i] = 1;
    if (i >= 1) gstride[i - 1] = strides_bytes[i];
  }
  CUtensorMapSwizzle sw = CU_TENSOR_MAP_SWIZZLE_NONE;
  if (swizzle == 1) sw = CU_TENSOR_MAP_SWIZZLE_32B;
  if (swizzle == 2) sw = CU_TENSOR_MAP_SWIZZLE_64B;
  if (swizzle == 3) sw = CU_TENSOR_MAP_SWIZZLE_128B;
  auto call = [&] {
    return encode(out, dtype, static_cast<cuuint32_t>(rank),
                  const_cast<void*>(base), gdim, gstride, bdim, estride,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, sw, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  };
  CUresult r = call();
  if (r == CUDA_ERROR_INVALID_CONTEXT || r == CUDA_ERROR_NOT_INITIALIZED) {
    // The encoder is a driver entry point and needs a context current on the
    // calling thread.  A thread that has made no runtime call yet (an autograd
    // worker running one of these ops as its first CUDA work) has none: a
    // runtime call binds the device's primary context, then encode again.
    cudaFree(nullptr);
    r = call();
  }
  return static_cast<int>(r);
}

int make_tensormap_nd_b16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box, int swizzle) {
  return make_tensormap_nd(out, base, 2, rank, dims, strides_bytes, box, swizzle);
}

int make_tensormap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner,
                      uint64_t outer, uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer) {
  uint64_t dims[2] = {inner, outer};
  uint64_t strides[2] = {0, ld_elems * static_cast<uint64_t>(elem_bytes)};
  uint32_t box[2] = {box_inner, box_outer};
  return make_tensormap_nd(out, base, elem_bytes, 2, dims, strides, box, 3);
}

int make_tensormap_2d_bf16(CUtensorMap* out, const void* base, uint64_t inner, uint64_t outer,
                           uint64_t ld_elems, uint32_t box_inner, uint32_t box_outer) {
  uint64_t dims[2] = {inner, outer};
  uint64_t strides[2] = {0, ld_elems * 2};
  uint32_t box[2] = {box_inner, box_outer};
  return make_tensormap_nd_b16(out, base, 2, dims, strides, box, 3);
}

}  // namespace sfl
