// Host-side launch helper: programmatic stream serialization.
//
// A kernel launched through launch_pdl() may be scheduled while its predecessor
// in the stream is still running; it must call pdl_wait() (ptx.cuh) before it
// reads or writes global data the predecessor may touch.  What it does before
// that call - barrier set-up, tensor-memory allocation, descriptor prefetch, or
// simply getting its CTAs resident - overlaps the predecessor's tail instead of
// following it.  SFL_NO_PDL=1 turns the attribute off (ordinary launches).
#pragma once
#include <cuda_runtime.h>
#include <stdlib.h>

namespace sfl {

inline bool pdl_enabled() {
  static const bool on = [] {
    const char* v = getenv("SFL_NO_PDL");
    return !(v != nullptr && v[0] == '1');
  }();
  return on;
}

template <typename Kernel, typename... Args>
int launch_pdl(Kernel kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
               Args... args) {
  cudaLaunchConfig_t config{};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute{};
  attribute.id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute.val.programmaticStreamSerializationAllowed = 1;
  config.attrs = &attribute;
  config.numAttrs = pdl_enabled() ? 1 : 0;
  return static_cast<int>(cudaLaunchKernelEx(&config, kernel, args...));
}

}  // namespace sfl
