// Tensor-core (tcgen05) prefill GEMM: placeholder translation unit, filled in next.
#include "turq_internal.h"

namespace turq {

size_t gemm_tc_scratch_bytes(int64_t m, int64_t k) { return (size_t)m * (size_t)k * 2 + 256; }

cudaError_t launch_gemm_tc(int, const uint8_t*, int64_t, int64_t, const void*, int, int64_t, float*, const float*,
                           uint8_t*, int, cudaStream_t, int*, int*) {
  return cudaErrorNotSupported;
}

}  // namespace turq
