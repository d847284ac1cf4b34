// Tensor-core (tcgen05 / TMEM) GEMM for row counts above the weight-streaming GEMV range.
#include "common.cuh"
#include "kernels.h"

namespace rk {

bool gemm_tc_supported(const LinearArgs&) { return false; }

int gemm_tc(cudaStream_t, const LinearArgs&) {
  set_error("gemm_tc: not available for this shape");
  return kShape;
}

}  // namespace rk
