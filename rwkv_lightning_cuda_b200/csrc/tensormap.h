// The driver's tensor-map encoder, looked up through the runtime (no link-time dependency on libcuda).
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

namespace rk {

using TensorMapEncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                       const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                       CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// nullptr when this driver does not export cuTensorMapEncodeTiled.
inline TensorMapEncodeFn tensor_map_encode_fn() {
  static TensorMapEncodeFn fn = [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      return static_cast<TensorMapEncodeFn>(nullptr);
    return reinterpret_cast<TensorMapEncodeFn>(sym);
  }();
  return fn;
}

}  // namespace rk
