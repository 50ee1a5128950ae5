// TEST INFRASTRUCTURE ONLY.  A launcher for the reference's gemv_quantized_int4
// (backend/cuda/hk/fastgemv.cuh:394-495), which the reference defines but never launches
// (hk/fastgemv.cu has wrappers for fp16 and int8 only).  The kernel itself is the reference's,
// included from its checkout at build time and wrapped in a namespace so that its other
// kernels do not collide with the copies in hk/fastgemv.cu's object file.  The launch shape is
// the one of the reference's int8 launcher (hk/fastgemv.cu:39-59): 128 x 4 threads, one block
// row per four weight rows, num_per_thread = K / 128.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <curand_kernel.h>
#include <driver_functions.h>
#include <stdio.h>

#include <cstdint>

namespace fastgate_ref_int4 {
#include "hk/fastgemv.cuh"
}

// W4 [N, K/2] bytes (device), x [K] fp16 (device), y [N] fp16 (device); returns the CUDA error code.
extern "C" int fastgate_ref_gemv_int4(const void* W4, const void* x, void* y, int N, int K, float scale,
                                      float zero_point, void* stream) {
  using namespace fastgate_ref_int4;
  dim3 grid(1, N / 4), block(128, 4);
  gemv_quantized_int4<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(
      reinterpret_cast<uint4_2*>(const_cast<void*>(W4)), reinterpret_cast<half*>(const_cast<void*>(x)),
      reinterpret_cast<half*>(y), static_cast<unsigned int>(K), __float2half(scale), __float2half(zero_point),
      static_cast<unsigned int>(K / 128));
  return static_cast<int>(cudaGetLastError());
}
