// TEST INFRASTRUCTURE ONLY.  pybind module over the UNMODIFIED host launchers of the
// reference (chanzhennan/Fastgate), compiled from the reference checkout where it lies by
// build_ref.py.  The reference's own backend/pybind.cpp binds only hgemm, fastgemm and mma
// (:22-27) and its setup.py cannot build the CUDA backend, so this file binds every
// hot-path prototype its headers declare.  No reference source is copied: the headers are
// found through -I at build time.
#include <torch/extension.h>

#include "hk/edgemm.h"      // backend/cuda/hk/edgemm.h:4-14
#include "hk/edgemm_tr.h"   // backend/cuda/hk/edgemm_tr.h:7-11
#include "hk/flatgemm.h"    // backend/cuda/hk/flatgemm.h:4-10
#include "hk/fastgemv.h"    // backend/cuda/hk/fastgemv.h:4-7
#include "czn/fastgemm.h"   // backend/cuda/czn/fastgemm.h:4

// launcher of ref_int4_launch.cu around the reference's gemv_quantized_int4 (hk/fastgemv.cuh:394-495)
extern "C" int fastgate_ref_gemv_int4(const void* W4, const void* x, void* y, int N, int K, float scale,
                                      float zero_point, void* stream);
static void gemv_int4(at::Tensor W4, at::Tensor x, at::Tensor y, double scale, double zero_point) {
  const int N = static_cast<int>(W4.size(0)), K = static_cast<int>(W4.size(1)) * 2;
  TORCH_CHECK(W4.is_cuda() && x.is_cuda() && y.is_cuda() && N % 4 == 0 && K % 128 == 0 && x.numel() == K && y.numel() == N);
  const int err = fastgate_ref_gemv_int4(W4.data_ptr(), x.data_ptr(), y.data_ptr(), N, K, static_cast<float>(scale),
                                         static_cast<float>(zero_point), nullptr);
  TORCH_CHECK(err == 0, "gemv_quantized_int4 launch failed: ", err);
}

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.def("gemv_int4", &gemv_int4);
  m.def("edgemm", &edgemm);
  m.def("edgemm_m8n256k64", &edgemm_m8n256k64);
  m.def("edgemm_m8n128k64", &edgemm_m8n128k64);
  m.def("edgemm_m8n128k128", &edgemm_m8n128k128);
  m.def("edgemv_m1n128k64x4", &edgemv_m1n128k64x4);
  m.def("edgemm_m8n128k64x4", &edgemm_m8n128k64x4);
  m.def("edgemm_m8n128k64x4_bt", &edgemm_m8n128k64x4_bt);
  m.def("edgemv_m1n256k64x4", &edgemv_m1n256k64x4);
  m.def("edgemm_m8n128k64x4_amd", &edgemm_m8n128k64x4_amd);
  m.def("edgemm_m8n256k32x8", &edgemm_m8n256k32x8);
  m.def("edgemm_m8n128k64x4_tr_amd", &edgemm_m8n128k64x4_tr_amd);
  m.def("gemm_m8n128k64x4_bt", &gemm_m8n128k64x4_bt);
  m.def("gemm_m8n32k128x8_bt", &gemm_m8n32k128x8_bt);
  m.def("gemm_m8n32k256x8_bt", &gemm_m8n32k256x8_bt);
  m.def("gemm_m8n32k256x8_bt_bz2", &gemm_m8n32k256x8_bt_bz2);
  m.def("gemm_m8n64k128x8_bt_exp", &gemm_m8n64k128x8_bt_exp);
  m.def("flat_gemm_m8n128k64x4_bz1", &flat_gemm_m8n128k64x4_bz1);
  m.def("flat_gemm_m8n256k32x8_bz1", &flat_gemm_m8n256k32x8_bz1);
  m.def("flat_gemm_m8n256k64x8", &flat_gemm_m8n256k64x8);
  m.def("flat_gemm_m8n256k32x16", &flat_gemm_m8n256k32x16);
  m.def("flat_gemm_m8n512k32x16", &flat_gemm_m8n512k32x16);
  m.def("flat_gemm_m8n64k128x8", &flat_gemm_m8n64k128x8);
  m.def("flat_gemm_m8n32k256x8", &flat_gemm_m8n32k256x8);
  m.def("fastgemv", &fastgemv);
  m.def("fastgemv_int8", &fastgemv_int8);
  m.def("fastgemv_tuned", &fastgemv_tuned);
  m.def("fastgemv_extend", &fastgemv_extend);
  m.def("fastgemm", &fastgemm);
}
