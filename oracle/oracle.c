/*
 * TEST INFRASTRUCTURE ONLY — CPU oracle for the small-batch matmul hot path.
 *
 * Nothing here is shipped or measured as the product: only tests/, the smoke check and
 * the CPU-baseline leg of bench.py may build, load or call this file.
 *
 * It restates, in plain C, the arithmetic of chanzhennan/Fastgate's kernels for the path
 * (file:line below are relative to that project).  Two kinds of function:
 *
 *  (1) order-exact restatements of the CUDA-core kernels, which accumulate fp16 products
 *      in fp32 in a documented per-thread order and reduce with a shuffle tree.  Every
 *      product of two fp16 values is exact in fp32 (11 + 11 significand bits), so FMA
 *      contraction cannot change a result and these functions reproduce the GPU kernels
 *      bit for bit:
 *        fgo_gemv_fp16_ref      gemv_fp16              backend/cuda/hk/fastgemv.cuh:503-562
 *                               (launch 128x4 threads) backend/cuda/hk/fastgemv.cu:12-33
 *        fgo_gemv_fp16_bs2_ref  gemv_fp16_bs2          backend/cuda/czn/fastgemm.cuh:302-392
 *        fgo_gemm_fp16_ref      gemm_fp16 (extend)     backend/cuda/hk/fastgemv.cuh:244-311
 *        fgo_gemv_int8_ref      gemv_quantized_int8    backend/cuda/hk/fastgemv.cuh:316-389
 *                               (scale 1, zero-point 0 as launched, hk/fastgemv.cu:50-59)
 *        fgo_gemv_int4_ref      gemv_quantized_int4    backend/cuda/hk/fastgemv.cuh:394-495
 *                               (no launcher in the reference: the int8 one's 128x4 shape)
 *
 *  (2) the "fp32-accumulated reference" the tolerance max|d| <= 1e-2*max(1,|ref|) is
 *      stated against, for all three operand layouts; the tensor-core kernels of the
 *      reference (eed_hgemm_m8n128k64x4_v7/_v7_bt, backend/cuda/hk/edgemm.cuh:1669-1868,
 *      1467-1667) accumulate in fp16 inside wmma in a hardware-defined order that cannot
 *      be restated bit-exactly, so for them this is the oracle:
 *        fgo_gemm_nk / fgo_gemm_kn / fgo_gemm_w8a16_nk / fgo_gemm_w4a16_nk
 *                                                         (double accumulation, fp32 out)
 *        fgo_gemm_nk_f32seq                               (sequential fp32 accumulation)
 *
 *  plus fgo_ref_splitk_bt, the reference's split-K choice (backend/cuda/hk/edgemm.cu:287-305).
 *
 * Pinning: the reference's only known-answer vector (all-ones operands, every output == K,
 * script/ncu-gemv-test.py:29-47) and fixtures produced by the reference's own kernels on a
 * B200 (tests/golden/) are checked by the CPU test-suite.
 */
#include <stdint.h>
#include <stddef.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

typedef _Float16 f16;

static inline float h2f(uint16_t h) {
  f16 v;
  memcpy(&v, &h, 2);
  return (float)v;
}
static inline uint16_t f2h(float f) {
  f16 v = (f16)f; /* round to nearest even, as __float2half */
  uint16_t h;
  memcpy(&h, &v, 2);
  return h;
}

int fgo_num_threads(void) {
#ifdef _OPENMP
  return omp_get_max_threads();
#else
  return 1;
#endif
}

/* warpReduceSum(sum, threadNum) over 32 lanes, hk/fastgemv.cuh:27-40: shfl_down by
 * 16,8,4,2,1 (only the offsets with threadNum >= 2*offset); a lane whose source is out of
 * range keeps its own value as the addend.  Returns lane 0. */
static float warp_reduce_ref(float* s, unsigned thread_num) {
  for (unsigned off = 16; off >= 1; off >>= 1) {
    if (thread_num >= 2 * off) {
      float nxt[32];
      for (unsigned l = 0; l < 32; ++l) nxt[l] = s[l] + (l + off < 32 ? s[l + off] : s[l]);
      memcpy(s, nxt, sizeof(nxt));
    }
  }
  return s[0];
}

/* Block-level tail shared by gemv_fp16 / gemv_quantized_int8 / gemv_fp16_bs2:
 * 128 per-thread sums -> 4 warp sums (lane 0 of each warp) -> warp 0 reduces the 4 values
 * with warpReduceSum(.., 4) (hk/fastgemv.cuh:538-561). */
static float block_reduce_ref(const float* thread_sum /*[128]*/) {
  float ws[32];
  memset(ws, 0, sizeof(ws));
  for (int w = 0; w < 4; ++w) {
    float lanes[32];
    memcpy(lanes, thread_sum + 32 * w, sizeof(lanes));
    ws[w] = warp_reduce_ref(lanes, 128);
  }
  return warp_reduce_ref(ws, 4);
}

/* Per-thread partial sums of one weight row against one activation row, in the order of
 * hk/fastgemv.cuh:513-536: thread tid visits float4 index j = tid + 128*iter (8 halves),
 * adds the 8 products in element order. */
static void thread_sums_f16(const uint16_t* wrow, const uint16_t* xrow, int K, float* ts /*[128]*/) {
  const int n8 = K >> 3;
  const int iters = ((K / 128) + 7) / 8; /* DIV_UP(num_per_thread, 8) */
  for (int tid = 0; tid < 128; ++tid) {
    float sum = 0.f;
    for (int it = 0; it < iters; ++it) {
      const int j = tid + it * 128;
      if (j < n8)
        for (int e = 0; e < 8; ++e) sum += h2f(xrow[8 * j + e]) * h2f(wrow[8 * j + e]);
    }
    ts[tid] = sum;
  }
}

/* y[N] = W[N,K] . x[K]; fastgemv (hk/fastgemv.cu:12-33) and fastgemm with M=1
 * (czn/fastgemm.cu:34-43, kernel czn/fastgemm.cuh:77-136 is the same code). */
void fgo_gemv_fp16_ref(const uint16_t* W, const uint16_t* x, uint16_t* y, int N, int K) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    float ts[128];
    thread_sums_f16(W + (size_t)n * K, x, K, ts);
    y[n] = f2h(block_reduce_ref(ts));
  }
}

/* C[2,N]: fastgemm with M=2 (czn/fastgemm.cu:44-52): one weight vector load feeds two
 * activation rows; each row's sum follows the same order as gemv_fp16
 * (czn/fastgemm.cuh:318-349), results go to res[row] and res[row + n] (:388-389). */
void fgo_gemv_fp16_bs2_ref(const uint16_t* W, const uint16_t* x2, uint16_t* C, int N, int K) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n)
    for (int m = 0; m < 2; ++m) {
      float ts[128];
      thread_sums_f16(W + (size_t)n * K, x2 + (size_t)m * K, K, ts);
      C[(size_t)m * N + n] = f2h(block_reduce_ref(ts));
    }
}

/* C[M,N] = x[M,K] . W[N,K]^T, M <= 8: fastgemv_extend (hk/fastgemv.cu:86-111): block n,
 * threadIdx.y = m, same per-thread order (hk/fastgemv.cuh:263-285); the warp step is a
 * shfl_xor butterfly (:289-292), whose lane-0 value equals the shfl_down tree; the four
 * warp sums of a row are then added sequentially, ((w0+w1)+w2)+w3 (:301-306). */
void fgo_gemm_fp16_ref(const uint16_t* W, const uint16_t* x, uint16_t* C, int M, int N, int K) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n)
    for (int m = 0; m < M; ++m) {
      float ts[128];
      thread_sums_f16(W + (size_t)n * K, x + (size_t)m * K, K, ts);
      float sum = 0.f;
      for (int w = 0; w < 4; ++w) {
        float lanes[32];
        memcpy(lanes, ts + 32 * w, sizeof(lanes));
        const float v = warp_reduce_ref(lanes, 128);
        sum = (w == 0) ? v : sum + v;
      }
      C[(size_t)m * N + n] = f2h(sum);
    }
}

/* y[n] = scale * sum_k x[k] * (float(W8[n,k]) - zero_point): gemv_quantized_int8
 * (hk/fastgemv.cuh:316-389).  Each thread scales its own partial sum before the reduction
 * (:363).  The launcher passes scale = 1.0 and zero_point = 0.0 (hk/fastgemv.cu:50-59). */
void fgo_gemv_int8_ref(const int8_t* W8, const uint16_t* x, uint16_t* y, int N, int K, float scale,
                       float zero_point) {
  const int n8 = K >> 3;
  const int iters = ((K / 128) + 7) / 8;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    float ts[128];
    const int8_t* wrow = W8 + (size_t)n * K;
    for (int tid = 0; tid < 128; ++tid) {
      float sum = 0.f;
      for (int it = 0; it < iters; ++it) {
        const int j = tid + it * 128;
        if (j < n8)
          for (int e = 0; e < 8; ++e) sum += h2f(x[8 * j + e]) * ((float)wrow[8 * j + e] - zero_point);
      }
      ts[tid] = sum * scale;
    }
    y[n] = f2h(block_reduce_ref(ts));
  }
}

/* y[n] = sum over threads of scale * sum_k x[k] * (float(nibble[n,k]) - zero_point):
 * gemv_quantized_int4 (hk/fastgemv.cuh:394-495).  W4 is [N, K/2] bytes, low nibble = even k
 * (uint4_2, hk/utility.cuh:13-36).  Thread tid of a 128-thread row takes 16 consecutive k at
 * 16 * (tid + 128 * iter) (:409-412, two float4 of activations against two uint4_2_4), adds the
 * sixteen products in k order (:437-468), scales its own sum (:472) and the block reduces as
 * in the other GEMV kernels (:474-494).  With an integer zero point every product is exact in
 * fp32, so contraction to FMA cannot change the result.  The reference has no launcher for
 * this kernel; the shape of its int8 launcher (128 x 4 threads, num_per_thread = K / 128,
 * hk/fastgemv.cu:39-59) is assumed. */
void fgo_gemv_int4_ref(const uint8_t* W4, const uint16_t* x, uint16_t* y, int N, int K, float scale,
                       float zero_point) {
  const int n8 = K >> 3;
  const int iters = ((K / 128) + 15) / 16;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    float ts[128];
    const uint8_t* wrow = W4 + (size_t)n * (K / 2);
    for (int tid = 0; tid < 128; ++tid) {
      float sum = 0.f;
      for (int it = 0; it < iters; ++it) {
        const int j = 2 * (tid + it * 128);
        if (j < n8)
          for (int e = 0; e < 16; ++e) {
            const int k = 8 * j + e;
            const uint8_t byte = wrow[k >> 1];
            const float w = (float)((k & 1) ? (byte >> 4) & 0x0F : byte & 0x0F);
            sum += h2f(x[k]) * (w - zero_point);
          }
      }
      ts[tid] = sum * scale;
    }
    y[n] = f2h(block_reduce_ref(ts));
  }
}

/* ---- fp32-accumulated reference ("the oracle" for the tolerance) ---------------------- */

/* C32[m,n] = sum_k x[m,k]*W[n,k], double accumulation, rounded once to fp32. */
void fgo_gemm_nk(const uint16_t* x, const uint16_t* W, float* C32, int M, int N, int K) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const uint16_t* w = W + (size_t)n * K;
    for (int m = 0; m < M; ++m) {
      const uint16_t* xr = x + (size_t)m * K;
      double acc = 0.0;
      for (int k = 0; k < K; ++k) acc += (double)(h2f(xr[k]) * h2f(w[k]));
      C32[(size_t)m * N + n] = (float)acc;
    }
  }
}

/* Same contraction with a plain sequential fp32 accumulator (k = 0..K-1). */
void fgo_gemm_nk_f32seq(const uint16_t* x, const uint16_t* W, float* C32, int M, int N, int K) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const uint16_t* w = W + (size_t)n * K;
    for (int m = 0; m < M; ++m) {
      const uint16_t* xr = x + (size_t)m * K;
      float acc = 0.f;
      for (int k = 0; k < K; ++k) acc += h2f(xr[k]) * h2f(w[k]);
      C32[(size_t)m * N + n] = acc;
    }
  }
}

/* C32[m,n] = sum_k A[m,k]*B[k,n]  (edgemm_m8n128k64x4 layout, hk/edgemm.cu:102-156). */
void fgo_gemm_kn(const uint16_t* A, const uint16_t* B, float* C32, int M, int N, int K) {
#pragma omp parallel for schedule(static)
  for (int nb = 0; nb < N; nb += 64) {
    const int ne = nb + 64 < N ? nb + 64 : N;
    for (int m = 0; m < M; ++m) {
      double acc[64];
      for (int i = 0; i < 64; ++i) acc[i] = 0.0;
      for (int k = 0; k < K; ++k) {
        const float a = h2f(A[(size_t)m * K + k]);
        const uint16_t* b = B + (size_t)k * N;
        for (int n = nb; n < ne; ++n) acc[n - nb] += (double)(a * h2f(b[n]));
      }
      for (int n = nb; n < ne; ++n) C32[(size_t)m * N + n] = (float)acc[n - nb];
    }
  }
}

/* C32[m,n] = (sum_k x[m,k]*W8[n,k]) * scales[n]; scales == NULL means 1 (the reference's
 * effective behaviour).  The scale is applied once, in fp32, after the K sum. */
void fgo_gemm_w8a16_nk(const uint16_t* x, const int8_t* W8, const uint16_t* scales, float* C32, int M,
                       int N, int K) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const int8_t* w = W8 + (size_t)n * K;
    const float s = scales ? h2f(scales[n]) : 1.0f;
    for (int m = 0; m < M; ++m) {
      const uint16_t* xr = x + (size_t)m * K;
      double acc = 0.0;
      for (int k = 0; k < K; ++k) acc += (double)(h2f(xr[k]) * (float)w[k]);
      C32[(size_t)m * N + n] = (float)acc * s;
    }
  }
}

/* C32[m,n] = sum_g scales[n,g] * sum_{k in group g} x[m,k] * (nibble[n,k] - zero_point); groups
 * scales per row (1, or K/128 for one per 128 consecutive k); scales NULL = 1.  Double accumulation. */
void fgo_gemm_w4a16_nk(const uint16_t* x, const uint8_t* W4, const uint16_t* scales, int groups, int zero_point,
                       float* C32, int M, int N, int K) {
  const int seg = K / groups;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const uint8_t* w = W4 + (size_t)n * (K / 2);
    for (int m = 0; m < M; ++m) {
      const uint16_t* xr = x + (size_t)m * K;
      double total = 0.0;
      for (int g = 0; g < groups; ++g) {
        double acc = 0.0;
        for (int k = g * seg; k < (g + 1) * seg; ++k) {
          const int q = (k & 1) ? (w[k >> 1] >> 4) & 0x0F : w[k >> 1] & 0x0F;
          acc += (double)h2f(xr[k]) * (double)(q - zero_point);
        }
        total += acc * (double)(scales ? h2f(scales[(size_t)n * groups + g]) : 1.0f);
      }
      C32[(size_t)m * N + n] = (float)total;
    }
  }
}

/* fp32 -> fp16 rounding of a whole array (round to nearest even). */
void fgo_round_to_f16(const float* src, uint16_t* dst, size_t n) {
  for (size_t i = 0; i < n; ++i) dst[i] = f2h(src[i]);
}

/* Split-K factor the reference picks for edgemm_m8n128k64x4_bt (hk/edgemm.cu:282-305).
 * edgemm_m8n128k64x4 itself always uses 8 (hk/edgemm.cu:115). */
int fgo_ref_splitk_bt(int M, int N, int K) {
  const int BX = N / 128, BY = (M + 7) / 8;
  int BZ = 1;
  const int tile_num = BX * BY;
  if (tile_num <= 64) {
    BZ = 4;
    if (tile_num <= 32) BZ = 8;
  }
  if (K % 1024) {
    BZ = BZ < 4 ? BZ : 4;
    if (K % 512) {
      BZ = BZ < 2 ? BZ : 2;
      if (K % 256) BZ = BZ < 1 ? BZ : 1;
    }
  }
  return BZ;
}

/* Per-output-channel int8 quantiser (no counterpart in the reference; restated here so that the
 * CUDA quantiser can be checked bit for bit): scale[n] = fp16(max|W[n,:]| / 127), 1 for an
 * all-zero row; W8 = clamp(rint(W / float(scale)), -127, 127), ties to even. */
#include <math.h>
void fgo_quantize_rows_w8(const uint16_t* W, int8_t* W8, uint16_t* scales, int N, int K) {
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const uint16_t* w = W + (size_t)n * K;
    float amax = 0.f;
    for (int k = 0; k < K; ++k) {
      const float a = fabsf(h2f(w[k]));
      if (a > amax) amax = a;
    }
    const uint16_t sh = amax > 0.f ? f2h(amax / 127.f) : f2h(1.f);
    const float s = h2f(sh);
    scales[n] = sh;
    for (int k = 0; k < K; ++k) {
      float q = nearbyintf(h2f(w[k]) / s);
      if (q > 127.f) q = 127.f;
      if (q < -127.f) q = -127.f;
      W8[(size_t)n * K + k] = (int8_t)q;
    }
  }
}

/* Group-wise int4 quantiser (no counterpart in the reference): per segment of K/groups values
 * scale = fp16(max|w| / 7) (1 if all zero), q = clamp(rint(w / scale) + 8, 0, 15), packed two
 * per byte with the even k in the low nibble. */
void fgo_quantize_rows_w4(const uint16_t* W, uint8_t* W4, uint16_t* scales, int groups, int N, int K) {
  const int seg = K / groups;
#pragma omp parallel for schedule(static)
  for (int n = 0; n < N; ++n) {
    const uint16_t* w = W + (size_t)n * K;
    uint8_t* out = W4 + (size_t)n * (K / 2);
    for (int g = 0; g < groups; ++g) {
      float amax = 0.f;
      for (int k = g * seg; k < (g + 1) * seg; ++k) {
        const float a = fabsf(h2f(w[k]));
        if (a > amax) amax = a;
      }
      const uint16_t sh = amax > 0.f ? f2h(amax / 7.f) : f2h(1.f);
      const float s = h2f(sh);
      scales[(size_t)n * groups + g] = sh;
      for (int k = g * seg; k < (g + 1) * seg; k += 2) {
        int q[2];
        for (int e = 0; e < 2; ++e) {
          float v = nearbyintf(h2f(w[k + e]) / s) + 8.f;
          if (v > 15.f) v = 15.f;
          if (v < 0.f) v = 0.f;
          q[e] = (int)v;
        }
        out[k >> 1] = (uint8_t)(q[0] | (q[1] << 4));
      }
    }
  }
}

/* Fused epilogue of a linear layer (no counterpart in the reference, which has no fused op):
 * out = act(acc + bias[n]) + residual[m,n], in fp32; act: 0 none, 1 GELU (erf), 2 GELU (tanh), 3 SiLU. */
void fgo_epilogue(float* C32, const uint16_t* bias, const uint16_t* residual, int act, int M, int N) {
  for (int m = 0; m < M; ++m)
    for (int n = 0; n < N; ++n) {
      float v = C32[(size_t)m * N + n];
      if (bias) v += h2f(bias[n]);
      if (act == 1) v = 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
      else if (act == 2) v = 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
      else if (act == 3) v = v / (1.f + expf(-v));
      if (residual) v += h2f(residual[(size_t)m * N + n]);
      C32[(size_t)m * N + n] = v;
    }
}
