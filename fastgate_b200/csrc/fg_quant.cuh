// Per-output-channel int8 quantiser: the producer of the (W8, scales) pair that
// fastgemv_int8 / fg_gemm_w8a16_nk consume.  The reference has no quantiser (its int8 GEMV is
// fed hand-made int8 data, script/fastgemv-int8.py:5-11); the container types it sketches for
// quantised weights are in backend/cuda/hk/utility.cuh:13-46.
//
//   scale[n] = fp16( max_k |W[n,k]| / 127 )        (1 if the row is all zero)
//   W8[n,k]  = clamp( rint( W[n,k] / float(scale[n]) ), -127, 127 )
//
// Dividing by the rounded fp16 scale (not the exact one) makes W8 * scale the closest
// representable reconstruction for the scale that is actually stored.  One CTA per weight
// row; the row is read twice (the second time from L2) and written once: HBM-bound.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace fg {

constexpr int kQuantThreads = 256;

__global__ void __launch_bounds__(kQuantThreads) fg_quantize_rows_kernel(const __half* __restrict__ W,
                                                                         int8_t* __restrict__ W8,
                                                                         __half* __restrict__ scales, int K) {
  const size_t row = blockIdx.x;
  const uint4* src = reinterpret_cast<const uint4*>(W + row * K);  // 8 halves per vector
  const int nvec = K >> 3;
  // pass 1: row maximum of |w|; for non-negative halves the bit pattern orders like the value
  uint32_t amax_bits = 0;
  for (int v = threadIdx.x; v < nvec; v += kQuantThreads) {
    const uint4 q = __ldg(src + v);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t lo = w[i] & 0x7fffu, hi = (w[i] >> 16) & 0x7fffu;
      amax_bits = max(amax_bits, max(lo, hi));
    }
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, off));
  __shared__ uint32_t warp_max[kQuantThreads / 32];
  if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = amax_bits;
  __syncthreads();
  amax_bits = 0;
#pragma unroll
  for (int i = 0; i < kQuantThreads / 32; ++i) amax_bits = max(amax_bits, warp_max[i]);
  const float amax = __half2float(__ushort_as_half(static_cast<unsigned short>(amax_bits)));
  const __half scale_h = (amax > 0.f) ? __float2half_rn(__fdiv_rn(amax, 127.f)) : __float2half_rn(1.f);
  const float scale = __half2float(scale_h);
  if (threadIdx.x == 0) scales[row] = scale_h;
  // pass 2: quantise (round to nearest even), 8 int8 per 8-byte store
  uint2* dst = reinterpret_cast<uint2*>(W8 + row * K);
  for (int v = threadIdx.x; v < nvec; v += kQuantThreads) {
    const uint4 q = __ldg(src + v);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    uint32_t out[2] = {0, 0};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 h2 = *reinterpret_cast<const __half2*>(&w[i]);
      int a = __float2int_rn(__fdiv_rn(__low2float(h2), scale));
      int b = __float2int_rn(__fdiv_rn(__high2float(h2), scale));
      a = min(127, max(-127, a));
      b = min(127, max(-127, b));
      out[i >> 1] |= (static_cast<uint32_t>(a & 0xff) | (static_cast<uint32_t>(b & 0xff) << 8)) << ((i & 1) * 16);
    }
    dst[v] = make_uint2(out[0], out[1]);
  }
}

// ---- int4 -------------------------------------------------------------------------------------
// Producer of the (W4, scales) pair of fg_gemm_w4a16_nk: unsigned 4-bit values with zero point 8,
// two per byte (low nibble = even k, the packing of uint4_2 in backend/cuda/hk/utility.cuh:13-36),
// one fp16 scale per `seg` consecutive k of a row (seg = 128: group-wise; seg = K: per channel):
//
//   scale = fp16( max |w| / 7 )                  (1 if the segment is all zero)
//   q     = clamp( rint( w / float(scale) ) + 8, 0, 15 )
//
// One warp per segment: each lane strides over the segment in 8-element vectors.
__global__ void __launch_bounds__(kQuantThreads) fg_quantize_rows_w4_kernel(const __half* __restrict__ W,
                                                                            uint8_t* __restrict__ W4,
                                                                            __half* __restrict__ scales, int K,
                                                                            int seg, long long segments) {
  const long long sidx = static_cast<long long>(blockIdx.x) * (kQuantThreads / 32) + (threadIdx.x >> 5);
  if (sidx >= segments) return;
  const int lane = threadIdx.x & 31;
  const int per_row = K / seg;
  const long long row = sidx / per_row;
  const int k0 = static_cast<int>(sidx - row * per_row) * seg;
  const uint4* src = reinterpret_cast<const uint4*>(W + row * K + k0);
  const int nvec = seg >> 3;
  uint32_t amax_bits = 0;
  for (int v = lane; v < nvec; v += 32) {
    const uint4 q = __ldg(src + v);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) amax_bits = max(amax_bits, max(w[i] & 0x7fffu, (w[i] >> 16) & 0x7fffu));
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) amax_bits = max(amax_bits, __shfl_xor_sync(0xffffffffu, amax_bits, off));
  const float amax = __half2float(__ushort_as_half(static_cast<unsigned short>(amax_bits)));
  const __half scale_h = (amax > 0.f) ? __float2half_rn(__fdiv_rn(amax, 7.f)) : __float2half_rn(1.f);
  const float scale = __half2float(scale_h);
  if (lane == 0) scales[sidx] = scale_h;
  uint32_t* dst = reinterpret_cast<uint32_t*>(W4 + (row * K + k0) / 2);
  for (int v = lane; v < nvec; v += 32) {
    const uint4 q = __ldg(src + v);
    const uint32_t w[4] = {q.x, q.y, q.z, q.w};
    uint32_t out = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __half2 h2 = *reinterpret_cast<const __half2*>(&w[i]);
      int a = __float2int_rn(__fdiv_rn(__low2float(h2), scale)) + 8;
      int b = __float2int_rn(__fdiv_rn(__high2float(h2), scale)) + 8;
      a = min(15, max(0, a));
      b = min(15, max(0, b));
      out |= (static_cast<uint32_t>(a) | (static_cast<uint32_t>(b) << 4)) << (8 * i);
    }
    dst[v] = out;
  }
}

// ---- one-time weight repacking ---------------------------------------------------------------
// B[K, N] -> W[N, K] (fp16): 64 x 64 tiles through shared memory, coalesced on both sides.  For
// callers of the KxN operators that can afford a one-time repack: the NxK kernels are faster.
__global__ void __launch_bounds__(256) fg_transpose_kn_to_nk_kernel(const __half* __restrict__ B, __half* __restrict__ W,
                                                                    int N, int K) {
  __shared__ __half tile[64][66];  // two halves of padding: conflict-free column reads
  const int n0 = blockIdx.x * 64, k0 = blockIdx.y * 64;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
  for (int r = ty; r < 64; r += 8) {
    const __half2 v = *reinterpret_cast<const __half2*>(B + static_cast<size_t>(k0 + r) * N + n0 + 2 * tx);
    tile[r][2 * tx] = __low2half(v);
    tile[r][2 * tx + 1] = __high2half(v);
  }
  __syncthreads();
  for (int r = ty; r < 64; r += 8)
    *reinterpret_cast<__half2*>(W + static_cast<size_t>(n0 + r) * K + k0 + 2 * tx) =
        __halves2half2(tile[2 * tx][r], tile[2 * tx + 1][r]);
}

// Gate and up projection weights Wg[N, K], Wu[N, K] -> Wgu[2N, K] in which every 128 rows hold 64
// gate rows followed by the matching 64 up rows: the layout the SiLU-gate epilogue reads.
// blockIdx.y = destination block of 64 rows; even blocks come from Wg, odd ones from Wu.
__global__ void __launch_bounds__(256) fg_interleave_gate_up_kernel(const uint4* __restrict__ Wg, const uint4* __restrict__ Wu,
                                                                    uint4* __restrict__ Wgu, int chunks16) {
  const int blk = blockIdx.y;
  const uint4* src = ((blk & 1) ? Wu : Wg) + static_cast<size_t>(blk >> 1) * chunks16;
  uint4* dst = Wgu + static_cast<size_t>(blk) * chunks16;
  for (int i = blockIdx.x * 1024 + threadIdx.x; i < chunks16 && i < (blockIdx.x + 1) * 1024; i += 256) dst[i] = src[i];
}

}  // namespace fg
