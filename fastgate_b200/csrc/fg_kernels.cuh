// Persistent stream-K skinny-GEMM kernel for sm_100a.
//
//   C[m, n] = sum_k x[m, k] * Wt[n, k]        m < M <= 16,  N % 128 == 0
//
// The weight is the only large operand; it is read from HBM exactly once, by TMA
// (cp.async.bulk.tensor, no cluster multicast) into a ring of 128B-swizzled
// shared-memory stages guarded by full/empty mbarriers.  One warp produces, the
// other warps consume whole stages in round-robin order (K is split across the
// warps), each keeping the full 128 x MT fp32 accumulator tile in registers.  The
// product is formed "swap-AB": weight rows are the 16-row A operand of
// mma.sync.m16n8k16 and the few token rows are its 8-column B operand, so a tile of
// 128 output columns needs 8 (MT=8) or 16 (MT=16) tensor-core ops per 16 k.
//
// Work list: tiles (N/128) x k_blocks stages, dealt to the CTAs in equal contiguous
// ranges.  A CTA that owns a whole tile writes C directly; otherwise it stores its
// fp32 partial tile to the workspace and takes a ticket; the last CTA to arrive sums
// the partials in CTA order (deterministic) and writes C.  Nobody waits on another
// CTA, and every mbarrier wait is bounded in time.
//
// Replaces eed_hgemm_m8n128k64x4_v7 / _v7_bt (backend/cuda/hk/edgemm.cuh:1669-1868,
// 1467-1667), gemv_fp16 / gemm_fp16 / gemv_quantized_int8
// (backend/cuda/hk/fastgemv.cuh:503-562, 244-311, 316-389) and gemv_fp16_bs2
// (backend/cuda/czn/fastgemm.cuh:302-392) of the reference.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "fg_ptx.cuh"

namespace fg {

constexpr int kTileN = 128;           // output columns per tile
constexpr int kRedStride = 132;       // floats per row of the cross-warp reduction buffer
constexpr int kChunkWBytes = 16384;   // weight bytes per chunk (128 columns x 128 B, or 64 k x 256 B)
constexpr int kMaxConsumerWarps = 8;
constexpr unsigned long long kWaitBudgetNs = 2000000000ull;  // 2 s per wait, then give up

enum { kOpF16KN = 0, kOpF16NK = 1, kOpW8A16NK = 2 };
enum { kStatusOk = 0, kStatusTimeout = 6 };

template <int OP>
struct OpTraits;
template <>
struct OpTraits<kOpF16NK> {
  static constexpr int chunkK = 64;       // k covered by one 16 KB weight chunk
  static constexpr int xBoxes = 1;        // 64-k activation boxes per chunk
};
template <>
struct OpTraits<kOpF16KN> {
  static constexpr int chunkK = 64;
  static constexpr int xBoxes = 1;
};
template <>
struct OpTraits<kOpW8A16NK> {
  static constexpr int chunkK = 128;
  static constexpr int xBoxes = 2;
};

struct KParams {
  __half* C;                 // [M, N]
  const __half* scales;      // [N] or nullptr (int8 op only)
  float* partials;           // [grid][2][MT * 128]
  unsigned int* tickets;     // [tiles], zero between launches
  int* status;               // device status word
  int M, N, K;
  int tiles;                 // N / 128
  int k_blocks;              // stages per tile
  int chunks_per_stage;
  int stages;
  int consumer_warps;
};

__host__ __device__ constexpr int chunk_bytes(int op, int mt) {
  return kChunkWBytes + (op == kOpW8A16NK ? 2 : 1) * mt * 128;
}

// ---- one 16 KB weight chunk against its activation tile ------------------------------
// All shared-memory tiles have 128-byte rows with the TMA 128B swizzle: the 16-byte
// piece c of row r sits at piece (c ^ (r & 7)).

template <int MT>
__device__ __forceinline__ void load_b_frags_f16(uint32_t xbase, int kk2, int q, int r,
                                                 uint32_t (&b)[2][MT / 8][2]) {
  // b[e][j] = fragments for k16 step (2*kk2 + e), token group j.
  if constexpr (MT == 16) {
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int kk = kk2 * 2 + e;
      const uint32_t addr = xbase + ((q >> 1) * 8 + r) * 128 + ((((kk * 2) + (q & 1)) ^ r) << 4);
      ldsm_x4(addr, b[e][0][0], b[e][0][1], b[e][1][0], b[e][1][1]);
    }
  } else {
    const uint32_t addr = xbase + r * 128 + (((kk2 * 4 + q) ^ r) << 4);
    ldsm_x4(addr, b[0][0][0], b[0][0][1], b[1][0][0], b[1][0][1]);
  }
}

template <int OP, int MT>
__device__ __forceinline__ void consume_chunk(uint32_t wbase, uint32_t xbase, int lane,
                                              float (&acc)[8][MT / 8][4]) {
  const int q = lane >> 3, r = lane & 7;
  if constexpr (OP == kOpF16NK || OP == kOpF16KN) {
#pragma unroll
    for (int kk2 = 0; kk2 < 2; ++kk2) {
      uint32_t b[2][MT / 8][2];
      load_b_frags_f16<MT>(xbase, kk2, q, r, b);
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int kk = kk2 * 2 + e;
#pragma unroll
        for (int rg = 0; rg < 8; ++rg) {
          uint32_t a0, a1, a2, a3;
          if constexpr (OP == kOpF16NK) {
            // weight chunk [128 n][64 k]: rows are output columns
            const uint32_t addr = wbase + (rg * 16 + (q & 1) * 8 + r) * 128 +
                                  ((((kk * 2) + (q >> 1)) ^ r) << 4);
            ldsm_x4(addr, a0, a1, a2, a3);
          } else {
            // weight chunk = two boxes [64 k][64 n]: rows are k, transpose on load
            const int krow = kk * 16 + (q >> 1) * 8 + r;
            const uint32_t addr = wbase + (rg >> 2) * 8192 + krow * 128 +
                                  (((((rg & 3) * 2) + (q & 1)) ^ r) << 4);
            ldsm_x4_trans(addr, a0, a1, a2, a3);
          }
#pragma unroll
          for (int j = 0; j < MT / 8; ++j) mma_16816(acc[rg][j], a0, a1, a2, a3, b[e][j][0], b[e][j][1]);
        }
      }
    }
  } else {
    // int8 weight chunk [128 n][128 k].  Within a k16 step the thread with t = lane % 4
    // owns bytes 4t..4t+3 of its rows; they are fed as MMA columns (2t, 2t+1, 2t+8, 2t+9),
    // and the activation fragment is read with the same permutation (8 contiguous bytes).
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int cp = 0; cp < 4; ++cp) {
      uint32_t b[2][MT / 8][2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int s = cp * 2 + e;
#pragma unroll
        for (int j = 0; j < MT / 8; ++j) {
          const int m = j * 8 + g;
          const uint32_t addr = xbase + (s >> 2) * (MT * 128) + m * 128 +
                                (((((s & 3) * 2) + (t >> 1)) ^ (m & 7)) << 4) + (t & 1) * 8;
          lds_v2(addr, b[e][j][0], b[e][j][1]);
        }
      }
#pragma unroll
      for (int rg = 0; rg < 8; ++rg) {
        uint32_t w0, w1, w2, w3;
        const uint32_t addr =
            wbase + (rg * 16 + (q & 1) * 8 + r) * 128 + ((((cp * 2) + (q >> 1)) ^ r) << 4);
        ldsm_x4(addr, w0, w1, w2, w3);
        uint32_t lo0, hi0, lo1, hi1;
        dequant_s8x4(w0, lo0, hi0);
        dequant_s8x4(w1, lo1, hi1);
#pragma unroll
        for (int j = 0; j < MT / 8; ++j) mma_16816(acc[rg][j], lo0, lo1, hi0, hi1, b[0][j][0], b[0][j][1]);
        dequant_s8x4(w2, lo0, hi0);
        dequant_s8x4(w3, lo1, hi1);
#pragma unroll
        for (int j = 0; j < MT / 8; ++j) mma_16816(acc[rg][j], lo0, lo1, hi0, hi1, b[1][j][0], b[1][j][1]);
      }
    }
  }
}

// First unit of CTA c when `total` units are dealt to `grid` CTAs.
__device__ __forceinline__ long long range_begin(long long c, long long total, long long grid) {
  return (c * total) / grid;
}
__device__ __forceinline__ int cta_of_unit(long long u, long long total, long long grid) {
  long long c = (u * grid) / total;
  while (c + 1 < grid && range_begin(c + 1, total, grid) <= u) ++c;
  while (c > 0 && range_begin(c, total, grid) > u) --c;
  return static_cast<int>(c);
}

template <int OP, int MT>
__global__ void __launch_bounds__((kMaxConsumerWarps + 1) * 32, 1)
    fg_streamk_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                      const KParams p) {
  using T = OpTraits<OP>;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;  // swizzled tiles need 1 KB alignment
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const int ncw = p.consumer_warps;
  const int S = p.stages;
  const int cps = p.chunks_per_stage;
  constexpr int cbytes = chunk_bytes(OP, MT);
  const uint32_t stage_bytes = cps * cbytes;
  const uint32_t ring_bytes = S * stage_bytes;
  float* red = reinterpret_cast<float*>(smem_gen + ring_bytes);
  const uint32_t red_bytes = ncw * MT * kRedStride * 4;
  const uint32_t bar_base = smem_base + ring_bytes + red_bytes;  // full[S] then empty[S]
  volatile int* flags = reinterpret_cast<volatile int*>(smem_gen + ring_bytes + red_bytes + 16 * S);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_base + 8 * s, 1);        // full: one arrive (the producer's expect_tx)
      mbar_init(bar_base + 8 * (S + s), 1);  // empty: one arrive (the consuming warp's lane 0)
    }
    flags[0] = 0;
    fence_mbar_init();
    fence_proxy_async();
  }
  __syncthreads();

  const long long total = static_cast<long long>(p.tiles) * p.k_blocks;
  const long long G = gridDim.x;
  const long long ub = range_begin(blockIdx.x, total, G);
  const long long ue = range_begin(blockIdx.x + 1, total, G);
  const int KB = p.k_blocks;
  const int k_per_stage = cps * T::chunkK;

  if (warp == ncw) {
    // ------------------------------ producer warp ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmW);
      tma_prefetch_desc(&tmX);
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_x = policy_evict_last();
      int tile = static_cast<int>(ub / KB);
      int kb = static_cast<int>(ub % KB);
      const int n_it = static_cast<int>(ue - ub);
      bool dead = false;
      int issued = 0;
      for (int it = 0; it < n_it; ++it) {
        const int s = it % S;
        const uint32_t use = it / S;
        if (!mbar_wait_bounded(bar_base + 8 * (S + s), (use & 1) ^ 1, kWaitBudgetNs)) {
          dead = true;
          break;
        }
        const int k0 = kb * k_per_stage;
        int nch = (p.K - k0 + T::chunkK - 1) / T::chunkK;
        nch = nch < cps ? nch : cps;
        const uint32_t full = bar_base + 8 * s;
        mbar_arrive_expect_tx(full, nch * cbytes);
        uint32_t dst = smem_base + s * stage_bytes;
        for (int c = 0; c < nch; ++c) {
          const int kc = k0 + c * T::chunkK;
          if constexpr (OP == kOpF16KN) {
            tma_load_2d(dst, &tmW, full, tile * kTileN, kc, pol_w);
            tma_load_2d(dst + 8192, &tmW, full, tile * kTileN + 64, kc, pol_w);
          } else {
            tma_load_2d(dst, &tmW, full, kc, tile * kTileN, pol_w);
          }
#pragma unroll
          for (int xb = 0; xb < T::xBoxes; ++xb)
            tma_load_2d(dst + kChunkWBytes + xb * MT * 128, &tmX, full, kc + xb * 64, 0, pol_x);
          dst += cbytes;
        }
        ++issued;
        if (++kb == KB) {
          kb = 0;
          ++tile;
        }
      }
      if (dead) {
        atomicExch(p.status, kStatusTimeout);
        // let copies already in flight land before the CTA's shared memory goes away
        const int back = issued < S ? issued : S;
        for (int i = issued - back; i < issued; ++i)
          mbar_wait_bounded(bar_base + 8 * (i % S), (i / S) & 1, kWaitBudgetNs);
      }
    }
    return;
  }

  // -------------------------------- consumer warps --------------------------------
  const int ctid = threadIdx.x;  // consumers are warps 0..ncw-1
  const int nct = ncw * 32;
  const int g = lane >> 2, t = lane & 3;
  bool dead = false;
  long long u = ub;
  int it0 = 0;  // CTA-local index of the first stage of the current segment
  float acc[8][MT / 8][4];

  while (u < ue) {
    const int tile = static_cast<int>(u / KB);
    const int kb0 = static_cast<int>(u % KB);
    const long long rest = ue - u;
    const int len = (KB - kb0) < rest ? (KB - kb0) : static_cast<int>(rest);

#pragma unroll
    for (int rg = 0; rg < 8; ++rg)
#pragma unroll
      for (int j = 0; j < MT / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[rg][j][i] = 0.f;

    // stages of this segment that belong to this warp: CTA-local index == warp (mod ncw)
    int first = it0 + ((warp - it0 % ncw) + ncw) % ncw;
    for (int it = first; it < it0 + len && !dead; it += ncw) {
      const int s = it % S;
      const uint32_t use = it / S;
      bool ok = mbar_wait_bounded(bar_base + 8 * s, use & 1, kWaitBudgetNs);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        dead = true;
        if (lane == 0) atomicExch(p.status, kStatusTimeout);
        break;
      }
      const int k0 = (kb0 + (it - it0)) * k_per_stage;
      int nch = (p.K - k0 + T::chunkK - 1) / T::chunkK;
      nch = nch < cps ? nch : cps;
      uint32_t base = smem_base + s * stage_bytes;
      for (int c = 0; c < nch; ++c) {
        consume_chunk<OP, MT>(base, base + kChunkWBytes, lane, acc);
        base += cbytes;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_base + 8 * (S + s));
    }

    // ---- cross-warp reduction of the K split (fixed order: warp 0, 1, ...) ----
    float* myred = red + warp * (MT * kRedStride);
#pragma unroll
    for (int rg = 0; rg < 8; ++rg)
#pragma unroll
      for (int j = 0; j < MT / 8; ++j) {
        const int n = rg * 16 + g, m = j * 8 + 2 * t;
        myred[m * kRedStride + n] = acc[rg][j][0];
        myred[(m + 1) * kRedStride + n] = acc[rg][j][1];
        myred[m * kRedStride + n + 8] = acc[rg][j][2];
        myred[(m + 1) * kRedStride + n + 8] = acc[rg][j][3];
      }
    named_bar_sync(1, nct);

    const bool whole = (len == KB);
    const int slot = (u == ub) ? 0 : 1;
    float* mypart = p.partials + (static_cast<size_t>(blockIdx.x) * 2 + slot) * (MT * kTileN);
    for (int e = ctid; e < MT * 64; e += nct) {
      const int m = e >> 6, n2 = (e & 63) * 2;
      float2 v = make_float2(0.f, 0.f);
      for (int w = 0; w < ncw; ++w) {
        const float2 a = *reinterpret_cast<const float2*>(red + w * (MT * kRedStride) + m * kRedStride + n2);
        v.x += a.x;
        v.y += a.y;
      }
      if (whole) {
        if (m < p.M) {
          const int n = tile * kTileN + n2;
          if (OP == kOpW8A16NK && p.scales != nullptr) {
            const float2 sc = __half22float2(*reinterpret_cast<const __half2*>(p.scales + n));
            v.x *= sc.x;
            v.y *= sc.y;
          }
          *reinterpret_cast<__half2*>(p.C + static_cast<size_t>(m) * p.N + n) = __floats2half2_rn(v.x, v.y);
        }
      } else {
        *reinterpret_cast<float2*>(mypart + 2 * e) = v;
      }
    }

    if (!whole) {
      // ---- split tile: publish the partial, the last CTA to arrive finishes the tile ----
      __threadfence();
      named_bar_sync(1, nct);
      const long long tb = static_cast<long long>(tile) * KB;
      const int c_first = cta_of_unit(tb, total, G);
      const int c_last = cta_of_unit(tb + KB - 1, total, G);
      if (ctid == 0) {
        const unsigned int prev = atomicAdd(p.tickets + tile, 1u);
        flags[0] = (prev == static_cast<unsigned int>(c_last - c_first)) ? 1 : 0;
      }
      named_bar_sync(1, nct);
      if (flags[0]) {
        __threadfence();
        for (int e = ctid; e < MT * 64; e += nct) {
          const int m = e >> 6, n2 = (e & 63) * 2;
          if (m >= p.M) continue;
          float2 v = make_float2(0.f, 0.f);
          for (int c = c_first; c <= c_last; ++c) {
            const int cslot = (static_cast<int>(range_begin(c, total, G) / KB) == tile) ? 0 : 1;
            const float2 a = __ldcg(reinterpret_cast<const float2*>(
                p.partials + (static_cast<size_t>(c) * 2 + cslot) * (MT * kTileN) + 2 * e));
            v.x += a.x;
            v.y += a.y;
          }
          const int n = tile * kTileN + n2;
          if (OP == kOpW8A16NK && p.scales != nullptr) {
            const float2 sc = __half22float2(*reinterpret_cast<const __half2*>(p.scales + n));
            v.x *= sc.x;
            v.y *= sc.y;
          }
          *reinterpret_cast<__half2*>(p.C + static_cast<size_t>(m) * p.N + n) = __floats2half2_rn(v.x, v.y);
        }
        if (ctid == 0) p.tickets[tile] = 0;  // ready for the next launch
      }
    }
    named_bar_sync(1, nct);  // `red` and flags[0] are free again

    u += len;
    it0 += len;
  }
}

}  // namespace fg
