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
// Ring discipline: CTA-local stage number `it` uses ring slot it % stages and is consumed
// by warp it % consumer_warps.  stages % consumer_warps == 0 (enforced by the planner), so
// a slot always meets the same warp and that warp observes every phase of the slot's
// barriers: an mbarrier parity wait is only meaningful to a waiter that misses no phase.
//
// Replaces eed_hgemm_m8n128k64x4_v7 / _v7_bt (backend/cuda/hk/edgemm.cuh:1669-1868,
// 1467-1667), gemv_fp16 / gemm_fp16 / gemv_quantized_int8
// (backend/cuda/hk/fastgemv.cuh:503-562, 244-311, 316-389) and gemv_fp16_bs2
// (backend/cuda/czn/fastgemm.cuh:302-392) of the reference.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include <type_traits>

#include "fg_ptx.cuh"

namespace fg {

constexpr int kTileN = 128;           // output columns per tile
constexpr int kRedStride = 132;       // floats per row of the cross-warp reduction buffer
constexpr int kChunkWBytes = 16384;   // weight bytes per chunk (128 columns x 128 B, or 64 k x 256 B)
constexpr int kMaxConsumerWarps = 8;
constexpr int kMaxPeers = 8;          // ranks of one NVLink box
constexpr int kTraceSlots = 16;       // 64-bit words per CTA of the built-in tracer
constexpr unsigned long long kWaitBudgetNs = 2000000000ull;  // 2 s per wait, then give up

enum { kOpF16KN = 0, kOpF16NK = 1, kOpW8A16NK = 2, kOpW4A16NK = 3 };
enum { kStatusOk = 0, kStatusTimeout = 6, kStatusBadLaunch = 7 };
enum { kActNone = 0, kActGeluErf = 1, kActGeluTanh = 2, kActSilu = 3, kActSiluGate = 4 };

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
template <>
struct OpTraits<kOpW4A16NK> {
  static constexpr int chunkK = 256;      // 128 rows x 128 bytes of packed 4-bit weights
  static constexpr int xBoxes = 4;
};
__host__ __device__ constexpr bool op_is_quantized(int op) { return op == kOpW8A16NK || op == kOpW4A16NK; }

struct KParams {
  __half* C;                 // [M, N]
  const __half* scales;      // quantized ops: [N] per output channel, or [N, scale_groups] (int4), or nullptr
  int scale_groups;          // int4 op: scales per row; > 1: one per 128 k, applied inside the k loop
  uint32_t w4_magic;         // int4 op: half2(1024 + zero_point) twice
  float* partials;           // [grid][2][MT * 128]
  unsigned int* tickets;     // [tiles], zero between launches
  int* status;               // device status word
  unsigned long long* trace; // nullptr, or kTraceSlots words per CTA for the built-in tracer
  int M, N, K;
  int tiles;                 // N / 128
  int k_blocks;              // stages per tile
  int chunks_per_stage;
  int stages;
  int consumer_warps;
  int pdl;                   // 1: launched with programmatic stream serialization
  int l2_prefetch;           // stages beyond the first ring-full whose weights are prefetched into L2 while waiting
  // Fused epilogue, applied in fp32 before the single rounding to fp16:
  //   out = act(acc * scale + bias[n]) + residual[m, n]
  const __half* bias;        // [N] or nullptr
  const __half* residual;    // [M, N] (this call's rows and columns) or nullptr
  int act;                   // kActNone, kActGeluErf, kActGeluTanh, kActSilu, kActSiluGate
  // kActSiluGate (tcgen05 fp16 kernel, NxK weights): the weight holds, per 128 rows, 64 rows of the gate
  // projection followed by the matching 64 rows of the up projection; the output has N / 2 columns,
  //   out[m, 64 t + j] = silu(acc[128 t + j] + bias) * (acc[128 t + 64 + j] + bias) + residual[m, 64 t + j]
  // Optional split of the output columns over up to three dense tensors (a fused QKV projection):
  // columns [0, split1) go to C, [split1, split2) to C2, [split2, N) to C3, each with its own row
  // length; split1 == 0: everything goes to C.  split1 and split2 are multiples of 8.
  int split1, split2;
  __half* C2;
  __half* C3;
  // Fused all-gather ("push") of an N-sharded layer: when world > 0 the output tile is stored
  // into the full [M, ldc] output of every rank at column col0 + n, and each finished tile
  // bumps every rank's arrival counter.  Plain stores and atomics over NVLink peer mappings.
  int world;                 // 0: plain local output
  int rank;                  // this rank; it bumps counter [rank] of every rank's flag array
  int col0;                  // first column of this rank's slice in the full output
  long long ldc;             // row length of the full output
  __half* peer_C[kMaxPeers];
  unsigned long long* peer_flag[kMaxPeers];
  __half* mc_C;              // multicast mapping of all ranks' outputs (nullptr: per-peer stores)
  unsigned long long* mc_flag;  // multicast mapping of all ranks' flag arrays
  // Optional dependency on an earlier pushed layer: the activations are only read once the
  // `wait_world` per-source counters at wait_flags have reached wait_target (nullptr: none).
  const unsigned long long* wait_flags;
  int wait_world;
  unsigned long long wait_target;
  // The same two numbers kept on the device, so that a captured graph can be replayed: a pushing
  // launch adds its tile count to *target_dev (this rank's running total for the buffers it pushes
  // into), and a dependent launch reads its wait target from *wait_target_dev once the grid
  // dependency has resolved (the launch that pushed into those buffers has added its share by then).
  unsigned long long* target_dev;
  const unsigned long long* wait_target_dev;
};

__host__ __device__ constexpr int chunk_bytes(int op, int mt) {
  return kChunkWBytes + (op == kOpW4A16NK ? 4 : op == kOpW8A16NK ? 2 : 1) * mt * 128;
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

// Weight fragments of all eight 16-row groups for one k16 step (fp16 ops).
template <int OP>
__device__ __forceinline__ void load_a_frags_f16(uint32_t wbase, int kk, int q, int r,
                                                 uint32_t (&a)[8][4]) {
#pragma unroll
  for (int rg = 0; rg < 8; ++rg) {
    if constexpr (OP == kOpF16NK) {
      // weight chunk [128 n][64 k]: rows are output columns
      const uint32_t addr =
          wbase + (rg * 16 + (q & 1) * 8 + r) * 128 + ((((kk * 2) + (q >> 1)) ^ r) << 4);
      ldsm_x4(addr, a[rg][0], a[rg][1], a[rg][2], a[rg][3]);
    } else {
      // weight chunk = two boxes [64 k][64 n]: rows are k, transpose on load
      const int krow = kk * 16 + (q >> 1) * 8 + r;
      const uint32_t addr =
          wbase + (rg >> 2) * 8192 + krow * 128 + (((((rg & 3) * 2) + (q & 1)) ^ r) << 4);
      ldsm_x4_trans(addr, a[rg][0], a[rg][1], a[rg][2], a[rg][3]);
    }
  }
}

template <int OP, int MT>
__device__ __forceinline__ void consume_chunk(uint32_t wbase, uint32_t xbase, int lane,
                                              float (&acc)[8][MT / 8][4], const KParams& p, int n0, int k0) {
  const int q = lane >> 3, r = lane & 7;
  if constexpr (OP == kOpW4A16NK) {
    // Packed 4-bit weight chunk [128 n][128 B = 256 k], low nibble first.  The thread with
    // t = lane % 4 owns one 32-bit word (eight consecutive k) of its rows per 32-k piece; the
    // word dequantises into four half2 (k, k+4), (k+1, k+5), (k+2, k+6), (k+3, k+7) that feed two
    // k16 steps, and the activation fragment is built with the same permutation from one
    // 16-byte shared load.  Each 128-k half of the chunk is summed into a fresh accumulator,
    // scaled by its group's scale (group-wise scales) and added in fp32.
    const int g = lane >> 2, t = lane & 3;
    const int G = p.scale_groups;
    const bool grouped = G > 1;
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      uint32_t b[4][MT / 8][4];
#pragma unroll
      for (int pc = 0; pc < 4; ++pc)
#pragma unroll
        for (int j = 0; j < MT / 8; ++j) {
          const int c = hf * 4 + pc, m = j * 8 + g;
          const uint32_t addr = xbase + (c >> 1) * (MT * 128) + m * 128 + (((((c & 1) * 4) + t) ^ (m & 7)) << 4);
          uint32_t x0, x1, x2, x3;
          lds_v4(addr, x0, x1, x2, x3);
          b[pc][j][0] = prmt(x0, x2, 0x5410);
          b[pc][j][1] = prmt(x0, x2, 0x7632);
          b[pc][j][2] = prmt(x1, x3, 0x5410);
          b[pc][j][3] = prmt(x1, x3, 0x7632);
        }
      __half sc[8][2];
      if (grouped) {
        int gi = (k0 >> 7) + hf;
        gi = gi < G ? gi : G - 1;  // a ragged last chunk: its second half is all zero activations
#pragma unroll
        for (int rg = 0; rg < 8; ++rg) {
          const __half* srow = p.scales + static_cast<size_t>(n0 + rg * 16 + g) * G + gi;
          sc[rg][0] = __ldg(srow);
          sc[rg][1] = __ldg(srow + 8 * static_cast<size_t>(G));
        }
      }
      // Two 16-row groups at a time, and with an 8-row token tile the two k16 steps of a word in
      // accumulators of their own: four independent MMA chains in flight either way.
      constexpr int SP = (MT == 8) ? 2 : 1;
#pragma unroll
      for (int rp = 0; rp < 4; ++rp) {
        uint32_t w[2][2][4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int ci = 0; ci < 2; ++ci) {
            const int rg = rp * 2 + h, cp = hf * 2 + ci;
            const uint32_t addr = wbase + (rg * 16 + (q & 1) * 8 + r) * 128 + ((((cp * 2) + (q >> 1)) ^ r) << 4);
            ldsm_x4(addr, w[h][ci][0], w[h][ci][1], w[h][ci][2], w[h][ci][3]);
          }
        float tmp[2][SP][MT / 8][4];
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int sp = 0; sp < SP; ++sp)
#pragma unroll
            for (int j = 0; j < MT / 8; ++j)
#pragma unroll
              for (int i = 0; i < 4; ++i) tmp[h][sp][j][i] = 0.f;
#pragma unroll
        for (int ci = 0; ci < 2; ++ci)
#pragma unroll
          for (int ph = 0; ph < 2; ++ph) {
            const int pc = ci * 2 + ph;
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t lo[4], hi[4];  // rows g and g + 8 of this 16-row group
              dequant_u4x8(w[h][ci][ph * 2], p.w4_magic, lo);
              dequant_u4x8(w[h][ci][ph * 2 + 1], p.w4_magic, hi);
#pragma unroll
              for (int j = 0; j < MT / 8; ++j) {
                mma_16816(tmp[h][0][j], lo[0], hi[0], lo[1], hi[1], b[pc][j][0], b[pc][j][1]);
                mma_16816(tmp[h][SP - 1][j], lo[2], hi[2], lo[3], hi[3], b[pc][j][2], b[pc][j][3]);
              }
            }
          }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int rg = rp * 2 + h;
          const float s0 = grouped ? __half2float(sc[rg][0]) : 1.f;
          const float s1 = grouped ? __half2float(sc[rg][1]) : 1.f;
#pragma unroll
          for (int j = 0; j < MT / 8; ++j) {
            float v[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = (SP == 2) ? tmp[h][0][j][i] + tmp[h][SP - 1][j][i] : tmp[h][0][j][i];
            acc[rg][j][0] += v[0] * s0;
            acc[rg][j][1] += v[1] * s0;
            acc[rg][j][2] += v[2] * s1;
            acc[rg][j][3] += v[3] * s1;
          }
        }
      }
    }
  } else if constexpr (OP == kOpF16NK || OP == kOpF16KN) {
    // Software pipeline over the four k16 steps: the fragments of step kk+1 are in flight
    // while the tensor-core ops of step kk issue.
    uint32_t a[2][8][4];
    uint32_t b[2][MT / 8][2];
    load_a_frags_f16<OP>(wbase, 0, q, r, a[0]);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
      if ((kk & 1) == 0) load_b_frags_f16<MT>(xbase, kk >> 1, q, r, b);
      if (kk < 3) load_a_frags_f16<OP>(wbase, kk + 1, q, r, a[(kk + 1) & 1]);
#pragma unroll
      for (int rg = 0; rg < 8; ++rg)
#pragma unroll
        for (int j = 0; j < MT / 8; ++j)
          mma_16816(acc[rg][j], a[kk & 1][rg][0], a[kk & 1][rg][1], a[kk & 1][rg][2], a[kk & 1][rg][3],
                    b[kk & 1][j][0], b[kk & 1][j][1]);
    }
  } else {
    // int8 weight chunk [128 n][128 k].  Within a k16 step the thread with t = lane % 4
    // owns bytes 4t..4t+3 of its rows; they are fed as MMA columns (2t, 2t+1, 2t+8, 2t+9),
    // and the activation fragment is read with the same permutation (8 contiguous bytes).
    //
    // The chunk is summed into a fresh accumulator that is then added to the running one
    // with an ordinary fp32 add: the running sums of unscaled int8 products reach several
    // thousand, where the tensor core's own accumulate step is too coarse for outputs that
    // end near zero.
    const int g = lane >> 2, t = lane & 3;
    uint32_t b[8][MT / 8][2];
#pragma unroll
    for (int s = 0; s < 8; ++s)
#pragma unroll
      for (int j = 0; j < MT / 8; ++j) {
        const int m = j * 8 + g;
        const uint32_t addr = xbase + (s >> 2) * (MT * 128) + m * 128 +
                              (((((s & 3) * 2) + (t >> 1)) ^ (m & 7)) << 4) + (t & 1) * 8;
        lds_v2(addr, b[s][j][0], b[s][j][1]);
      }
#pragma unroll
    for (int rp = 0; rp < 4; ++rp) {  // two 16-row groups at a time: four independent chains
      uint32_t w[2][4][4];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int cp = 0; cp < 4; ++cp) {
          const int rg = rp * 2 + h;
          const uint32_t addr =
              wbase + (rg * 16 + (q & 1) * 8 + r) * 128 + ((((cp * 2) + (q >> 1)) ^ r) << 4);
          ldsm_x4(addr, w[h][cp][0], w[h][cp][1], w[h][cp][2], w[h][cp][3]);
        }
      float tmp[2][MT / 8][4];
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < MT / 8; ++j)
#pragma unroll
          for (int i = 0; i < 4; ++i) tmp[h][j][i] = 0.f;
#pragma unroll
      for (int cp = 0; cp < 4; ++cp)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          uint32_t lo0, hi0, lo1, hi1;
          dequant_s8x4(w[h][cp][0], lo0, hi0);
          dequant_s8x4(w[h][cp][1], lo1, hi1);
#pragma unroll
          for (int j = 0; j < MT / 8; ++j)
            mma_16816(tmp[h][j], lo0, lo1, hi0, hi1, b[cp * 2][j][0], b[cp * 2][j][1]);
          dequant_s8x4(w[h][cp][2], lo0, hi0);
          dequant_s8x4(w[h][cp][3], lo1, hi1);
#pragma unroll
          for (int j = 0; j < MT / 8; ++j)
            mma_16816(tmp[h][j], lo0, lo1, hi0, hi1, b[cp * 2 + 1][j][0], b[cp * 2 + 1][j][1]);
        }
#pragma unroll
      for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < MT / 8; ++j)
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[rp * 2 + h][j][i] += tmp[h][j][i];
    }
  }
}

// First unit of CTA c when `total` units are dealt to `grid` CTAs.  The host guarantees
// total * grid < 2^31, so 32-bit arithmetic is exact.
__device__ __forceinline__ uint32_t range_begin(uint32_t c, uint32_t total, uint32_t grid) {
  return (c * total) / grid;
}
__device__ __forceinline__ uint32_t cta_of_unit(uint32_t u, uint32_t total, uint32_t grid) {
  uint32_t c = (u * grid) / total;
  while (c + 1 < grid && range_begin(c + 1, total, grid) <= u) ++c;
  while (c > 0 && range_begin(c, total, grid) > u) --c;
  return c;
}

// Activation chosen at compile time, and a dispatcher that turns the runtime code into it ONCE
// around a whole loop nest: a per-element switch costs microseconds in the single-warp tails.
template <int ACT>
__device__ __forceinline__ float act_fn(float v) {
  if constexpr (ACT == kActGeluErf) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
  else if constexpr (ACT == kActGeluTanh) return 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
  else if constexpr (ACT == kActSilu) return v / (1.f + expf(-v));
  else return v;
}
template <typename F>
__device__ __forceinline__ void with_act(int act, F&& f) {
  switch (act) {
    case kActGeluErf: f(std::integral_constant<int, kActGeluErf>{}); break;
    case kActGeluTanh: f(std::integral_constant<int, kActGeluTanh>{}); break;
    case kActSilu: f(std::integral_constant<int, kActSilu>{}); break;
    default: f(std::integral_constant<int, kActNone>{}); break;
  }
}

// Where output element (m, n) lives: C[M, N], or one of the three tensors of a split output.
__device__ __forceinline__ __half* out_ptr(const KParams& p, int m, int n) {
  if (p.split1 == 0) return p.C + static_cast<size_t>(m) * p.N + n;
  if (n < p.split1) return p.C + static_cast<size_t>(m) * p.split1 + n;
  if (n < p.split2) return p.C2 + static_cast<size_t>(m) * (p.split2 - p.split1) + (n - p.split1);
  return p.C3 + static_cast<size_t>(m) * (p.N - p.split2) + (n - p.split2);
}

// One output of the SiLU-gated pair: g and u are the fp32 sums of gate row and up row `j` of tile `tile`.
__device__ __forceinline__ void store_gate(const KParams& p, int m, int tile, int j, float g, float u) {
  if (p.bias != nullptr) {
    g += __half2float(p.bias[tile * kTileN + j]);
    u += __half2float(p.bias[tile * kTileN + 64 + j]);
  }
  const int n_out = tile * 64 + j, width = p.N >> 1;
  float v = act_fn<kActSilu>(g) * u;
  if (p.residual != nullptr) v += __half2float(p.residual[static_cast<size_t>(m) * width + n_out]);
  p.C[static_cast<size_t>(m) * width + n_out] = __float2half_rn(v);
}

// bias, activation and residual of one output element (fp32).
template <int ACT>
__device__ __forceinline__ float epilogue1(const KParams& p, int m, int n, float v) {
  if (p.bias != nullptr) v += __half2float(p.bias[n]);
  v = act_fn<ACT>(v);
  if (p.residual != nullptr) v += __half2float(p.residual[static_cast<size_t>(m) * p.N + n]);
  return v;
}

// Scale (int8 op), fused epilogue and rounding of two adjacent outputs of row m.
template <int OP, int ACT>
__device__ __forceinline__ __half2 finish_out2(const KParams& p, int m, int n, float2 v) {
  if ((OP == kOpW8A16NK || (OP == kOpW4A16NK && p.scale_groups <= 1)) && p.scales != nullptr) {
    const float2 sc = __half22float2(*reinterpret_cast<const __half2*>(p.scales + n));
    v.x *= sc.x;
    v.y *= sc.y;
  }
  if (ACT != kActNone || p.bias != nullptr || p.residual != nullptr) {
    v.x = epilogue1<ACT>(p, m, n, v.x);
    v.y = epilogue1<ACT>(p, m, n + 1, v.y);
  }
  return __floats2half2_rn(v.x, v.y);
}

// ... and their store (local, multicast or one store per rank).
template <int OP, int ACT>
__device__ __forceinline__ void store_out2(const KParams& p, int m, int n, float2 v) {
  const __half2 h = finish_out2<OP, ACT>(p, m, n, v);
  if (p.world == 0) {
    *reinterpret_cast<__half2*>(out_ptr(p, m, n)) = h;
  } else if (p.mc_C != nullptr) {
    multimem_st_b32(p.mc_C + static_cast<size_t>(m) * p.ldc + p.col0 + n, *reinterpret_cast<const uint32_t*>(&h));
  } else {
    const size_t off = static_cast<size_t>(m) * p.ldc + p.col0 + n;
    for (int q = 0; q < p.world; ++q) *reinterpret_cast<__half2*>(p.peer_C[q] + off) = h;
  }
}

// Eight adjacent outputs (n a multiple of 8) as one 16-byte store: the finishing team's stores sit at
// the very end of a call, and their number, not their bytes, is what the tail of the call feels
// (measured: 4-byte stores against 16-byte ones cost 0.2-0.9 us per call).
template <int OP, int ACT>
__device__ __forceinline__ void store_out8(const KParams& p, int m, int n, float4 a, float4 b) {
  const __half2 h0 = finish_out2<OP, ACT>(p, m, n, make_float2(a.x, a.y));
  const __half2 h1 = finish_out2<OP, ACT>(p, m, n + 2, make_float2(a.z, a.w));
  const __half2 h2 = finish_out2<OP, ACT>(p, m, n + 4, make_float2(b.x, b.y));
  const __half2 h3 = finish_out2<OP, ACT>(p, m, n + 6, make_float2(b.z, b.w));
  uint4 w;
  w.x = *reinterpret_cast<const uint32_t*>(&h0);
  w.y = *reinterpret_cast<const uint32_t*>(&h1);
  w.z = *reinterpret_cast<const uint32_t*>(&h2);
  w.w = *reinterpret_cast<const uint32_t*>(&h3);
  if (p.world == 0) {
    // eight columns never straddle a split (split1 and split2 are multiples of 8) and start 16-byte aligned
    *reinterpret_cast<uint4*>(out_ptr(p, m, n)) = w;
  } else if (p.mc_C != nullptr) {
    multimem_st_v4_f16x2(p.mc_C + static_cast<size_t>(m) * p.ldc + p.col0 + n, w.x, w.y, w.z, w.w);
  } else {
    const size_t off = static_cast<size_t>(m) * p.ldc + p.col0 + n;
    for (int q = 0; q < p.world; ++q) *reinterpret_cast<uint4*>(p.peer_C[q] + off) = w;
  }
}

// One thread tells every rank that one more output tile of this rank has been delivered.
// It is called after a barrier that all threads which stored parts of the tile have passed: one
// release at system scope by this thread (the multicast reduction carries it; otherwise one fence
// before the per-rank atomics) then orders all their stores before the counters, which is far
// cheaper than a system-scope fence in each of the storing threads.
__device__ __forceinline__ void signal_tile_delivered(const KParams& p) {
  if (p.mc_flag != nullptr) {
    multimem_red_release_add_u64(p.mc_flag + p.rank, 1ull);
    return;
  }
  fence_acq_rel_sys();
  for (int q = 0; q < p.world; ++q) atomicAdd_system(p.peer_flag[q] + p.rank, 1ull);
}

// Bounded wait until the first `world` per-source arrival counters at `flags` have all reached
// `target`.  One counter per source rank: a fast rank that is already pushing its next call
// cannot stand in for a slow one.
__device__ __forceinline__ bool wait_counters(const unsigned long long* flags, int world,
                                              unsigned long long target) {
  const unsigned long long t0 = globaltimer_ns();
  uint32_t spins = 0;
  for (int src = 0; src < world; ++src) {
    for (;;) {
      unsigned long long v;
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(flags + src) : "memory");
      if (v >= target) break;
      if ((++spins & 0xffu) == 0 && globaltimer_ns() - t0 > kWaitBudgetNs) return false;
    }
  }
  return true;
}

// What every role of a CTA needs to know about its share of the work list.
struct CtaRange {
  uint32_t KB;     // stages per output tile
  uint32_t total;  // tiles * KB
  uint32_t G;      // CTAs
  uint32_t ub, ue; // this CTA's stages [ub, ue)
};

// ------------------------------------ producer ------------------------------------------
// One thread.  Streams this CTA's stages into the ring: per stage the weight tile(s) and the
// matching slice of the activations, completing on full[s]; a slot is refilled once its
// consumer has arrived on empty[s].  MT = rows of the activation box.
template <int OP, int MT>
__device__ __forceinline__ void run_producer(const CUtensorMap& tmW, const CUtensorMap& tmX, const KParams& p,
                                             const CtaRange& r, uint32_t smem_base, uint32_t bar_base, int S,
                                             int cps, unsigned long long* trace) {
  using T = OpTraits<OP>;
  constexpr int cbytes = chunk_bytes(OP, MT);
  const uint32_t stage_bytes = cps * cbytes;
  const int k_per_stage = cps * T::chunkK;
  const uint32_t KB = r.KB, ub = r.ub, ue = r.ue;
  tma_prefetch_desc(&tmW);
  tma_prefetch_desc(&tmX);
  const uint64_t pol_w = policy_evict_first();
  const uint64_t pol_x = policy_evict_last();
  int tile = static_cast<int>(ub / KB);
  int kb = static_cast<int>(ub % KB);
  const int n_it = static_cast<int>(ue - ub);
  bool dead = false;
  int issued = 0;
  if (trace) trace[1] = globaltimer_ns();  // first copy about to be issued

  auto stage_chunks = [&](int kblock) {
    const int k0 = kblock * k_per_stage;
    const int nch = (p.K - k0 + T::chunkK - 1) / T::chunkK;
    return nch < cps ? nch : cps;
  };
  auto issue_w = [&](int s, int tl, int kblock, int nch) {
    const uint32_t full = bar_base + 8 * s;
    uint32_t dst = smem_base + s * stage_bytes;
    for (int c = 0; c < nch; ++c) {
      const int kc = kblock * k_per_stage + c * T::chunkK;
      if constexpr (OP == kOpF16KN) {
        tma_load_2d(dst, &tmW, full, tl * kTileN, kc, pol_w);
        tma_load_2d(dst + 8192, &tmW, full, tl * kTileN + 64, kc, pol_w);
      } else {
        // the weight map counts elements of its own type: two k per byte for the int4 op
        tma_load_2d(dst, &tmW, full, OP == kOpW4A16NK ? kc >> 1 : kc, tl * kTileN, pol_w);
      }
      dst += cbytes;
    }
  };
  auto issue_x = [&](int s, int kblock, int nch) {
    const uint32_t full = bar_base + 8 * s;
    uint32_t dst = smem_base + s * stage_bytes + kChunkWBytes;
    for (int c = 0; c < nch; ++c) {
      const int kc = kblock * k_per_stage + c * T::chunkK;
#pragma unroll
      for (int xb = 0; xb < T::xBoxes; ++xb)
        tma_load_2d(dst + xb * MT * 128, &tmX, full, kc + xb * 64, 0, pol_x);
      dst += cbytes;
    }
  };

  // The weight never depends on earlier kernels, so the first ring-full of weight tiles is
  // requested right away.  Activations may be the output of the previous kernel of the
  // stream (programmatic dependent launch: this grid may have started while that kernel
  // was still draining) or of a layer that other ranks are still pushing, so they are
  // only read after griddepcontrol.wait (a no-op for an ordinary launch) and, if asked,
  // after the arrival counters of that layer have reached their target.
  griddep_launch_dependents();
  const int pre = n_it < S ? n_it : S;
  {
    int t2 = tile, k2 = kb;
    for (int i = 0; i < pre; ++i) {
      const int nch = stage_chunks(k2);
      mbar_arrive_expect_tx(bar_base + 8 * i, nch * cbytes);
      issue_w(i, t2, k2, nch);
      if (++k2 == static_cast<int>(KB)) { k2 = 0; ++t2; }
    }
  }
  // While the previous kernel drains, HBM would idle once the ring is full: ask for the next
  // stages' weights to be brought into L2 meanwhile (they are loaded from there later).
  if (p.l2_prefetch > 0) {
    int t2 = tile, k2 = kb;
    for (int i = 0; i < pre; ++i)
      if (++k2 == static_cast<int>(KB)) { k2 = 0; ++t2; }
    const int last = (pre + p.l2_prefetch) < n_it ? (pre + p.l2_prefetch) : n_it;
    for (int i = pre; i < last; ++i) {
      const int nch = stage_chunks(k2);
      for (int c = 0; c < nch; ++c) {
        const int kc = k2 * k_per_stage + c * T::chunkK;
        if constexpr (OP == kOpF16KN) {
          tma_prefetch_l2_2d(&tmW, t2 * kTileN, kc);
          tma_prefetch_l2_2d(&tmW, t2 * kTileN + 64, kc);
        } else {
          tma_prefetch_l2_2d(&tmW, OP == kOpW4A16NK ? kc >> 1 : kc, t2 * kTileN);
        }
      }
      if (++k2 == static_cast<int>(KB)) { k2 = 0; ++t2; }
    }
  }
  griddep_wait();
  // after the wait: every earlier launch of the stream, including one that still compared these
  // buffers' counters with the old total, has completed
  if (blockIdx.x == 0 && p.target_dev != nullptr) atomicAdd(p.target_dev, static_cast<unsigned long long>(p.tiles));
  unsigned long long wait_target = p.wait_target;
  if (p.wait_flags != nullptr && p.wait_target_dev != nullptr) wait_target = __ldcg(p.wait_target_dev);
  if (p.wait_flags != nullptr && !wait_counters(p.wait_flags, p.wait_world, wait_target)) {
    // The activations never became ready.  Complete the armed stages with what is there
    // so that no copy is left in flight; the status word tells the caller.
    atomicExch(p.status, kStatusTimeout);
  }
  for (int i = 0; i < pre; ++i) {
    issue_x(i, kb, stage_chunks(kb));
    if (++kb == static_cast<int>(KB)) { kb = 0; ++tile; }
  }
  int it = pre;
  issued = pre;
  // ring slot and its use count advance by increments: this loop is single-threaded and on the
  // critical path of the ring, a runtime division per stage would show up in the call time
  int s = (pre == S) ? 0 : pre;
  uint32_t use = (pre == S) ? 1u : 0u;
  for (; it < n_it; ++it, s = (s + 1 == S) ? 0 : s + 1, use += (s == 0)) {
    if (!mbar_wait_bounded(bar_base + 8 * (S + s), (use & 1) ^ 1, kWaitBudgetNs)) {
      dead = true;
      break;
    }
    const int nch = stage_chunks(kb);
    mbar_arrive_expect_tx(bar_base + 8 * s, nch * cbytes);
    issue_w(s, tile, kb, nch);
    issue_x(s, kb, nch);
    ++issued;
    if (++kb == static_cast<int>(KB)) {
      kb = 0;
      ++tile;
    }
  }
  if (trace) trace[2] = globaltimer_ns();  // last copy issued
  if (dead) {
    atomicExch(p.status, kStatusTimeout);
    // let copies already in flight land before the CTA's shared memory goes away
    const int back = issued < S ? issued : S;
    for (int i = issued - back; i < issued; ++i)
      mbar_wait_bounded(bar_base + 8 * (i % S), (i / S) & 1, kWaitBudgetNs);
  }
}

// ------------------------------------ finisher ------------------------------------------
// Two teams of MT/4 warps (named barriers kFinBarrier, kFinBarrier + 1).  A CTA has at most two
// partial segments: the tail of the tile its share starts in and the head of the tile it ends
// in.  Team 0 takes the first partial of the CTA, team 1 the second, so that a CTA whose first
// partial turns out to be the last contribution to its tile (a reduction of a few microseconds)
// does not hold back the ticket of its second partial.  The teams walk the same segment list
// as the consumers.
// For its partial segment a team waits until all consumer threads have stored their share of
// the partial tile; one thread publishes it (fence + ticket) and, if this CTA was the last
// contributor of the tile, the warps add up all partials in CTA order and write C: warp w
// takes rows 4w..4w+3, lane l columns 4l..4l+3, contributors four at a time, so every lane
// has sixteen 16-byte loads in flight and the whole tile is fetched in one round trip (two
// beyond four contributors).  Each element is summed in CTA order whatever the arrival
// order, which keeps the result bit-reproducible.  The consumers meanwhile go on streaming.
constexpr int kFinBarrier = 3;
template <int MT>
__host__ __device__ constexpr int finisher_warps() { return MT < 16 ? MT / 4 : 4; }  // taller tiles: 16 rows at a time

template <int OP, int MT>
__device__ __forceinline__ void run_finisher(const KParams& p, const CtaRange& r, uint32_t bar_flush,
                                             volatile uint32_t* prev_slot, int team, int fin_warp,
                                             int lane, unsigned long long* trace) {
  constexpr int FW = finisher_warps<MT>();
  bar_flush += 8 * team;
  prev_slot += team;
  const int bar_id = kFinBarrier + team;
  const uint32_t KB = r.KB, total = r.total, G = r.G, ub = r.ub, ue = r.ue;
  uint32_t u = ub;
  uint32_t ev = 0;
  bool dead = false;
  const bool leader = (fin_warp == 0 && lane == 0);
  while (u < ue) {
    const uint32_t tile = u / KB;
    const uint32_t kb0 = u - tile * KB;
    const uint32_t len = (KB - kb0) < (ue - u) ? (KB - kb0) : (ue - u);
    if (len != KB && ev == static_cast<uint32_t>(team) && !dead) {
      bool ok = mbar_wait_bounded(bar_flush, 0, kWaitBudgetNs * 4);
      ok = __all_sync(0xffffffffu, ok);
      const uint32_t c_first = cta_of_unit(tile * KB, total, G);
      const uint32_t c_last = cta_of_unit(tile * KB + KB - 1, total, G);
      if (leader) {
        // a timeout is published like a ticket that is never the last one
        uint32_t prev = 0xffffffffu;
        if (ok) {
          __threadfence();
          prev = atomicAdd(p.tickets + tile, 1u);
          // the last contributor: acquire the other CTAs' partial tiles for the whole team (the barrier
          // below carries this thread's fence to the other warps; one fence instead of one per thread)
          if (prev == c_last - c_first) fence_acq_rel_gpu();
        } else {
          atomicExch(p.status, kStatusTimeout);
        }
        *prev_slot = prev;
      }
      named_bar_sync(bar_id, FW * 32);
      const uint32_t prev = *prev_slot;
      if (prev == 0xffffffffu) dead = true;
      if (prev == c_last - c_first && p.act != kActSiluGate) {
        // Warp w takes rows 4w..4w+3 of the tile: lanes 0-15 rows 4w and 4w + 2, lanes 16-31 rows 4w + 1 and
        // 4w + 3, eight columns per lane, so a row leaves as sixteen 16-byte stores of one instruction.
        // Contributors are added in CTA order, four at a time (sixteen 16-byte loads in flight per lane).
        const int hw = lane >> 4, cl = lane & 15;
        const int n0 = tile * kTileN + 8 * cl;
#pragma unroll 1
        for (int m0 = 4 * fin_warp; m0 < MT && m0 < p.M; m0 += 4 * FW) {
          float4 sum[2][2];
#pragma unroll
          for (int i = 0; i < 2; ++i) sum[i][0] = sum[i][1] = make_float4(0.f, 0.f, 0.f, 0.f);
          for (uint32_t c0 = c_first; c0 <= c_last; c0 += 4) {
            float4 v[4][2][2];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t c = c0 + j;
              if (c <= c_last) {
                const uint32_t cslot = (range_begin(c, total, G) / KB == tile) ? 0u : 1u;
                const float4* src = reinterpret_cast<const float4*>(
                    p.partials + (static_cast<size_t>(c) * 2 + cslot) * (MT * kTileN));
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                  v[j][i][0] = __ldcg(src + (m0 + hw + 2 * i) * 32 + 2 * cl);
                  v[j][i][1] = __ldcg(src + (m0 + hw + 2 * i) * 32 + 2 * cl + 1);
                }
              } else {
#pragma unroll
                for (int i = 0; i < 2; ++i) v[j][i][0] = v[j][i][1] = make_float4(0.f, 0.f, 0.f, 0.f);
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
              for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                  sum[i][h].x += v[j][i][h].x;
                  sum[i][h].y += v[j][i][h].y;
                  sum[i][h].z += v[j][i][h].z;
                  sum[i][h].w += v[j][i][h].w;
                }
          }
          with_act(p.act, [&](auto tag) {
            constexpr int ACT = decltype(tag)::value;
#pragma unroll
            for (int i = 0; i < 2; ++i) {
              const int m = m0 + hw + 2 * i;
              if (m < p.M) store_out8<OP, ACT>(p, m, n0, sum[i][0], sum[i][1]);
            }
          });
        }
      } else if (prev == c_last - c_first) {
        // SiLU gate: lanes 0-15 hold gate columns 4l..4l+3 of the tile, lanes 16-31 the matching up columns
#pragma unroll 1
        for (int m0 = 4 * fin_warp; m0 < MT && m0 < p.M; m0 += 4 * FW) {
          float4 sum[4];
#pragma unroll
          for (int i = 0; i < 4; ++i) sum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
          for (uint32_t c0 = c_first; c0 <= c_last; c0 += 4) {
            float4 v[4][4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t c = c0 + j;
              if (c <= c_last) {
                const uint32_t cslot = (range_begin(c, total, G) / KB == tile) ? 0u : 1u;
                const float4* src = reinterpret_cast<const float4*>(
                    p.partials + (static_cast<size_t>(c) * 2 + cslot) * (MT * kTileN));
#pragma unroll
                for (int i = 0; i < 4; ++i) v[j][i] = __ldcg(src + (m0 + i) * 32 + lane);
              } else {
#pragma unroll
                for (int i = 0; i < 4; ++i) v[j][i] = make_float4(0.f, 0.f, 0.f, 0.f);
              }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                sum[i].x += v[j][i].x;
                sum[i].y += v[j][i].y;
                sum[i].z += v[j][i].z;
                sum[i].w += v[j][i].w;
              }
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float ux = __shfl_down_sync(0xffffffffu, sum[i].x, 16), uy = __shfl_down_sync(0xffffffffu, sum[i].y, 16);
            const float uz = __shfl_down_sync(0xffffffffu, sum[i].z, 16), uw = __shfl_down_sync(0xffffffffu, sum[i].w, 16);
            const int m = m0 + i;
            if (lane < 16 && m < p.M) {
              store_gate(p, m, tile, 4 * lane, sum[i].x, ux);
              store_gate(p, m, tile, 4 * lane + 1, sum[i].y, uy);
              store_gate(p, m, tile, 4 * lane + 2, sum[i].z, uz);
              store_gate(p, m, tile, 4 * lane + 3, sum[i].w, uw);
            }
          }
        }
      }
      // every warp of the team is done with the tile's partials before the ticket is reset (and
      // has issued its stores into the other ranks' outputs before the leader signals them)
      named_bar_sync(bar_id, FW * 32);
      if (leader) {
        if (prev == c_last - c_first) {
          p.tickets[tile] = 0;  // ready for the next launch
          if (p.world > 0) signal_tile_delivered(p);
        }
      }
    }
    if (len != KB) ++ev;
    u += len;
  }
  if (trace && leader) trace[5 + 8 * team] = globaltimer_ns();  // team done (slot 5: team 0, slot 13: team 1)
}

// Warp roles: [0, ncw) consume, ncw produces (TMA), then two teams of MT/4 warps finish split tiles.
// The quantized ops are planned with at most six consumer warps (three with a 16-row tile), which
// keeps the CTA at 384 threads or fewer and leaves their dequantising inner loops 168 registers.
template <int OP, int MT>
__host__ __device__ constexpr int streamk_max_threads() {
  return ((op_is_quantized(OP) ? (MT == 16 ? 3 : 6) : kMaxConsumerWarps) + 1 + 2 * finisher_warps<MT>()) * 32;
}

template <int OP, int MT>
__global__ void __launch_bounds__(streamk_max_threads<OP, MT>(), 1)
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
  const uint32_t bar_base = smem_base + ring_bytes + red_bytes;  // full[S], empty[S], flush[2]
  const uint32_t bar_flush = bar_base + 16 * S;     // consumers -> team t: "my partial #t is stored"
  volatile uint32_t* prev_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + ring_bytes + red_bytes + 16 * S + 16);

  // A launch whose thread count or shared memory does not fit the parameters would index
  // shared memory out of bounds: refuse it instead (the host reads the status word).
  if (blockDim.x != static_cast<unsigned>((ncw + 1 + 2 * finisher_warps<MT>()) * 32) ||
      dynamic_smem_size() < 1023u + ring_bytes + red_bytes + 16u * S + 32u) {
    if (threadIdx.x == 0) atomicExch(p.status, kStatusBadLaunch);
    return;
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int nct = ncw * 32;
  unsigned long long* trace = p.trace ? p.trace + kTraceSlots * blockIdx.x : nullptr;
  if (trace && threadIdx.x == 0) trace[0] = globaltimer_ns();  // CTA start
  if (trace && threadIdx.x == 0) trace[12] = smid();                     // which SM ran this CTA

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_base + 8 * s, 1);        // full: one arrive (the producer's expect_tx)
      mbar_init(bar_base + 8 * (S + s), 1);  // empty: one arrive (the consuming warp's lane 0)
    }
    mbar_init(bar_flush, nct);
    mbar_init(bar_flush + 8, nct);
    fence_mbar_init();
    fence_proxy_async();
  }
  __syncthreads();

  const uint32_t KB = p.k_blocks;
  const uint32_t total = static_cast<uint32_t>(p.tiles) * KB;
  const uint32_t G = gridDim.x;
  const uint32_t ub = range_begin(blockIdx.x, total, G);
  const uint32_t ue = range_begin(blockIdx.x + 1, total, G);
  const int k_per_stage = cps * T::chunkK;

  const CtaRange range{KB, total, G, ub, ue};
  if (warp == ncw) {
    if (lane == 0) run_producer<OP, MT>(tmW, tmX, p, range, smem_base, bar_base, S, cps, trace);
    return;
  }
  if (warp > ncw) {
    const int fw = warp - ncw - 1;
    run_finisher<OP, MT>(p, range, bar_flush, prev_slot, fw / finisher_warps<MT>(), fw % finisher_warps<MT>(), lane,
                         trace);
    return;
  }

  // -------------------------------- consumer warps --------------------------------
  const int ctid = threadIdx.x;  // consumers are warps 0..ncw-1
  const int g = lane >> 2, t = lane & 3;
  bool dead = false;
  uint32_t u = ub;
  uint32_t ev = 0;  // partial segments flushed so far
  int it0 = 0;      // CTA-local index of the first stage of the current segment
  float acc[8][MT / 8][4];

  while (u < ue) {
    const uint32_t tile = u / KB;
    const int kb0 = static_cast<int>(u - tile * KB);
    const int len = static_cast<int>((KB - kb0) < (ue - u) ? (KB - kb0) : (ue - u));

#pragma unroll
    for (int rg = 0; rg < 8; ++rg)
#pragma unroll
      for (int j = 0; j < MT / 8; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) acc[rg][j][i] = 0.f;

    // stages of this segment that belong to this warp: CTA-local index == warp (mod ncw)
    const int first = it0 + ((warp - it0 % ncw) + ncw) % ncw;
    int s = first % S;
    uint32_t use = first / S;
    for (int it = first; it < it0 + len && !dead; it += ncw, s += ncw) {
      if (s >= S) {  // stages % warps == 0: the slot index wraps exactly
        s -= S;
        ++use;
      }
      bool ok = mbar_wait_bounded(bar_base + 8 * s, use & 1, kWaitBudgetNs);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        dead = true;
        if (lane == 0) atomicExch(p.status, kStatusTimeout);
        break;
      }
      if (trace && it == 0 && lane == 0) trace[3] = globaltimer_ns();  // first stage landed
      const int k0 = (kb0 + (it - it0)) * k_per_stage;
      int nch = (p.K - k0 + T::chunkK - 1) / T::chunkK;
      nch = nch < cps ? nch : cps;
      uint32_t base = smem_base + s * stage_bytes;
      for (int c = 0; c < nch; ++c) {
        consume_chunk<OP, MT>(base, base + kChunkWBytes, lane, acc, p, tile * kTileN, k0 + c * T::chunkK);
        base += cbytes;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_base + 8 * (S + s));
    }

    if (trace && ctid == 0) trace[4] = globaltimer_ns();  // warp 0 done with the segment's math
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
    const bool whole = (len == static_cast<int>(KB));
    named_bar_sync(1, nct);
    if (trace && ctid == 0) trace[7] = globaltimer_ns();  // all warps done with the segment's math

    const int slot = (u == ub) ? 0 : 1;
    float* mypart = p.partials + (static_cast<size_t>(blockIdx.x) * 2 + slot) * (MT * kTileN);
    auto reduce_warps = [&](int e) {  // sum of the consumer warps' copies of outputs 2e, 2e+1 of the tile
      const int m = e >> 6, n2 = (e & 63) * 2;
      float2 v = make_float2(0.f, 0.f);
      for (int w = 0; w < ncw; ++w) {
        const float2 a = *reinterpret_cast<const float2*>(red + w * (MT * kRedStride) + m * kRedStride + n2);
        v.x += a.x;
        v.y += a.y;
      }
      return v;
    };
    if (whole) {
      with_act(p.act, [&](auto tag) {
        constexpr int ACT = decltype(tag)::value;
        for (int e = ctid; e < MT * 64; e += nct) {
          const int m = e >> 6, n2 = (e & 63) * 2;
          if (m < p.M) store_out2<OP, ACT>(p, m, tile * kTileN + n2, reduce_warps(e));
        }
      });
    } else {
      for (int e = ctid; e < MT * 64; e += nct) *reinterpret_cast<float2*>(mypart + 2 * e) = reduce_warps(e);
    }
    if (!whole) {
      mbar_arrive(bar_flush + 8 * ev);  // release: this thread's share of partial #ev is stored
      ++ev;
    }
    named_bar_sync(1, nct);  // `red` is free again; a pushed tile's stores are issued
    if (whole && p.world > 0 && ctid == 0) signal_tile_delivered(p);
    if (trace && ctid == 0) trace[6] += 1;  // segments of this CTA

    u += len;
    it0 += len;
  }
}

// Waits (bounded) until each of the `world` per-source arrival counters of this rank has
// reached `target`, i.e. until every rank has delivered all its tiles of the calls enqueued so
// far.  One thread; ordered on the stream, so whatever follows it sees the complete output.
// Launched with programmatic stream serialization: the launch after it may start at once (a GEMM
// then streams its first weight tiles while this kernel still waits; it touches nothing else before
// its own griddepcontrol.wait, which returns when this kernel has completed), and this kernel itself
// starts early and begins to look at the counters once everything before it in the stream is done.
__global__ void fg_push_wait_kernel(const unsigned long long* flags, int world, unsigned long long target,
                                    int* status) {
  griddep_launch_dependents();
  griddep_wait();
  if (threadIdx.x != 0) return;
  if (!wait_counters(flags, world, target)) atomicExch(status, kStatusTimeout);
}
// The same with the target read from device memory (the running total that pushing launches keep
// in *target_dev): nothing in the launch changes from call to call, so it can be replayed in a graph.
__global__ void fg_push_wait_dev_kernel(const unsigned long long* flags, int world,
                                        const unsigned long long* target_dev, int* status) {
  griddep_launch_dependents();
  griddep_wait();  // the launches that add to *target_dev have completed
  if (threadIdx.x != 0) return;
  const unsigned long long target = __ldcg(target_dev);
  if (!wait_counters(flags, world, target)) atomicExch(status, kStatusTimeout);
}

// Several such waits in one launch (one lane per flag array): the step of a caller that closes
// many pushed outputs at once pays one launch instead of one per output.
constexpr int kMaxWaits = 16;
struct WaitList {
  const unsigned long long* flags[kMaxWaits];
  const unsigned long long* target_dev[kMaxWaits];
  int count;
};
__global__ void fg_push_wait_many_kernel(const WaitList w, int world, int* status) {
  griddep_launch_dependents();
  griddep_wait();
  const int i = threadIdx.x;
  if (i >= w.count) return;
  if (!wait_counters(w.flags[i], world, __ldcg(w.target_dev[i]))) atomicExch(status, kStatusTimeout);
}

}  // namespace fg
