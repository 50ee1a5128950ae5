// Row-split GEMV for one or two token rows, CUDA-core math, sm_100a.
//
//   C[m, n] = sum_k x[m, k] * W[n, k]        m < M <= 2,  W fp16
//   C[0, n] = scale[n] * sum_k x[0, k] * W8[n, k]         W8 int8, one token row
//
// With so few token rows the tensor cores buy nothing; what costs time is everything around the
// stream: a reduction between CTAs, a tail of dependent memory round trips, SMs that finish at
// different times.  So here a CTA owns WHOLE weight rows (output columns): every output element is
// summed inside one CTA in a fixed order and nothing is ever exchanged between CTAs.
//
//  * One persistent CTA per SM.  Rows of an NxK weight are contiguous, so a ring stage is one
//    untiled bulk copy (cp.async.bulk, no cluster multicast) of 1-8 whole rows, about 16 KB.
//  * Each CTA first streams a fixed share of rows (known without asking anybody, so the first
//    ring-full is requested before griddepcontrol.wait) and then takes blocks of rows from a
//    counter in the workspace until none are left; the result does not depend on who computed a
//    row.  The planner deals out every whole stage up front and leaves only the remainder to the
//    counter (measured on B200: a larger on-demand share costs more in atomic round trips of the
//    single copy-issuing thread than it gains in balance: 8192 x 8192, M = 1: 22.4 us all up front,
//    22.7 us with 20 % on demand, 28 us all on demand).  The last CTA to stop asking puts the
//    counter back to zero for the next launch.
//  * x (at most 64 KB) is copied into shared memory once, after the grid dependency is resolved, by
//    ordinary loads of the consumer warps (not through the copy engine, where it would wait behind
//    the weight rows already requested).
//  * A stage belongs to ONE consumer warp (stage i to warp i mod warps; the ring depth is a multiple
//    of the warp count, so a slot always meets the same warp): lane l multiplies the 16-byte pieces
//    l, l + 32, ... of each row of the stage (fma.rn.f32.f16: fp16 operands, exact product, fp32 sum), the
//    lanes' sums are added by shuffles, and one lane per output applies scale, bias, activation and
//    residual and rounds once to fp16.  No barrier and no reduction spans the warps: they work on
//    different stages at the same time, and the per-stage overhead of a thread is amortised over
//    hundreds of weights.  The order of every sum is fixed.
//  * How many warps: a warp multiplies about 12 GB/s of fp16 weights for one token row and an SM
//    receives 47 GB/s, so the planner gives one row of fp16 weights five to nine warps that own two
//    or three ring slots each (a warp multiplies one slot while its others refill); two token rows
//    and int8 weights, which do two and four times the work per byte, get up to twelve.
//
// Replaces gemv_fp16 (backend/cuda/hk/fastgemv.cuh:503-562),
// gemv_fp16_bs2 (backend/cuda/czn/fastgemm.cuh:302-392) and gemv_quantized_int8
// (backend/cuda/hk/fastgemv.cuh:316-389) of the reference, and serves
// edgemm_m8n128k64x4_bt and its aliases when they are called with one row (two rows for weights of up to 48 Mi elements).
#pragma once
#include "fg_kernels.cuh"

namespace fg {

constexpr int kGemvMaxWarps = 12;   // consumer warps
constexpr int kGemvMaxM = 2;
constexpr int kGemvMaxOut = 8;      // rows per stage x token rows: outputs one stage produces

struct GemvParams {
  const void* W;             // [N, K] fp16, or int8 (then M == 1)
  const __half* scales;      // int8 weights: one fp16 scale per row, or nullptr (scale 1)
  const __half* x;           // [M, K]
  __half* C;                 // [M, N]
  const __half* bias;        // [N] or nullptr
  const __half* residual;    // [M, N] or nullptr
  int act;
  int split1, split2;        // output columns split over C, C2, C3 (see KParams); split1 == 0: all in C
  __half* C2;
  __half* C3;
  int M, N, K;
  int rows_per_stage;        // 1, 2, 4 or 8, times M at most kGemvMaxOut
  int stage_bytes;           // ring slot size = rows_per_stage * bytes per row
  int stages;
  int static_rows;           // CTA c first streams rows [c * static_rows, (c + 1) * static_rows)
  int l2_prefetch_bytes;     // of the static share, asked into L2 while waiting for the previous kernel
  unsigned int* next;        // workspace: next dynamic block of rows (zero between launches)
  unsigned int* exited;      // workspace: CTAs that have left (wraps to zero)
  int* status;
  unsigned long long* trace;
};

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
      ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(policy)
      : "memory");
}
__device__ __forceinline__ void bulk_prefetch_l2(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

// acc0 += w.lo * x.lo, acc1 += w.hi * x.hi: fp16 operands taken as they are, product and sum in
// fp32 with one rounding (the mixed-precision FMA of sm_100: no conversion instructions).
__device__ __forceinline__ void fma_f16x2_f32(float& acc0, float& acc1, uint32_t w, uint32_t x) {
  asm("{\n\t.reg .b16 wl, wh, xl, xh;\n\t"
      "mov.b32 {wl, wh}, %2;\n\t"
      "mov.b32 {xl, xh}, %3;\n\t"
      "fma.rn.f32.f16 %0, wl, xl, %0;\n\t"
      "fma.rn.f32.f16 %1, wh, xh, %1;\n\t}"
      : "+f"(acc0), "+f"(acc1)
      : "r"(w), "r"(x));
}

// Four int8 weights (one 32-bit word, k ascending with the byte index) against four fp16 activations
// (two words).  An int8 b becomes the fp16 number b exactly in three integer-pipe steps: flip the sign
// bit (b + 128 as an unsigned byte), put the byte under the exponent of 1024 (0x6400 | byte = 1024 +
// byte, two bytes per `prmt`), subtract 1152.
__device__ __forceinline__ void fma_i8x4_f32(float& acc0, float& acc1, uint32_t w, uint32_t x01, uint32_t x23) {
  const uint32_t u = w ^ 0x80808080u;
  uint32_t h01, h23;
  asm("prmt.b32 %0, %1, %2, 0x4140;" : "=r"(h01) : "r"(u), "r"(0x64646464u));
  asm("prmt.b32 %0, %1, %2, 0x4342;" : "=r"(h23) : "r"(u), "r"(0x64646464u));
  asm("sub.rn.f16x2 %0, %0, %1;" : "+r"(h01) : "r"(0x64806480u));
  asm("sub.rn.f16x2 %0, %0, %1;" : "+r"(h23) : "r"(0x64806480u));
  fma_f16x2_f32(acc0, acc1, h01, x01);
  fma_f16x2_f32(acc0, acc1, h23, x23);
}

// The same stage for int8 weights (one token row): lane l takes the 16-byte pieces l, l + 32, ... of
// every row, sixteen k each, against 32 bytes of x.  x sits in shared memory as two halves: the
// first eight activations of every group of sixteen, then the second eight, so that each of the two
// loads is 16 bytes per lane at a lane stride of 16 bytes (no bank conflicts).
template <int RB>
__device__ __forceinline__ void gemv_stage_i8(uint32_t wbase, uint32_t xbase, int K, int nrows, int lane,
                                              float (&out)[kGemvMaxOut]) {
  const int pieces = K >> 4;
  const uint32_t row_bytes = static_cast<uint32_t>(K);
  float acc[RB][4];
#pragma unroll
  for (int r = 0; r < RB; ++r) acc[r][0] = acc[r][1] = acc[r][2] = acc[r][3] = 0.f;
#pragma unroll 4
  for (int i = lane; i < pieces; i += 32) {
    uint32_t xv[8];
    lds_v4(xbase + i * 16, xv[0], xv[1], xv[2], xv[3]);
    lds_v4(xbase + row_bytes + i * 16, xv[4], xv[5], xv[6], xv[7]);
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      uint32_t wv[4];
      lds_v4(wbase + r * row_bytes + i * 16, wv[0], wv[1], wv[2], wv[3]);
      fma_i8x4_f32(acc[r][0], acc[r][1], wv[0], xv[0], xv[1]);
      fma_i8x4_f32(acc[r][2], acc[r][3], wv[1], xv[2], xv[3]);
      fma_i8x4_f32(acc[r][0], acc[r][1], wv[2], xv[4], xv[5]);
      fma_i8x4_f32(acc[r][2], acc[r][3], wv[3], xv[6], xv[7]);
    }
  }
#pragma unroll
  for (int r = 0; r < RB; ++r) out[r] = (acc[r][0] + acc[r][1]) + (acc[r][2] + acc[r][3]);
}

// One stage, one warp: RB rows (nrows of them valid) against the M rows of x in shared memory.
// Lane l takes the 16-byte pieces l, l + 32, ... of every row; even and odd k go to separate
// accumulators so that two FMA chains are in flight per output.
template <int M, int RB>
__device__ __forceinline__ void gemv_stage(uint32_t wbase, uint32_t xbase, int K, int nrows, int lane,
                                           float (&out)[kGemvMaxOut]) {
  const int pieces = K >> 3;  // eight k per piece
  const uint32_t row_bytes = static_cast<uint32_t>(K) * 2;
  float acc[RB][M][2];
#pragma unroll
  for (int r = 0; r < RB; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) acc[r][m][0] = acc[r][m][1] = 0.f;
#pragma unroll 4
  for (int i = lane; i < pieces; i += 32) {
    uint32_t xv[M][4];
#pragma unroll
    for (int m = 0; m < M; ++m) lds_v4(xbase + (static_cast<uint32_t>(m) * K + i * 8) * 2, xv[m][0], xv[m][1], xv[m][2], xv[m][3]);
    // all RB rows of the slot, also where the stage holds fewer (the last block of a share): what the
    // slot's other rows hold is stale but readable, and their sums are never stored
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      uint32_t wv[4];
      lds_v4(wbase + r * row_bytes + i * 16, wv[0], wv[1], wv[2], wv[3]);
#pragma unroll
      for (int m = 0; m < M; ++m)
#pragma unroll
        for (int j = 0; j < 4; ++j) fma_f16x2_f32(acc[r][m][0], acc[r][m][1], wv[j], xv[m][j]);
    }
  }
#pragma unroll
  for (int r = 0; r < RB; ++r)
#pragma unroll
    for (int m = 0; m < M; ++m) out[r * M + m] = acc[r][m][0] + acc[r][m][1];
}

// WB = bytes per weight: 2 (fp16) or 1 (int8, one token row, per-row scale in the epilogue).
template <int M, int WB = 2>
__global__ void __launch_bounds__((kGemvMaxWarps + 1) * 32, 1) fg_gemv_kernel(const GemvParams p) {
  static_assert(M >= 1 && M <= kGemvMaxM, "token rows");
  static_assert(WB == 2 || (WB == 1 && M == 1), "int8 weights: one token row");
  constexpr int wbytes = WB;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 127u) & ~127u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const int S = p.stages;
  const int K = p.K;
  const int nw = (static_cast<int>(blockDim.x) >> 5) - 1;  // consumer warps; the last warp produces
  const uint32_t x_bytes = (static_cast<uint32_t>(M) * K * 2 + 127u) & ~127u;
  const uint32_t ring_base = smem_base + x_bytes;
  const uint32_t ring_bytes = static_cast<uint32_t>(S) * p.stage_bytes;
  const uint32_t meta_off = x_bytes + ring_bytes;                  // [S] {first row, rows}
  const uint32_t bar_off = meta_off + 8 * S;                       // full[S], empty[S], x
  const uint32_t bar_base = smem_base + bar_off;
  const uint32_t bar_x = bar_base + 16 * S;
  const int RB = p.rows_per_stage;

  if (nw < 1 || nw > kGemvMaxWarps || (blockDim.x & 31u) != 0 || RB < 1 || RB * M > kGemvMaxOut || (S % nw) != 0 ||
      dynamic_smem_size() < 127u + bar_off + 16u * S + 8u) {
    if (threadIdx.x == 0) atomicExch(p.status, kStatusBadLaunch);
    return;
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned long long* trace = p.trace ? p.trace + kTraceSlots * blockIdx.x : nullptr;
  if (trace && threadIdx.x == 0) {
    trace[0] = globaltimer_ns();
    trace[12] = smid();
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_base + 8 * s, 1);        // full: the producer's arrive
      mbar_init(bar_base + 8 * (S + s), 1);  // empty: lane 0 of the warp the slot belongs to
    }
    mbar_init(bar_x, 1);
    fence_mbar_init();
    fence_proxy_async();
  }
  __syncthreads();

  const int G = gridDim.x;
  const int row_bytes = K * wbytes;
  int2* meta = reinterpret_cast<int2*>(smem_gen + meta_off);

  if (warp == nw) {
    // ------------------------------------ producer ------------------------------------
    if (lane == 0) {
      const uint64_t pol_w = policy_evict_first();
      const uint8_t* Wb = static_cast<const uint8_t*>(p.W);
      if (trace) trace[1] = globaltimer_ns();
      auto arm = [&](int s, int row0, int nrows) {
        meta[s] = make_int2(row0, nrows);
        const uint32_t bytes = static_cast<uint32_t>(nrows) * row_bytes;
        mbar_arrive_expect_tx(bar_base + 8 * s, bytes);
        bulk_load_1d(ring_base + s * p.stage_bytes, Wb + static_cast<size_t>(row0) * row_bytes, bytes, bar_base + 8 * s, pol_w);
      };
      griddep_launch_dependents();
      int row = blockIdx.x * p.static_rows;
      const int end = row + p.static_rows;
      int s = 0;
      uint32_t use = 0;
      int issued = 0;
      bool dead = false;
      // the static share never depends on anybody: its first ring-full goes out at once
      for (; issued < S && row < end; ++issued, row += RB) {
        arm(s, row, (end - row) < RB ? (end - row) : RB);
        s = (s + 1 == S) ? 0 : s + 1;
        use += (s == 0);
      }
      if (p.l2_prefetch_bytes > 0 && row < end) {
        const long long left = static_cast<long long>(end - row) * row_bytes;
        const uint32_t n = left < p.l2_prefetch_bytes ? static_cast<uint32_t>(left) : static_cast<uint32_t>(p.l2_prefetch_bytes);
        const uint8_t* src = Wb + static_cast<size_t>(row) * row_bytes;
        for (uint32_t o = 0; o < n; o += 16384) bulk_prefetch_l2(src + o, (n - o) < 16384u ? (n - o) : 16384u);
      }
      griddep_wait();
      if (trace) trace[14] = globaltimer_ns();
      // x may be read now.  The consumer warps fetch it with ordinary loads: a bulk copy would
      // queue in this SM's copy engine behind the ring-full of weight rows requested above.
      mbar_arrive(bar_x);
      // the first dynamic block is asked for now, long before it is needed
      const int dyn0 = G * p.static_rows;
      unsigned int nxt = atomicAdd(p.next, 1u);
      auto wait_slot = [&]() {
        // before slot s is armed for the (use + 1)-th time its consumers must have released use number `use`
        if (use == 0) return true;
        return mbar_wait_bounded(bar_base + 8 * (S + s), (use - 1) & 1, kWaitBudgetNs);
      };
      while (row < end && !dead) {
        if (!wait_slot()) { dead = true; break; }
        arm(s, row, (end - row) < RB ? (end - row) : RB);
        row += RB;
        s = (s + 1 == S) ? 0 : s + 1;
        use += (s == 0);
      }
      if (trace) trace[9] = globaltimer_ns();  // static share issued
      while (!dead) {
        const long long r0 = static_cast<long long>(dyn0) + static_cast<long long>(nxt) * RB;
        if (r0 >= p.N) break;
        nxt = atomicAdd(p.next, 1u);  // one ahead: its round trip hides behind the wait for a slot
        if (!wait_slot()) { dead = true; break; }
        const int left = p.N - static_cast<int>(r0);
        arm(s, static_cast<int>(r0), left < RB ? left : RB);
        s = (s + 1 == S) ? 0 : s + 1;
        use += (s == 0);
      }
      if (trace) trace[2] = globaltimer_ns();
      // This CTA asks for no more blocks.  The last CTA to say so puts the block counter back for the
      // next launch (which asks for blocks only after this kernel has completed); the round trip
      // of the atomic is over long before the consumers are.
      __threadfence();
      const unsigned int gone = atomicInc(p.exited, static_cast<unsigned int>(G - 1));
      // end markers: one stage without rows for every consumer warp
      for (int w = 0; w < nw && !dead; ++w) {
        if (!wait_slot()) { dead = true; break; }
        meta[s] = make_int2(0, 0);
        mbar_arrive(bar_base + 8 * s);
        s = (s + 1 == S) ? 0 : s + 1;
        use += (s == 0);
      }
      if (dead) atomicExch(p.status, kStatusTimeout);
      if (gone == static_cast<unsigned int>(G - 1)) {
        __threadfence();
        atomicExch(p.next, 0u);
      }
    }
  } else {
    // ------------------------------------ consumers ------------------------------------
    // Warp w takes the CTA's stages w, w + nw, ...; S % nw == 0, so they always sit in the slots
    // w, w + nw, ... and this warp sees every phase of the barriers it waits on.
    bool dead = false;
    {
      bool ok = mbar_wait_bounded(bar_x, 0, kWaitBudgetNs * 2);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        dead = true;
        if (lane == 0) atomicExch(p.status, kStatusTimeout);
      }
    }
    {
      // all consumer threads copy x into shared memory, 16 bytes at a time (every warp passes the
      // barrier below even after a timeout)
      const int nt = nw * 32;
      const uint4* src = reinterpret_cast<const uint4*>(p.x);
      uint4* dst = reinterpret_cast<uint4*>(smem_gen);
      const int n16 = (M * K) >> 3;
      if (!dead) {
        if constexpr (WB == 1) {
          // int8 weights: even 16-byte chunks first, then the odd ones (see gemv_stage_i8)
          for (int i = threadIdx.x; i < n16; i += nt) dst[(i & 1) * (K >> 4) + (i >> 1)] = __ldg(src + i);
        } else {
          for (int i = threadIdx.x; i < n16; i += nt) dst[i] = __ldg(src + i);
        }
      }
      named_bar_sync(1, nt);
      if (trace && threadIdx.x == 0) trace[10] = globaltimer_ns();  // x is in shared memory
    }
    int s = warp;
    uint32_t ph = 0;
    unsigned long long t_wait = 0, t_work = 0;
    int n_stages = 0;
    bool first = true;
    while (!dead) {
      const unsigned long long tc0 = (trace && lane == 0) ? globaltimer_ns() : 0;
      bool ok = mbar_wait_bounded(bar_base + 8 * s, ph, kWaitBudgetNs * 2);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) {
        dead = true;
        if (lane == 0) atomicExch(p.status, kStatusTimeout);
        break;
      }
      const unsigned long long tc1 = (trace && lane == 0) ? globaltimer_ns() : 0;
      const int2 mt = meta[s];
      const int row0 = mt.x, nrows = mt.y;
      if (nrows == 0) break;
      if (trace && threadIdx.x == 0 && first) trace[3] = tc1;
      first = false;
      float out[kGemvMaxOut];
#pragma unroll
      for (int i = 0; i < kGemvMaxOut; ++i) out[i] = 0.f;
      const uint32_t wbase = ring_base + s * p.stage_bytes;
      if constexpr (WB == 1) {
        switch (RB) {
          case 1: gemv_stage_i8<1>(wbase, smem_base, K, nrows, lane, out); break;
          case 2: gemv_stage_i8<2>(wbase, smem_base, K, nrows, lane, out); break;
          case 4: gemv_stage_i8<4>(wbase, smem_base, K, nrows, lane, out); break;
          default: gemv_stage_i8<8>(wbase, smem_base, K, nrows, lane, out); break;
        }
      } else {
        switch (RB) {
          case 1: gemv_stage<M, 1>(wbase, smem_base, K, nrows, lane, out); break;
          case 2: if constexpr (2 * M <= kGemvMaxOut) gemv_stage<M, 2>(wbase, smem_base, K, nrows, lane, out); break;
          case 4: if constexpr (4 * M <= kGemvMaxOut) gemv_stage<M, 4>(wbase, smem_base, K, nrows, lane, out); break;
          default: if constexpr (8 * M <= kGemvMaxOut) gemv_stage<M, 8>(wbase, smem_base, K, nrows, lane, out); break;
        }
      }
      // the stage's bytes have been read: hand the slot back before the sums are finished
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_base + 8 * (S + s));
      // lane (m * nrows + r) keeps the sum of output (row0 + r, m): adjacent lanes, adjacent columns
      float mine = 0.f;
#pragma unroll
      for (int i = 0; i < kGemvMaxOut; ++i) {
        if (i >= RB * M) break;
        float v = out[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
        const int r = i / M, m = i - r * M;
        if (r < nrows && lane == m * nrows + r) mine = v;
      }
      if (lane < nrows * M) {
        const int m = lane / nrows, r = lane - m * nrows;
        const int n = row0 + r;
        float v = mine;
        if (WB == 1 && p.scales != nullptr) v *= __half2float(p.scales[n]);  // one scale per output channel, in fp32
        if (p.bias != nullptr) v += __half2float(p.bias[n]);
        switch (p.act) {
          case kActGeluErf: v = act_fn<kActGeluErf>(v); break;
          case kActGeluTanh: v = act_fn<kActGeluTanh>(v); break;
          case kActSilu: v = act_fn<kActSilu>(v); break;
          default: break;
        }
        if (p.residual != nullptr) v += __half2float(p.residual[static_cast<size_t>(m) * p.N + n]);
        __half* dst;
        if (p.split1 == 0) dst = p.C + static_cast<size_t>(m) * p.N + n;
        else if (n < p.split1) dst = p.C + static_cast<size_t>(m) * p.split1 + n;
        else if (n < p.split2) dst = p.C2 + static_cast<size_t>(m) * (p.split2 - p.split1) + (n - p.split1);
        else dst = p.C3 + static_cast<size_t>(m) * (p.N - p.split2) + (n - p.split2);
        *dst = __float2half_rn(v);
      }
      if (trace && lane == 0) {
        t_wait += tc1 - tc0;
        t_work += globaltimer_ns() - tc1;
        ++n_stages;
      }
      s += nw;
      if (s >= S) {
        s -= S;
        ph ^= 1;
      }
    }
    if (trace && lane == 0) {
      atomicMax(trace + 5, globaltimer_ns());  // last consumer warp done
      if (warp == 0) {
        trace[11] = t_wait;  // warp 0: waiting for its stages to land
        trace[13] = t_work;  // warp 0: multiplying and storing
        trace[6] = n_stages;
      }
    }
  }
}

}  // namespace fg
