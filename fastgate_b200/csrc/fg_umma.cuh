// tcgen05 (5th-generation tensor core) variant of the stream-K kernel for the fp16 ops.
//
// Same work split, producer, ring, finisher and workspace protocol as fg_streamk_kernel; only
// the math differs.  One thread issues tcgen05.mma instructions that read the 128B-swizzled
// weight and activation tiles straight from shared memory and accumulate a 128 (output
// columns) x 16 (token rows) fp32 tile in tensor memory (TMEM), so no warp spends issue slots
// or registers on fragments and there is no cross-warp reduction: a tile segment's K range is
// accumulated in place.  Two TMEM accumulators alternate, so the epilogue of one segment
// (tcgen05.ld, 32 lanes x 32 columns per warp) overlaps the MMAs of the next.
//
//   swap-AB:  D[n, m] (+)= sum_k W[n, k] * x[m, k]      UMMA M = 128, N = 16, K = 16 per instruction
//   NxK weight: A operand K-major  (tile [128 n][64 k], rows of 128 B)
//   KxN weight: A operand MN-major (two boxes [64 k][64 n], rows of 128 B)
//   x tile [16 m][64 k]: B operand K-major; rows >= M are zero-filled by the TMA
//
// Warp roles: 0-3 epilogue (TMEM lane quadrant = warp), 4 producer (TMA), 5 MMA issue and
// TMEM allocation, 6-9 finishers.
#pragma once
#include "fg_kernels.cuh"

namespace fg {

constexpr int kUmmaMT = 16;            // token rows of the accumulator (UMMA N) of the grouped, chained and quantized kernels
constexpr int kUmmaThreads = (6 + 2 * 4) * 32;             // two finisher teams of four warps (see run_finisher)
constexpr int kUmmaGroupThreads = (6 + kUmmaMT / 4) * 32;  // grouped and chained kernels: one team
constexpr int kUmmaChains = 2;         // independent accumulation chains per tile (summed in the epilogue)
constexpr uint32_t kTmemCols = 64;     // 2 buffers x 2 chains x 16 columns (16-row kernels)
constexpr uint32_t kGateXchBytes = 16 * kTileN * 4;  // SiLU gate: the epilogue's swap buffer

// ---- tcgen05 wrappers ------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_slot), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]; accumulate == 0 overwrites D.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// The mbarrier gets one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
               : "memory");
}
// 32 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor, 128B swizzle (layout type 2), descriptor version 1.
// Addresses and offsets in units of 16 bytes.
__host__ __device__ constexpr uint64_t umma_smem_desc(uint32_t smem_addr, uint32_t lbo16, uint32_t sbo16) {
  return static_cast<uint64_t>((smem_addr >> 4) & 0x3FFFu) | (static_cast<uint64_t>(lbo16 & 0x3FFFu) << 16) |
         (static_cast<uint64_t>(sbo16 & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor, kind::f16: fp16 A and B, fp32 D, M = 128, N = 16, B K-major,
// A K-major (NxK weight) or MN-major (KxN weight).
__host__ __device__ constexpr uint32_t umma_idesc(bool a_mn_major, int n = kUmmaMT) {
  return (1u << 4) | ((a_mn_major ? 1u : 0u) << 15) | ((static_cast<uint32_t>(n) >> 3) << 17) | ((kTileN >> 4) << 24);
}
// 16 consecutive 32-bit columns of this thread's TMEM lane.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// One output element of row m, column n (scale, round, store; push-aware like store_out2).
template <int OP, int ACT>
__device__ __forceinline__ void store_out1(const KParams& p, int m, int n, float v) {
  if ((OP == kOpW8A16NK || (OP == kOpW4A16NK && p.scale_groups <= 1)) && p.scales != nullptr)
    v *= __half2float(p.scales[n]);  // one scale per output channel, applied in fp32
  if (ACT != kActNone || p.bias != nullptr || p.residual != nullptr) v = epilogue1<ACT>(p, m, n, v);
  const __half h = __float2half_rn(v);
  if (p.world == 0) {
    *out_ptr(p, m, n) = h;
  } else if (p.mc_C != nullptr) {
    // multicast stores are at least 32 bits wide: even lanes store their column and the next one
    // (called by whole warps with a uniform m: lane = column within the tile)
    const unsigned short mine = __half_as_ushort(h);
    const unsigned int next = __shfl_down_sync(0xffffffffu, static_cast<unsigned int>(mine), 1);
    if ((n & 1) == 0)
      multimem_st_b32(p.mc_C + static_cast<size_t>(m) * p.ldc + p.col0 + n, static_cast<uint32_t>(mine) | (next << 16));
  } else {
    const size_t off = static_cast<size_t>(m) * p.ldc + p.col0 + n;
    for (int q = 0; q < p.world; ++q) p.peer_C[q][off] = h;
  }
}

// MT = token rows of the accumulator = N of the MMA instruction: 16, 32 or 64.  Up to 64 rows of
// activations ride along with one pass over the weight; the instruction count, and with it the
// issuing thread's time, does not depend on MT.
template <int OP, int MT>
__global__ void __launch_bounds__(kUmmaThreads, 1)
    fg_umma_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                   const KParams p) {
  static_assert(OP == kOpF16KN || OP == kOpF16NK, "tcgen05 path: fp16 weights only");
  static_assert(MT == 16 || MT == 32 || MT == 64, "accumulator height");
  using T = OpTraits<OP>;
  constexpr uint32_t kCols = 2 * kUmmaChains * MT;  // TMEM columns: 2 buffers x 2 chains x MT (64, 128 or 256)
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const int S = p.stages;
  const int cps = p.chunks_per_stage;
  constexpr int cbytes = chunk_bytes(OP, MT);
  const uint32_t stage_bytes = cps * cbytes;
  const uint32_t ring_bytes = S * stage_bytes;
  const uint32_t bar_base = smem_base + ring_bytes;         // full[S], empty[S]
  const uint32_t bar_acc_full = bar_base + 16 * S;          // [2] MMA -> epilogue
  const uint32_t bar_acc_empty = bar_acc_full + 16;         // [2] epilogue -> MMA
  const uint32_t bar_flush = bar_acc_empty + 16;            // [2] epilogue -> finisher team
  const uint32_t tmem_slot = bar_flush + 16;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + ring_bytes + 16 * S + 48);
  volatile uint32_t* prev_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + ring_bytes + 16 * S + 52);  // [2]
  // SiLU gate: 16 x 128 floats through which the epilogue warps swap gate and up sums
  float* gate_xch = reinterpret_cast<float*>(smem_gen + ring_bytes + 16 * S + 64);
  const bool gated = (p.act == kActSiluGate);

  // refuse a launch that does not fit the parameters (see fg_streamk_kernel)
  if (blockDim.x != static_cast<unsigned>(kUmmaThreads) ||
      dynamic_smem_size() < 1023u + ring_bytes + 16u * S + 64u + (gated ? kGateXchBytes : 0u)) {
    if (threadIdx.x == 0) atomicExch(p.status, kStatusBadLaunch);
    return;
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  unsigned long long* trace = p.trace ? p.trace + kTraceSlots * blockIdx.x : nullptr;
  if (trace && threadIdx.x == 0) trace[0] = globaltimer_ns();
  if (trace && threadIdx.x == 0) trace[12] = smid();                     // which SM ran this CTA

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_base + 8 * s, 1);        // full: the producer's expect_tx arrive
      mbar_init(bar_base + 8 * (S + s), 1);  // empty: one tcgen05.commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);    // one tcgen05.commit
      mbar_init(bar_acc_empty + 8 * b, 4);   // lane 0 of each epilogue warp
    }
    mbar_init(bar_flush, 128);
    mbar_init(bar_flush + 8, 128);
    fence_mbar_init();
    fence_proxy_async();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, kCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;

  const uint32_t KB = p.k_blocks;
  const uint32_t total = static_cast<uint32_t>(p.tiles) * KB;
  const uint32_t G = gridDim.x;
  const CtaRange range{KB, total, G, range_begin(blockIdx.x, total, G), range_begin(blockIdx.x + 1, total, G)};
  const uint32_t ub = range.ub, ue = range.ue;
  const int k_per_stage = cps * T::chunkK;

  if (warp == 4) {
    if (lane == 0) run_producer<OP, MT>(tmW, tmX, p, range, smem_base, bar_base, S, cps, trace);
    return;
  }
  if (warp >= 6) {
    run_finisher<OP, MT>(p, range, bar_flush, prev_slot, (warp - 6) / finisher_warps<MT>(),
                         (warp - 6) % finisher_warps<MT>(), lane, trace);
    return;
  }

  if (warp == 5) {
    // ------------------------------------ MMA issue ------------------------------------
    // One thread does everything here: it waits for a stage to land, issues the stage's
    // MMAs (asynchronous: they queue up behind each other in the tensor core) and commits
    // them to the slot's empty barrier.  The mbarrier wait orders the TMA's writes before
    // the MMA's reads; tcgen05 fences are only needed around the accumulator hand-off.
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(OP == kOpF16KN, MT);
      uint32_t u = ub;
      int it0 = 0;
      uint32_t sg = 0;
      bool dead = false;
      int s = 0;        // ring slot and phase of the next stage, advanced by increments
      uint32_t ph = 0;
      while (u < ue && !dead) {
        const uint32_t tile = u / KB;
        const int kb0 = static_cast<int>(u - tile * KB);
        const int len = static_cast<int>((KB - kb0) < (ue - u) ? (KB - kb0) : (ue - u));
        const uint32_t b = sg & 1, use = sg >> 1;
        if (!mbar_wait_bounded(bar_acc_empty + 8 * b, (use & 1) ^ 1, kWaitBudgetNs)) {
          dead = true;
          break;
        }
        tc_fence_after_sync();
        // Even and odd k16 steps accumulate into two separate TMEM tiles: consecutive MMAs
        // then do not wait for each other's accumulator; the epilogue adds the two.
        const uint32_t tmem_d = tmem_base + b * (kUmmaChains * MT);
        for (int it = it0; it < it0 + len; ++it, s = (s + 1 == S) ? 0 : s + 1, ph ^= (s == 0)) {
          const unsigned long long tw0 = trace ? globaltimer_ns() : 0;
          if (!mbar_wait_bounded(bar_base + 8 * s, ph, kWaitBudgetNs)) {
            dead = true;
            break;
          }
          const unsigned long long tw1 = trace ? globaltimer_ns() : 0;
          if (trace) trace[9] += tw1 - tw0;                   // waiting for the stage to land
          if (trace && it == 0) trace[3] = tw1;               // first stage landed
          const int k0 = (kb0 + (it - it0)) * k_per_stage;
          int nch = (p.K - k0 + T::chunkK - 1) / T::chunkK;
          nch = nch < cps ? nch : cps;
          // Descriptors differ only in their start-address field (bits 0-13, in 16-byte units;
          // shared-memory addresses stay below 2^18), so a chunk's descriptor is one OR and
          // each k16 step one add: this thread is alone in issuing and its instruction
          // latency, not the tensor core, bounds the rate.
          // K-major: a k16 step is 32 bytes further along the 128-byte rows (8-row groups
          // 1024 B apart).  MN-major: it is sixteen 128-byte k-rows = 2048 B further; the
          // two 64-column boxes are 8192 B apart (LBO), 8-row k-groups 1024 B (SBO).
          constexpr uint64_t a_hi = (OP == kOpF16NK) ? umma_smem_desc(0, 1, 64) : umma_smem_desc(0, 512, 64);
          constexpr uint64_t b_hi = umma_smem_desc(0, 1, 64);
          constexpr uint64_t a_step = (OP == kOpF16NK) ? 2 : 128;
          uint32_t wb = smem_base + s * stage_bytes;
          uint32_t acc_flag = (it > it0) ? 1u : 0u;
          for (int c = 0; c < nch; ++c) {
            const uint64_t a0 = a_hi | (wb >> 4);
            const uint64_t b0 = b_hi | ((wb + kChunkWBytes) >> 4);
            umma_f16(tmem_d, a0, b0, idesc, acc_flag);
            umma_f16(tmem_d + MT, a0 + a_step, b0 + 2, idesc, acc_flag);
            umma_f16(tmem_d, a0 + 2 * a_step, b0 + 4, idesc, 1u);
            umma_f16(tmem_d + MT, a0 + 3 * a_step, b0 + 6, idesc, 1u);
            acc_flag = 1u;
            wb += cbytes;
          }
          umma_commit(bar_base + 8 * (S + s));  // the slot is free once these MMAs have read it
          if (trace) trace[10] += globaltimer_ns() - tw1;     // issuing
        }
        if (dead) break;
        umma_commit(bar_acc_full + 8 * b);
        if (trace) trace[4] = globaltimer_ns();  // last MMA of the segment issued
        ++sg;
        u += len;
        it0 += len;
      }
      if (dead) atomicExch(p.status, kStatusTimeout);
    }
    __syncwarp();
  } else {
    // ------------------------------------ epilogue warps 0-3 ------------------------------------
    const int n_in_tile = warp * 32 + lane;  // TMEM lane = output column within the tile
    uint32_t u = ub;
    uint32_t sg = 0, ev = 0;
    bool dead = false;
    while (u < ue) {
      const uint32_t tile = u / KB;
      const uint32_t kb0 = u - tile * KB;
      const uint32_t len = (KB - kb0) < (ue - u) ? (KB - kb0) : (ue - u);
      const bool whole = (len == KB);
      const uint32_t b = sg & 1, use = sg >> 1;
      const unsigned long long te0 = (trace && threadIdx.x == 0) ? globaltimer_ns() : 0;
      if (!dead) {
        bool ok = mbar_wait_bounded(bar_acc_full + 8 * b, use & 1, kWaitBudgetNs * 2);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          dead = true;
          if (lane == 0) atomicExch(p.status, kStatusTimeout);
        }
      }
      if (!dead) tc_fence_after_sync();
      const int n = tile * kTileN + n_in_tile;
      const int slot = (u == ub) ? 0 : 1;
      float* mypart = p.partials + (static_cast<size_t>(blockIdx.x) * 2 + slot) * (MT * kTileN);
      const uint32_t tbase = tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + b * (kUmmaChains * MT);
      // sixteen token rows at a time: the two chains' columns, summed, then stored or parked
#pragma unroll
      for (int mg = 0; mg < MT / 16; ++mg) {
        uint32_t r[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) r[i] = 0;
        if (!dead) {
          if constexpr (MT == 16) {
            uint32_t q[32];
            tmem_ld32(tbase, q);
            tmem_ld_wait();
#pragma unroll
            for (int m = 0; m < 16; ++m) r[m] = __float_as_uint(__uint_as_float(q[m]) + __uint_as_float(q[16 + m]));
          } else {
            uint32_t q0[16], q1[16];
            tmem_ld16(tbase + mg * 16, q0);
            tmem_ld16(tbase + MT + mg * 16, q1);
            tmem_ld_wait();
#pragma unroll
            for (int m = 0; m < 16; ++m) r[m] = __float_as_uint(__uint_as_float(q0[m]) + __uint_as_float(q1[m]));
          }
          if (mg == MT / 16 - 1) {
            tc_fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_acc_empty + 8 * b);  // the MMA warp may reuse this accumulator
          }
        }
        if (trace && threadIdx.x == 0 && mg == MT / 16 - 1) {
          trace[7] = globaltimer_ns();  // accumulator read back
          trace[11] += trace[7] - te0;  // waiting for it
        }
        if (whole && gated) {
          // warps 0-1 hold the gate rows of the tile, warps 2-3 the up rows: swap through shared
          // memory (every epilogue thread takes both barriers, whatever its own state)
#pragma unroll
          for (int m = 0; m < 16; ++m) gate_xch[m * kTileN + n_in_tile] = __uint_as_float(r[m]);
          named_bar_sync(1, 128);
          if (n_in_tile < 64) {
#pragma unroll
            for (int m = 0; m < 16; ++m)
              if (mg * 16 + m < p.M)
                store_gate(p, mg * 16 + m, tile, n_in_tile, __uint_as_float(r[m]), gate_xch[m * kTileN + 64 + n_in_tile]);
          }
          named_bar_sync(1, 128);
        } else if (whole) {
          with_act(p.act, [&](auto tag) {
            constexpr int ACT = decltype(tag)::value;
#pragma unroll
            for (int m = 0; m < 16; ++m)
              if (mg * 16 + m < p.M) store_out1<OP, ACT>(p, mg * 16 + m, n, __uint_as_float(r[m]));
          });
        } else {
#pragma unroll
          for (int m = 0; m < 16; ++m) mypart[(mg * 16 + m) * kTileN + n_in_tile] = __uint_as_float(r[m]);
        }
      }
      if (whole) {
        if (p.world > 0) {
          named_bar_sync(1, 128);  // all four warps have issued the tile's stores
          if (threadIdx.x == 0) signal_tile_delivered(p);
        }
      } else {
        mbar_arrive(bar_flush + 8 * ev);
        ++ev;
      }
      if (trace && threadIdx.x == 0) trace[6] += 1;
      ++sg;
      u += len;
    }
  }

  // ---- teardown: TMEM goes back once the epilogue warps have read their last accumulator ----
  tc_fence_before_sync();
  named_bar_sync(2, 160);
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kCols);
  }
}

}  // namespace fg
