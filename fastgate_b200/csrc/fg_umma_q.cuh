// tcgen05 kernel for the quantized ops (int8 and packed int4 weights, fp16 activations).
//
// The tensor core only takes fp16 operands from shared memory, so the packed weights cannot go
// from the TMA ring straight into tcgen05.mma as the fp16 ops do.  Eight warps stand in between:
// they read a landed stage's packed rows, dequantise them in registers and write fp16 tiles in
// the layout the TMA would have produced for an fp16 weight (K-major [128 n][64 k], rows of
// 128 B, 128B swizzle) into one of three 32 KB staging buffers, each holding 128 consecutive k of
// the 128 output columns.  Two threads (one accumulation chain each) then issue the MMAs against
// the staging buffer and the activation boxes of the stage, as fg_umma_kernel's one thread does.  With fragments and
// accumulators out of the register file, dequantisation is the only per-element work left to
// the SM's issue slots (about 13 instructions per eight int4 weights), which keeps an int4
// stream (half the bytes of int8 per weight) within what the tensor-core-free part of an SM
// can convert, where the mma.sync kernel is bound by its fragment traffic and MMA issue.
//
//   staging buffer = 128 k:  int8: one 16 KB chunk of the ring;  int4: half a chunk, i.e. exactly
//   one 128-k scale group.  Per-channel scales are applied in the fp32 epilogue as in the other
//   kernels.  Group-wise int4 scales ("group mode"): every staging buffer is accumulated into a
//   TMEM tile of its own (the MMA overwrites instead of accumulating), the epilogue warps read it
//   back as soon as it is complete and add it, times the group's scale, to fp32 sums they keep in
//   registers.  (Folding the scale into the dequantisation, one fp16 multiply per weight, was
//   measured at about 1e-2 absolute error for K of a few thousand: the whole tolerance of the
//   path for outputs near zero.)
//
// Warp roles: 0-3 epilogue, 4 producer (TMA), 5 MMA issue and TMEM allocation, 6-9 finishers
// (the four warps serve both of a CTA's partial tiles, one after the other), 10-17 dequantise,
// 18 second MMA issuer (the tensor core takes MMAs from several threads; one thread alone spends
// about 50 ns per instruction, which at 16 token columns per MMA is the kernel's bottleneck).
#pragma once
#include "fg_layout.h"
#include "fg_umma.cuh"

namespace fg {

constexpr int kUmmaQDequantWarps = 8;
constexpr int kUmmaQIssuers = 2;  // MMA-issuing threads, one accumulation chain each
constexpr int kUmmaQThreads = (6 + kUmmaMT / 4 + kUmmaQDequantWarps + (kUmmaQIssuers - 1)) * 32;  // 608
constexpr uint32_t kStagingBytes = 32768;  // fp16 [128 n][128 k]: two K-major sub-tiles of 16 KB
constexpr int kNStaging = FG_UMMA_Q_STAGING_BYTES / 32768;  // staging buffers in flight between the dequantisers and the MMA thread
constexpr uint32_t kTmemColsQ = 128;  // kNStaging accumulator tiles of 2 chains x 16 columns (group mode), rounded up
static_assert(kNStaging * kUmmaChains * kUmmaMT <= 128, "group mode keeps one accumulator tile per staging buffer");

__device__ __forceinline__ void sts_v4(uint32_t addr, uint32_t r0, uint32_t r1, uint32_t r2, uint32_t r3) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(r0), "r"(r1), "r"(r2), "r"(r3) : "memory");
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// Eight unsigned 4-bit weights of one word (nibble i = element i) to four half2 in element
// order, minus the zero point (`magic` = half2(1024 + zero_point), see dequant_u4x8).
__device__ __forceinline__ void dequant_u4x8_ordered(uint32_t w, uint32_t magic, uint32_t (&out)[4]) {
  const uint32_t even = w & 0x0F0F0F0Fu;         // bytes: elements 0, 2, 4, 6
  const uint32_t odd = (w >> 4) & 0x0F0F0F0Fu;   // bytes: elements 1, 3, 5, 7
  const uint32_t lo = prmt(even, odd, 0x5140);   // bytes: elements 0, 1, 2, 3
  const uint32_t hi = prmt(even, odd, 0x7362);   // bytes: elements 4, 5, 6, 7
  const uint32_t e64 = 0x64646464u;
  uint32_t v[4] = {prmt(lo, e64, 0x5140), prmt(lo, e64, 0x5342), prmt(hi, e64, 0x5140), prmt(hi, e64, 0x5342)};
#pragma unroll
  for (int i = 0; i < 4; ++i) asm("sub.f16x2 %0, %1, %2;" : "=r"(out[i]) : "r"(v[i]), "r"(magic));
}

template <int OP>
__global__ void __launch_bounds__(kUmmaQThreads, 1)
    fg_umma_q_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                     const KParams p) {
  static_assert(OP == kOpW8A16NK || OP == kOpW4A16NK, "quantized weights only");
  using T = OpTraits<OP>;
  constexpr int MT = kUmmaMT;
  constexpr int kHalves = T::chunkK / 128;  // staging buffers per ring chunk: int8 1, int4 2
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const int S = p.stages;
  const int cps = p.chunks_per_stage;
  constexpr int cbytes = chunk_bytes(OP, MT);
  const uint32_t stage_bytes = cps * cbytes;
  const uint32_t ring_bytes = S * stage_bytes;
  const uint32_t staging = smem_base + ring_bytes;              // [kNStaging] x 32 KB, 1 KB aligned
  const uint32_t bar_base = staging + kNStaging * kStagingBytes;  // full[S], empty[S]
  const uint32_t bar_acc_full = bar_base + 16 * S;              // [2] MMA -> epilogue
  const uint32_t bar_acc_empty = bar_acc_full + 16;             // [2] epilogue -> MMA
  const uint32_t bar_flush = bar_acc_empty + 16;                // [2] epilogue -> finishers (per partial)
  const uint32_t bar_a_full = bar_flush + 16;                   // [kNStaging] dequantisers -> MMA
  const uint32_t bar_a_empty = bar_a_full + 8 * kNStaging;      // [kNStaging] MMA -> dequantisers (and, in group mode, -> epilogue)
  const uint32_t bar_g_empty = bar_a_empty + 8 * kNStaging;     // [kNStaging] group mode: epilogue -> MMA (accumulator tile read back)
  const uint32_t tmem_slot = bar_g_empty + 8 * kNStaging;
  const uint32_t tail = ring_bytes + kNStaging * kStagingBytes + 16 * S;
  constexpr uint32_t kBarBytes = 48 + 24 * kNStaging;           // the barriers after full[] / empty[]
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + tail + kBarBytes);
  volatile uint32_t* prev_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + tail + kBarBytes + 4);  // [2]
  static_assert(kBarBytes + 16 <= 160, "barrier block outgrew its reservation (fg_umma_q_smem_bytes)");

  if (blockDim.x != static_cast<unsigned>(kUmmaQThreads) || dynamic_smem_size() < 1023u + tail + 160u) {
    if (threadIdx.x == 0) atomicExch(p.status, kStatusBadLaunch);
    return;
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  unsigned long long* trace = p.trace ? p.trace + kTraceSlots * blockIdx.x : nullptr;
  if (trace && threadIdx.x == 0) {
    trace[0] = globaltimer_ns();
    trace[12] = smid();
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_base + 8 * s, 1);
      mbar_init(bar_base + 8 * (S + s), kUmmaQIssuers);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, kUmmaQIssuers);
      mbar_init(bar_acc_empty + 8 * b, 4);
      mbar_init(bar_flush + 8 * b, 128);
    }
    for (int b = 0; b < kNStaging; ++b) {
      mbar_init(bar_a_full + 8 * b, kUmmaQDequantWarps * 32);
      mbar_init(bar_a_empty + 8 * b, kUmmaQIssuers);
      mbar_init(bar_g_empty + 8 * b, 4);
    }
    fence_mbar_init();
    fence_proxy_async();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, kTmemColsQ);
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
  const bool gmode = (OP == kOpW4A16NK) && p.scale_groups > 1;  // one accumulator tile per 128-k group

  if (warp == 4) {
    if (lane == 0) run_producer<OP, MT>(tmW, tmX, p, range, smem_base, bar_base, S, cps, trace);
    return;
  }
  if (warp >= 6 && warp < 10) {
    // one set of warps for both partial tiles of the CTA: the first, then the second
    run_finisher<OP, MT>(p, range, bar_flush, prev_slot, 0, warp - 6, lane, trace);
    run_finisher<OP, MT>(p, range, bar_flush, prev_slot, 1, warp - 6, lane, trace);
    return;
  }

  if (warp >= 10 && warp < 10 + kUmmaQDequantWarps) {
    // ------------------------------------ dequantise ------------------------------------
    // Thread d converts 64 k of one weight row per staging buffer: row = d % 128, k half = d / 128.
    // Consecutive lanes take consecutive rows, whose 16-byte pieces the swizzle spreads over
    // all banks, for the packed reads as for the fp16 writes.
    const int d = threadIdx.x - 10 * 32;
    const int row = d & 127, khalf = d >> 7;
    const uint32_t sw = static_cast<uint32_t>(row & 7);
    uint32_t u = ub;
    int s = 0;
    uint32_t ph = 0;
    uint32_t buf = 0, bph = 0;  // staging buffer in turn and the parity of its use count
    bool dead = false;
    while (u < ue && !dead) {
      const uint32_t tile = u / KB;
      const int kb0 = static_cast<int>(u - tile * KB);
      const int len = static_cast<int>((KB - kb0) < (ue - u) ? (KB - kb0) : (ue - u));
      for (int it = 0; it < len && !dead; ++it, s = (s + 1 == S) ? 0 : s + 1, ph ^= (s == 0)) {
        const int k0 = (kb0 + it) * k_per_stage;
        int nch = (p.K - k0 + T::chunkK - 1) / T::chunkK;
        nch = nch < cps ? nch : cps;
        if (!mbar_wait_bounded(bar_base + 8 * s, ph, kWaitBudgetNs * 2)) {
          dead = true;
          break;
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) {  // at most four chunks per stage; unrolled so that gs[] stays in registers
          if (c >= nch || dead) break;
          const uint32_t src_row = smem_base + s * stage_bytes + c * cbytes + row * 128;
#pragma unroll
          for (int hf = 0; hf < kHalves; ++hf) {
            if (!mbar_wait_bounded(bar_a_empty + 8 * buf, bph ^ 1, kWaitBudgetNs * 2)) {
              dead = true;
              break;
            }
            const uint32_t dst_row = staging + buf * kStagingBytes + khalf * 16384 + row * 128;
            if constexpr (OP == kOpW4A16NK) {
#pragma unroll
              for (int pc = 0; pc < 2; ++pc) {
                const uint32_t piece = hf * 4 + khalf * 2 + pc;
                uint32_t w[4];
                lds_v4(src_row + ((piece ^ sw) << 4), w[0], w[1], w[2], w[3]);
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) {
                  uint32_t o[4];
                  dequant_u4x8_ordered(w[wi], p.w4_magic, o);
                  sts_v4(dst_row + (((pc * 4 + wi) ^ sw) << 4), o[0], o[1], o[2], o[3]);
                }
              }
            } else {
#pragma unroll
              for (int pc = 0; pc < 4; ++pc) {
                const uint32_t piece = khalf * 4 + pc;
                uint32_t w[4];
                lds_v4(src_row + ((piece ^ sw) << 4), w[0], w[1], w[2], w[3]);
                uint32_t o[8];
#pragma unroll
                for (int wi = 0; wi < 4; ++wi) dequant_s8x4(w[wi], o[2 * wi], o[2 * wi + 1]);
                sts_v4(dst_row + (((pc * 2) ^ sw) << 4), o[0], o[1], o[2], o[3]);
                sts_v4(dst_row + (((pc * 2 + 1) ^ sw) << 4), o[4], o[5], o[6], o[7]);
              }
            }
            fence_proxy_async();  // these generic-proxy writes are read by the tensor core
            mbar_arrive(bar_a_full + 8 * buf);
            if (++buf == kNStaging) {
              buf = 0;
              bph ^= 1;
            }
          }
        }
      }
      u += len;
    }
    if (dead && lane == 0) atomicExch(p.status, kStatusTimeout);
    return;
  }

  if (warp == 5 || warp >= 10 + kUmmaQDequantWarps) {
    // ------------------------------------ MMA issue ------------------------------------
    // Issuer i owns accumulation chain i (its own TMEM columns) and the k16 steps i, i + 2 of
    // every 64-k sub-tile; the issuers never touch the same accumulator, so nothing orders them
    // against each other, and every hand-off barrier counts one commit per issuer.
    const int iss = (warp == 5) ? 0 : warp - (10 + kUmmaQDequantWarps) + 1;
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(false);
      constexpr uint64_t a_hi = umma_smem_desc(0, 1, 64);
      constexpr uint64_t b_hi = umma_smem_desc(0, 1, 64);
      uint32_t u = ub;
      uint32_t sg = 0;
      uint32_t buf = 0, bph = 0;
      bool dead = false;
      int s = 0;
      while (u < ue && !dead) {
        const uint32_t tile = u / KB;
        const int kb0 = static_cast<int>(u - tile * KB);
        const int len = static_cast<int>((KB - kb0) < (ue - u) ? (KB - kb0) : (ue - u));
        const uint32_t b = sg & 1, use = sg >> 1;
        if (!gmode && !mbar_wait_bounded(bar_acc_empty + 8 * b, (use & 1) ^ 1, kWaitBudgetNs * 2)) {
          dead = true;
          break;
        }
        tc_fence_after_sync();
        uint32_t tmem_d = tmem_base + b * (kUmmaChains * kUmmaMT) + iss * kUmmaMT;
        uint32_t acc_flag = 0;
        for (int it = 0; it < len && !dead; ++it, s = (s + 1 == S) ? 0 : s + 1) {
          const int k0 = (kb0 + it) * k_per_stage;
          int nch = (p.K - k0 + T::chunkK - 1) / T::chunkK;
          nch = nch < cps ? nch : cps;
          if (trace && iss == 0 && it == 0 && u == ub) trace[3] = globaltimer_ns();
          for (int c = 0; c < nch && !dead; ++c) {
            const uint32_t xb = smem_base + s * stage_bytes + c * cbytes + kChunkWBytes;
#pragma unroll
            for (int hf = 0; hf < kHalves; ++hf) {
              // the staging buffer is complete, which also says that the stage (and with it the
              // activation boxes) has landed: the dequantisers waited for it
              if (!mbar_wait_bounded(bar_a_full + 8 * buf, bph, kWaitBudgetNs * 2)) {
                dead = true;
                break;
              }
              if (gmode) {
                // this group's accumulator tile: free once the epilogue has read its previous content
                if (!mbar_wait_bounded(bar_g_empty + 8 * buf, bph ^ 1, kWaitBudgetNs * 2)) {
                  dead = true;
                  break;
                }
                tmem_d = tmem_base + buf * (kUmmaChains * kUmmaMT) + iss * kUmmaMT;
                acc_flag = 0;
              }
              tc_fence_after_sync();
              const uint32_t ab = staging + buf * kStagingBytes;
#pragma unroll
              for (int t2 = 0; t2 < 2; ++t2) {  // two 64-k sub-tiles, one activation box each
                const uint64_t a0 = a_hi | ((ab + t2 * 16384) >> 4);
                const uint64_t b0 = b_hi | ((xb + (hf * 2 + t2) * (MT * 128)) >> 4);
                umma_f16(tmem_d, a0 + 2 * iss, b0 + 2 * iss, idesc, acc_flag);
                umma_f16(tmem_d, a0 + 2 * iss + 4, b0 + 2 * iss + 4, idesc, 1u);
                acc_flag = 1u;
              }
              umma_commit(bar_a_empty + 8 * buf);
              if (++buf == kNStaging) {
                buf = 0;
                bph ^= 1;
              }
            }
          }
          if (dead) break;
          umma_commit(bar_base + 8 * (S + s));  // the ring slot is free once these MMAs have read its activations
        }
        if (dead) break;
        if (!gmode) umma_commit(bar_acc_full + 8 * b);
        if (trace && iss == 0) trace[4] = globaltimer_ns();
        ++sg;
        u += len;
      }
      if (dead) atomicExch(p.status, kStatusTimeout);
    }
    __syncwarp();
    if (warp != 5) return;  // warp 5 stays for the teardown (it owns the TMEM allocation)
  } else {
    // ------------------------------------ epilogue warps 0-3 ------------------------------------
    const int n_in_tile = warp * 32 + lane;
    uint32_t u = ub;
    uint32_t sg = 0, ev = 0;
    uint32_t buf = 0, bph = 0;  // group mode: accumulator tile in turn (= staging buffer) and its parity
    bool dead = false;
    while (u < ue) {
      const uint32_t tile = u / KB;
      const uint32_t kb0 = u - tile * KB;
      const uint32_t len = (KB - kb0) < (ue - u) ? (KB - kb0) : (ue - u);
      const bool whole = (len == KB);
      const uint32_t b = sg & 1, use = sg >> 1;
      uint32_t r[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = 0;
      if (gmode) {
        // one accumulator tile per 128-k group: read each back as it completes and add it, times
        // the group's scale, to the running fp32 sums of this thread's output column
        float acc[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = 0.f;
        const __half* srow = p.scales + static_cast<size_t>(tile * kTileN + n_in_tile) * p.scale_groups;
        for (uint32_t it = 0; it < len; ++it) {
          const int k0 = static_cast<int>(kb0 + it) * k_per_stage;
          int nch = (p.K - k0 + T::chunkK - 1) / T::chunkK;
          nch = nch < cps ? nch : cps;
          const int ngroups = nch * kHalves;
          __half gs[4 * kHalves];  // the stage's scales, requested before its first tile is waited for
#pragma unroll
          for (int i = 0; i < 4 * kHalves; ++i) {
            int gi = (k0 >> 7) + i;
            gi = gi < p.scale_groups ? gi : p.scale_groups - 1;
            gs[i] = (i < ngroups) ? __ldg(srow + gi) : __half(0.f);
          }
#pragma unroll
          for (int i = 0; i < 4 * kHalves; ++i) {
            if (i >= ngroups) break;
            if (!dead) {
              bool ok = mbar_wait_bounded(bar_a_empty + 8 * buf, bph, kWaitBudgetNs * 4);
              ok = __all_sync(0xffffffffu, ok);
              if (!ok) {
                dead = true;
                if (lane == 0) atomicExch(p.status, kStatusTimeout);
              }
            }
            if (!dead) {
              uint32_t q[32];
              tc_fence_after_sync();
              tmem_ld32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + buf * (kUmmaChains * kUmmaMT), q);
              tmem_ld_wait();
              tc_fence_before_sync();
              __syncwarp();
              if (lane == 0) mbar_arrive(bar_g_empty + 8 * buf);
              const float sc = __half2float(gs[i]);
#pragma unroll
              for (int m = 0; m < MT; ++m) acc[m] += (__uint_as_float(q[m]) + __uint_as_float(q[MT + m])) * sc;
            }
            if (++buf == kNStaging) {
              buf = 0;
              bph ^= 1;
            }
          }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) r[m] = __float_as_uint(acc[m]);
      } else if (!dead) {
        bool ok = mbar_wait_bounded(bar_acc_full + 8 * b, use & 1, kWaitBudgetNs * 4);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          dead = true;
          if (lane == 0) atomicExch(p.status, kStatusTimeout);
        }
      }
      if (!gmode && !dead) {
        tc_fence_after_sync();
        tmem_ld32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + b * (kUmmaChains * kUmmaMT), r);
        tmem_ld_wait();
#pragma unroll
        for (int m = 0; m < MT; ++m) r[m] = __float_as_uint(__uint_as_float(r[m]) + __uint_as_float(r[MT + m]));
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty + 8 * b);
      }
      const int n = tile * kTileN + n_in_tile;
      if (whole) {
        with_act(p.act, [&](auto tag) {
          constexpr int ACT = decltype(tag)::value;
#pragma unroll
          for (int m = 0; m < MT; ++m)
            if (m < p.M) store_out1<OP, ACT>(p, m, n, __uint_as_float(r[m]));
        });
      } else {
        const int slot = (u == ub) ? 0 : 1;
        float* mypart = p.partials + (static_cast<size_t>(blockIdx.x) * 2 + slot) * (MT * kTileN);
#pragma unroll
        for (int m = 0; m < MT; ++m) mypart[m * kTileN + n_in_tile] = __uint_as_float(r[m]);
        mbar_arrive(bar_flush + 8 * ev);
        ++ev;
      }
      if (trace && threadIdx.x == 0) trace[6] += 1;
      ++sg;
      u += len;
    }
  }

  tc_fence_before_sync();
  named_bar_sync(2, 160);
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemColsQ);
  }
}

}  // namespace fg
