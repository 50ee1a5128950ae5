// Grouped launch of the tcgen05 kernel: many independent fp16 problems
// C_i[M_i, N_i] = x_i[M_i, K_i] . W_i^T (M_i <= 16), one persistent kernel.
//
// The stages of all problems are concatenated into one work list and dealt to the CTAs in
// equal contiguous ranges, exactly as fg_umma_kernel does for one problem: a CTA streams
// through problem boundaries without draining its ring, the fixed cost of a launch (prologue,
// DRAM ramp, tail of split tiles) is paid once per group instead of once per problem, and the
// split of every output tile is still reduced in CTA order (bit-reproducible).  This is what
// a stack of projections with independent inputs (the DiT linear stack) wants; layers that
// feed each other must stay separate launches.
//
// The problems are described by a table in global memory (one GroupEntry each, with the
// problem's two tensor maps), written by the host when the group is created.
#pragma once
#include "fg_umma.cuh"

namespace fg {

struct alignas(128) GroupEntry {
  CUtensorMap tmW;            // weight [N, K] (NxK op) or [K, N] (KxN op), 128B swizzle
  CUtensorMap tmX;            // activations [M, K], box of 16 rows
  __half* C;                  // local output [M, N]            (world == 0)
  __half* peer_C[kMaxPeers];  // full outputs [M, ldc] of every rank (world > 0)
  __half* mc_C;               // multicast mapping of those outputs, or nullptr
  long long ldc;
  int col0;                   // first column of this rank's slice in the full output
  int M, N, K;
  uint32_t KB;                // stages per output tile
  uint32_t tiles;             // N / 128
  uint32_t unit_begin;        // first stage of this problem in the concatenated list
  uint32_t tile_begin;        // first output tile of this problem (ticket index)
};

struct GParams {
  const GroupEntry* table;
  int count;
  uint32_t total_units;
  float* partials;
  unsigned int* tickets;
  int* status;
  unsigned long long* trace;
  int chunks_per_stage;
  int stages;
  int world;                  // 0: local outputs
  int rank;
  unsigned long long* peer_flag[kMaxPeers];
  unsigned long long* mc_flag;  // multicast mapping of the flag arrays: tiles go out by multimem.st / multimem.red
  unsigned long long* target_dev;  // optional: this rank's running total of tiles per source; a run adds total_tiles
  uint32_t total_tiles;
};

// Position of one stage of the concatenated list.
struct Cursor {
  int pi;
  const GroupEntry* e;
  uint32_t KB, tiles, tile, kb;
};

__device__ __forceinline__ void cursor_load(const GParams& g, Cursor& c, int pi) {
  c.pi = pi;
  c.e = g.table + pi;
  c.KB = c.e->KB;
  c.tiles = c.e->tiles;
}
__device__ __forceinline__ void cursor_seek(const GParams& g, Cursor& c, uint32_t u) {
  int lo = 0, hi = g.count - 1;  // last problem whose unit_begin <= u
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (g.table[mid].unit_begin <= u) lo = mid; else hi = mid - 1;
  }
  cursor_load(g, c, lo);
  const uint32_t local = u - c.e->unit_begin;
  c.tile = local / c.KB;
  c.kb = local - c.tile * c.KB;
}
// Advance by `n` stages that stay inside the current tile (n <= KB - kb).
__device__ __forceinline__ void cursor_advance(const GParams& g, Cursor& c, uint32_t n) {
  c.kb += n;
  if (c.kb == c.KB) {
    c.kb = 0;
    if (++c.tile == c.tiles && c.pi + 1 < g.count) {
      cursor_load(g, c, c.pi + 1);
      c.tile = 0;
    }
  }
}

__device__ __forceinline__ void fence_tensormap_acquire(const void* tmap) {
  asm volatile("fence.proxy.tensormap::generic.acquire.sys [%0], 128;" ::"l"(tmap) : "memory");
}

__device__ __forceinline__ void group_store1(const GParams& g, const GroupEntry* e, int m, int n, float v) {
  const __half h = __float2half_rn(v);
  if (g.world == 0) {
    e->C[static_cast<size_t>(m) * e->N + n] = h;
  } else if (g.mc_flag != nullptr) {
    // multicast stores are at least 32 bits wide: even lanes store their column and the next one
    const unsigned int mine = __half_as_ushort(h);
    const unsigned int next = __shfl_down_sync(0xffffffffu, mine, 1);
    if ((n & 1) == 0)
      multimem_st_b32(e->mc_C + static_cast<size_t>(m) * e->ldc + e->col0 + n, mine | (next << 16));
  } else {
    const size_t off = static_cast<size_t>(m) * e->ldc + e->col0 + n;
    for (int q = 0; q < g.world; ++q) e->peer_C[q][off] = h;
  }
}
__device__ __forceinline__ void group_store2(const GParams& g, const GroupEntry* e, int m, int n, float2 v) {
  const __half2 h = __floats2half2_rn(v.x, v.y);
  if (g.world == 0) {
    *reinterpret_cast<__half2*>(e->C + static_cast<size_t>(m) * e->N + n) = h;
  } else if (g.mc_flag != nullptr) {
    multimem_st_b32(e->mc_C + static_cast<size_t>(m) * e->ldc + e->col0 + n, *reinterpret_cast<const uint32_t*>(&h));
  } else {
    const size_t off = static_cast<size_t>(m) * e->ldc + e->col0 + n;
    for (int q = 0; q < g.world; ++q) *reinterpret_cast<__half2*>(e->peer_C[q] + off) = h;
  }
}
// Four adjacent outputs (n a multiple of 4) as one 8-byte store where the destination is plain memory.
__device__ __forceinline__ void group_store4(const GParams& g, const GroupEntry* e, int m, int n, float4 v) {
  const __half2 lo = __floats2half2_rn(v.x, v.y), hi = __floats2half2_rn(v.z, v.w);
  uint2 w;
  w.x = *reinterpret_cast<const uint32_t*>(&lo);
  w.y = *reinterpret_cast<const uint32_t*>(&hi);
  if (g.world != 0 && g.mc_flag != nullptr) {
    multimem_st_v2_f16x2(e->mc_C + static_cast<size_t>(m) * e->ldc + e->col0 + n, w.x, w.y);
  } else if (g.world == 0) {
    *reinterpret_cast<uint2*>(e->C + static_cast<size_t>(m) * e->N + n) = w;
  } else {
    const size_t off = static_cast<size_t>(m) * e->ldc + e->col0 + n;
    for (int q = 0; q < g.world; ++q) *reinterpret_cast<uint2*>(e->peer_C[q] + off) = w;
  }
}
__device__ __forceinline__ void group_signal(const GParams& g) {
  if (g.mc_flag != nullptr) {
    multimem_red_release_add_u64(g.mc_flag + g.rank, 1ull);
    return;
  }
  fence_acq_rel_sys();  // one release for the stores of all threads that passed the barrier before this call
  for (int q = 0; q < g.world; ++q) atomicAdd_system(g.peer_flag[q] + g.rank, 1ull);
}

template <int OP>
__global__ void __launch_bounds__(kUmmaGroupThreads, 1) fg_umma_group_kernel(const GParams g) {
  static_assert(OP == kOpF16KN || OP == kOpF16NK, "tcgen05 path: fp16 weights only");
  constexpr int MT = kUmmaMT;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

  const int S = g.stages;
  const int cps = g.chunks_per_stage;
  constexpr int cbytes = chunk_bytes(OP, MT);
  const uint32_t stage_bytes = cps * cbytes;
  const uint32_t ring_bytes = S * stage_bytes;
  const uint32_t bar_base = smem_base + ring_bytes;
  const uint32_t bar_acc_full = bar_base + 16 * S;
  const uint32_t bar_acc_empty = bar_acc_full + 16;
  const uint32_t bar_flush = bar_acc_empty + 16;
  const uint32_t bar_fin = bar_flush + 8;
  const uint32_t tmem_slot = bar_fin + 8;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + ring_bytes + 16 * S + 48);
  volatile uint32_t* prev_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + ring_bytes + 16 * S + 52);

  if (blockDim.x != static_cast<unsigned>(kUmmaGroupThreads) || dynamic_smem_size() < 1023u + ring_bytes + 16u * S + 64u) {
    if (threadIdx.x == 0) atomicExch(g.status, kStatusBadLaunch);
    return;
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  unsigned long long* trace = g.trace ? g.trace + kTraceSlots * blockIdx.x : nullptr;
  if (trace && threadIdx.x == 0) trace[0] = globaltimer_ns();

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_base + 8 * s, 1);
      mbar_init(bar_base + 8 * (S + s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 4);
    }
    mbar_init(bar_flush, 128);
    mbar_init(bar_fin, 1);
    fence_mbar_init();
    fence_proxy_async();
  }
  if (warp == 5) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot_gen;

  const uint32_t total = g.total_units;
  const uint32_t G = gridDim.x;
  const uint32_t ub = range_begin(blockIdx.x, total, G);
  const uint32_t ue = range_begin(blockIdx.x + 1, total, G);
  const int k_per_stage = cps * 64;

  if (warp == 4) {
    // ------------------------------------ producer ------------------------------------
    if (lane == 0) {
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_x = policy_evict_last();
      const int n_it = static_cast<int>(ue - ub);
      Cursor cw, cx;  // the weight cursor runs ahead of the activation cursor by the first ring-full
      cursor_seek(g, cw, ub);
      cx = cw;
      int fenced = -1;  // tensor maps of problems <= fenced have been acquired
      auto acquire = [&](const Cursor& c) {
        if (c.pi > fenced) {
          fence_tensormap_acquire(&c.e->tmW);
          fence_tensormap_acquire(&c.e->tmX);
          fenced = c.pi;
        }
      };
      auto stage_chunks = [&](const Cursor& c) {
        const int k0 = c.kb * k_per_stage;
        const int nch = (c.e->K - k0 + 63) / 64;
        return nch < cps ? nch : cps;
      };
      auto issue_w = [&](int s, const Cursor& c, int nch) {
        const uint32_t full = bar_base + 8 * s;
        uint32_t dst = smem_base + s * stage_bytes;
        for (int ch = 0; ch < nch; ++ch) {
          const int kc = c.kb * k_per_stage + ch * 64;
          if constexpr (OP == kOpF16KN) {
            tma_load_2d(dst, &c.e->tmW, full, c.tile * kTileN, kc, pol_w);
            tma_load_2d(dst + 8192, &c.e->tmW, full, c.tile * kTileN + 64, kc, pol_w);
          } else {
            tma_load_2d(dst, &c.e->tmW, full, kc, c.tile * kTileN, pol_w);
          }
          dst += cbytes;
        }
      };
      auto issue_x = [&](int s, const Cursor& c, int nch) {
        const uint32_t full = bar_base + 8 * s;
        uint32_t dst = smem_base + s * stage_bytes + kChunkWBytes;
        for (int ch = 0; ch < nch; ++ch) {
          tma_load_2d(dst, &c.e->tmX, full, c.kb * k_per_stage + ch * 64, 0, pol_x);
          dst += cbytes;
        }
      };
      if (trace) trace[1] = globaltimer_ns();
      // weights first (they never depend on earlier kernels), activations after the wait
      griddep_launch_dependents();
      const int pre = n_it < S ? n_it : S;
      for (int i = 0; i < pre; ++i) {
        acquire(cw);
        const int nch = stage_chunks(cw);
        mbar_arrive_expect_tx(bar_base + 8 * i, nch * cbytes);
        issue_w(i, cw, nch);
        cursor_advance(g, cw, 1);
      }
      griddep_wait();
      if (blockIdx.x == 0 && g.target_dev != nullptr) atomicAdd(g.target_dev, static_cast<unsigned long long>(g.total_tiles));
      for (int i = 0; i < pre; ++i) {
        issue_x(i, cx, stage_chunks(cx));
        cursor_advance(g, cx, 1);
      }
      bool dead = false;
      int issued = pre;
      int s = (pre == S) ? 0 : pre;
      uint32_t use = (pre == S) ? 1u : 0u;
      for (int it = pre; it < n_it; ++it, s = (s + 1 == S) ? 0 : s + 1, use += (s == 0)) {
        if (!mbar_wait_bounded(bar_base + 8 * (S + s), (use & 1) ^ 1, kWaitBudgetNs)) {
          dead = true;
          break;
        }
        acquire(cw);
        const int nch = stage_chunks(cw);
        mbar_arrive_expect_tx(bar_base + 8 * s, nch * cbytes);
        issue_w(s, cw, nch);
        issue_x(s, cw, nch);
        cursor_advance(g, cw, 1);
        ++issued;
      }
      if (trace) trace[2] = globaltimer_ns();
      if (dead) {
        atomicExch(g.status, kStatusTimeout);
        const int back = issued < S ? issued : S;
        for (int i = issued - back; i < issued; ++i)
          mbar_wait_bounded(bar_base + 8 * (i % S), (i / S) & 1, kWaitBudgetNs);
      }
    }
    return;
  }

  if (warp >= 6) {
    // ------------------------------------ finishers ------------------------------------
    constexpr int FW = finisher_warps<MT>();
    const int fin_warp = warp - 6;
    const bool leader = (fin_warp == 0 && lane == 0);
    Cursor c;
    cursor_seek(g, c, ub);
    uint32_t u = ub, ev = 0;
    bool dead = false;
    while (u < ue) {
      const uint32_t len = (c.KB - c.kb) < (ue - u) ? (c.KB - c.kb) : (ue - u);
      if (len != c.KB && !dead) {
        bool ok = mbar_wait_bounded(bar_flush, ev & 1, kWaitBudgetNs * 4);
        ok = __all_sync(0xffffffffu, ok);
        const uint32_t t0 = c.e->unit_begin + c.tile * c.KB;  // first stage of this tile
        const uint32_t c_first = cta_of_unit(t0, total, G);
        const uint32_t c_last = cta_of_unit(t0 + c.KB - 1, total, G);
        const uint32_t gtile = c.e->tile_begin + c.tile;
        if (leader) {
          uint32_t prev = 0xffffffffu;
          if (ok) {
            __threadfence();
            prev = atomicAdd(g.tickets + gtile, 1u);
          } else {
            atomicExch(g.status, kStatusTimeout);
          }
          *prev_slot = prev;
        }
        named_bar_sync(kFinBarrier, FW * 32);
        const uint32_t prev = *prev_slot;
        if (prev == 0xffffffffu) dead = true;
        if (prev == c_last - c_first) {
          __threadfence();
          const int n0 = c.tile * kTileN + 4 * lane;
          const int m0 = 4 * fin_warp;
          const int M = c.e->M;
          if (m0 < M) {
            float4 sum[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) sum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (uint32_t c0 = c_first; c0 <= c_last; c0 += 4) {
              float4 v[4][4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const uint32_t cc = c0 + j;
                if (cc <= c_last) {
                  const uint32_t rb = range_begin(cc, total, G);
                  const uint32_t cslot = (rb >= t0 && rb < t0 + c.KB) ? 0u : 1u;
                  const float4* src = reinterpret_cast<const float4*>(
                      g.partials + (static_cast<size_t>(cc) * 2 + cslot) * (MT * kTileN));
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
              const int m = m0 + i;
              if (m < M) group_store4(g, c.e, m, n0, sum[i]);
            }
          }
        }
        named_bar_sync(kFinBarrier, FW * 32);
        if (leader) {
          if (prev == c_last - c_first) {
            g.tickets[gtile] = 0;
            if (g.world > 0) group_signal(g);
          }
          mbar_arrive(bar_fin);
        }
        ++ev;
      }
      u += len;
      cursor_advance(g, c, len);
    }
    if (trace && leader) trace[5] = globaltimer_ns();
    return;
  }

  if (warp == 5) {
    // ------------------------------------ MMA issue ------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(OP == kOpF16KN);
      constexpr uint64_t a_hi = (OP == kOpF16NK) ? umma_smem_desc(0, 1, 64) : umma_smem_desc(0, 512, 64);
      constexpr uint64_t b_hi = umma_smem_desc(0, 1, 64);
      constexpr uint64_t a_step = (OP == kOpF16NK) ? 2 : 128;
      Cursor c;
      cursor_seek(g, c, ub);
      uint32_t u = ub;
      int it0 = 0;
      uint32_t sg = 0;
      bool dead = false;
      int s = 0;
      uint32_t ph = 0;
      while (u < ue && !dead) {
        const int kb0 = static_cast<int>(c.kb);
        const int len = static_cast<int>((c.KB - c.kb) < (ue - u) ? (c.KB - c.kb) : (ue - u));
        const int K = c.e->K;
        const uint32_t b = sg & 1, use = sg >> 1;
        if (!mbar_wait_bounded(bar_acc_empty + 8 * b, (use & 1) ^ 1, kWaitBudgetNs)) {
          dead = true;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + b * (kUmmaChains * kUmmaMT);
        for (int it = it0; it < it0 + len; ++it, s = (s + 1 == S) ? 0 : s + 1, ph ^= (s == 0)) {
          const unsigned long long tw0 = trace ? globaltimer_ns() : 0;
          if (!mbar_wait_bounded(bar_base + 8 * s, ph, kWaitBudgetNs)) {
            dead = true;
            break;
          }
          const unsigned long long tw1 = trace ? globaltimer_ns() : 0;
          if (trace) trace[9] += tw1 - tw0;
          if (trace && it == 0) trace[3] = tw1;
          const int k0 = (kb0 + (it - it0)) * k_per_stage;
          int nch = (K - k0 + 63) / 64;
          nch = nch < cps ? nch : cps;
          uint32_t wb = smem_base + s * stage_bytes;
          uint32_t acc_flag = (it > it0) ? 1u : 0u;
          for (int ch = 0; ch < nch; ++ch) {
            const uint64_t a0 = a_hi | (wb >> 4);
            const uint64_t b0 = b_hi | ((wb + kChunkWBytes) >> 4);
            umma_f16(tmem_d, a0, b0, idesc, acc_flag);
            umma_f16(tmem_d + kUmmaMT, a0 + a_step, b0 + 2, idesc, acc_flag);
            umma_f16(tmem_d, a0 + 2 * a_step, b0 + 4, idesc, 1u);
            umma_f16(tmem_d + kUmmaMT, a0 + 3 * a_step, b0 + 6, idesc, 1u);
            acc_flag = 1u;
            wb += cbytes;
          }
          umma_commit(bar_base + 8 * (S + s));
          if (trace) trace[10] += globaltimer_ns() - tw1;
        }
        if (dead) break;
        umma_commit(bar_acc_full + 8 * b);
        if (trace) trace[4] = globaltimer_ns();
        ++sg;
        u += len;
        it0 += len;
        cursor_advance(g, c, len);
      }
      if (dead) atomicExch(g.status, kStatusTimeout);
    }
    __syncwarp();
  } else {
    // ------------------------------------ epilogue warps 0-3 ------------------------------------
    const int n_in_tile = warp * 32 + lane;
    Cursor c;
    cursor_seek(g, c, ub);
    uint32_t u = ub;
    uint32_t sg = 0, ev = 0;
    bool dead = false;
    while (u < ue) {
      const uint32_t len = (c.KB - c.kb) < (ue - u) ? (c.KB - c.kb) : (ue - u);
      const bool whole = (len == c.KB);
      const uint32_t b = sg & 1, use = sg >> 1;
      uint32_t r[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = 0;
      if (!dead) {
        bool ok = mbar_wait_bounded(bar_acc_full + 8 * b, use & 1, kWaitBudgetNs * 2);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
          dead = true;
          if (lane == 0) atomicExch(g.status, kStatusTimeout);
        }
      }
      if (!dead) {
        tc_fence_after_sync();
        tmem_ld32(tmem_base + (static_cast<uint32_t>(warp * 32) << 16) + b * (kUmmaChains * kUmmaMT), r);
        tmem_ld_wait();
#pragma unroll
        for (int m = 0; m < MT; ++m) r[m] = __float_as_uint(__uint_as_float(r[m]) + __uint_as_float(r[MT + m]));
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_acc_empty + 8 * b);
      }
      if (trace && threadIdx.x == 0) trace[7] = globaltimer_ns();
      if (whole) {
        const int n = c.tile * kTileN + n_in_tile;
        const int M = c.e->M;
#pragma unroll
        for (int m = 0; m < MT; ++m)
          if (m < M) group_store1(g, c.e, m, n, __uint_as_float(r[m]));
        if (g.world > 0) {
          named_bar_sync(1, 128);
          if (threadIdx.x == 0) group_signal(g);
        }
      } else {
        if (ev >= 1) {
          bool ok = mbar_wait_bounded(bar_fin, (ev - 1) & 1, kWaitBudgetNs * 4);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok && !dead) {
            dead = true;
            if (lane == 0) atomicExch(g.status, kStatusTimeout);
          }
        }
        const int slot = (u == ub) ? 0 : 1;
        float* mypart = g.partials + (static_cast<size_t>(blockIdx.x) * 2 + slot) * (MT * kTileN);
#pragma unroll
        for (int m = 0; m < MT; ++m) mypart[m * kTileN + n_in_tile] = __uint_as_float(r[m]);
        mbar_arrive(bar_flush);
        ++ev;
      }
      if (trace && threadIdx.x == 0) trace[6] += 1;
      ++sg;
      u += len;
      cursor_advance(g, c, len);
    }
  }

  tc_fence_before_sync();
  named_bar_sync(2, 160);
  if (warp == 5) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace fg
