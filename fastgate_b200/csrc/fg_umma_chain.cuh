// A stack of dependent fp16 projections in ONE persistent tcgen05 kernel.
//
// Layer i computes C_i[M, N_i] = act(x_i[M, K_i] . W_i^T + bias_i) + residual_i with M <= 16,
// and x_i may be (a column slice of) the output of an earlier layer of the same chain.  The
// layers run in order; inside a layer the stages are dealt to the CTAs in equal contiguous
// ranges exactly as fg_umma_kernel does (stream-K, split tiles reduced in CTA order).  What a
// launch per layer cannot do is keep HBM busy across the layer boundary: here every CTA goes on
// prefetching the next layer's weights into its ring while the tail of the previous layer
// (partial tiles, tickets, last stores) drains, and only the activations wait - on a per-layer
// counter of finished output tiles, with a bounded wait.
//
// Inter-CTA waits need all CTAs resident at once: the host launches this kernel cooperatively.
#pragma once
#include "fg_layout.h"
#include "fg_umma.cuh"
#include "fg_umma_group.cuh"

namespace fg {

struct alignas(128) ChainEntry {
  CUtensorMap tmW;        // weight [N, K] (NxK op) or [K, N] (KxN op), 128B swizzle
  CUtensorMap tmX;        // activations [M, K] (row stride ldx), box of 16 rows
  __half* C;              // output [M, N], row stride ldc
  const __half* bias;     // [N] or null
  const __half* residual; // [M, N], row stride ldr, or null
  long long ldc, ldr;
  int M, N, K;
  int act;
  int dep;                // layer whose finished output the activations read, or -1
  uint32_t KB;            // stages per output tile
  uint32_t tiles;         // N / 128
  uint32_t tile_begin;    // first output tile of this layer (ticket index)
};

struct CParams {
  const ChainEntry* table;
  int count;
  float* partials;        // [grid][4] tiles of 16 x 128 fp32: two per CTA and layer parity
  unsigned int* tickets;  // one per output tile of the chain, zero between launches
  unsigned int* done;     // finished output tiles per layer, zeroed by the host before a launch
  int* status;
  unsigned long long* trace;  // optional [layer][cta][8] words: timestamps (ns) of activations ready,
                              // first stage landed, last stage committed, last tile or partial handed
                              // on, last partial written, its ticket back, its reduction loaded; then
                              // the number of contributors if this CTA reduced its last split tile
  int chunks_per_stage;
  int stages;
};

__device__ __forceinline__ void chain_note(const CParams& g, int pi, int what, unsigned long long v) {
  if (g.trace != nullptr) g.trace[(static_cast<size_t>(pi) * gridDim.x + blockIdx.x) * 8 + what] = v;
}
__device__ __forceinline__ void chain_stamp(const CParams& g, int pi, int what) {
  if (g.trace != nullptr)
    g.trace[(static_cast<size_t>(pi) * gridDim.x + blockIdx.x) * 8 + what] = globaltimer_ns();
}

// This CTA's position inside its share [u, ue) of layer pi.
struct ChainCursor {
  int pi;
  const ChainEntry* e;
  uint32_t U, G, ub, ue, u;  // G: CTAs that share this layer (the first min(grid, U))
  uint32_t KB, tile, kb;
  int K;
};

// Move to the first layer >= pi in which this CTA owns stages; false past the last layer.
__device__ __forceinline__ bool chain_enter(const CParams& g, ChainCursor& c, int pi) {
  for (; pi < g.count; ++pi) {
    const ChainEntry* e = g.table + pi;
    const uint32_t U = e->tiles * e->KB;
    const uint32_t G = U < gridDim.x ? U : gridDim.x;  // every sharing CTA owns at least one stage
    if (blockIdx.x < G) {
      const uint32_t ub = range_begin(blockIdx.x, U, G);
      const uint32_t ue = range_begin(blockIdx.x + 1, U, G);
      c.pi = pi;
      c.e = e;
      c.U = U;
      c.G = G;
      c.ub = c.u = ub;
      c.ue = ue;
      c.KB = e->KB;
      c.K = e->K;
      c.tile = ub / c.KB;
      c.kb = ub - c.tile * c.KB;
      return true;
    }
  }
  c.pi = g.count;
  c.e = nullptr;
  return false;
}
// Advance by n stages that stay inside the current tile and share.
__device__ __forceinline__ void chain_advance(const CParams& g, ChainCursor& c, uint32_t n) {
  c.u += n;
  c.kb += n;
  if (c.kb == c.KB) {
    c.kb = 0;
    ++c.tile;
  }
  if (c.u == c.ue) chain_enter(g, c, c.pi + 1);
}
__device__ __forceinline__ bool chain_valid(const CParams& g, const ChainCursor& c) { return c.pi < g.count; }
__device__ __forceinline__ uint32_t chain_seg_len(const ChainCursor& c) {
  return (c.KB - c.kb) < (c.ue - c.u) ? (c.KB - c.kb) : (c.ue - c.u);
}

__device__ __forceinline__ unsigned int ld_acquire_gpu(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Orders earlier generic-proxy accesses (the acquire above) before later async-proxy ones (TMA).
__device__ __forceinline__ void fence_proxy_async_global() {
  asm volatile("fence.proxy.async.global;" ::: "memory");
}
// Bounded wait until layer `dep` has delivered all its output tiles.
__device__ __forceinline__ bool chain_wait_done(const CParams& g, int dep) {
  const unsigned int want = g.table[dep].tiles;
  if (ld_acquire_gpu(g.done + dep) >= want) return true;
  const unsigned long long t0 = globaltimer_ns();
  while (ld_acquire_gpu(g.done + dep) < want) {
    if (globaltimer_ns() - t0 > kWaitBudgetNs) return false;
    __nanosleep(64);
  }
  return true;
}

// A 16-bit global load the compiler may not sink to its first use (the point of issuing it
// early is that it travels during the ticket's round trip).
__device__ __forceinline__ __half ld_half_now(const __half* p) {
  unsigned short v;
  asm volatile("ld.global.u16 %0, [%1];" : "=h"(v) : "l"(p) : "memory");
  return __ushort_as_half(v);
}

// The fused epilogue of a layer, read once per segment (not per element) from the table.
struct ChainEpilogue {
  const __half* bias;
  const __half* residual;
  long long ldr;
  int act;
  bool any;
};
__device__ __forceinline__ ChainEpilogue chain_epilogue_of(const ChainEntry* e) {
  ChainEpilogue ep{e->bias, e->residual, e->ldr, e->act, false};
  ep.any = ep.bias != nullptr || ep.residual != nullptr || ep.act != kActNone;
  return ep;
}
template <int ACT>
__device__ __forceinline__ float chain_epilogue(const ChainEpilogue& ep, int m, int n, float v) {
  if (ep.bias != nullptr) v += __half2float(__ldg(ep.bias + n));
  v = act_fn<ACT>(v);
  if (ep.residual != nullptr) v += __half2float(ep.residual[static_cast<size_t>(m) * ep.ldr + n]);
  return v;
}

template <int OP>
__global__ void __launch_bounds__(kUmmaThreads, 1) fg_umma_chain_kernel(const CParams g) {
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
  const uint32_t bar_flush = bar_acc_empty + 16;  // [2] epilogue -> finisher team
  const uint32_t bar_fin = bar_flush + 16;        // [2] finisher team -> epilogue
  const uint32_t tmem_slot = bar_fin + 16;
  volatile uint32_t* tmem_slot_gen = reinterpret_cast<volatile uint32_t*>(smem_gen + ring_bytes + 16 * S + 64);
  volatile uint32_t* prev_slots = reinterpret_cast<volatile uint32_t*>(smem_gen + ring_bytes + 16 * S + 68);  // [2]

  if (blockDim.x != static_cast<unsigned>(kUmmaThreads) || dynamic_smem_size() < 1023u + ring_bytes + 16u * S + 96u) {
    if (threadIdx.x == 0) atomicExch(g.status, kStatusBadLaunch);
    return;
  }

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(bar_base + 8 * s, 1);
      mbar_init(bar_base + 8 * (S + s), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar_acc_full + 8 * b, 1);
      mbar_init(bar_acc_empty + 8 * b, 4);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(bar_flush + 8 * t, 128);
      mbar_init(bar_fin + 8 * t, 1);
    }
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

  const int k_per_stage = cps * 64;

  if (warp == 4) {
    // ------------------------------------ producer ------------------------------------
    // One thread feeds the ring.  Weights never wait: they are issued as soon as a slot is
    // free, up to a ring-full ahead of the activations.  The activations of a stage are issued
    // once the layer they come from has delivered all its tiles; until then the thread polls
    // both conditions in turn, so a slot that frees up is refilled during the wait.
    if (lane == 0) {
      const uint64_t pol_w = policy_evict_first();
      const uint64_t pol_x = policy_evict_last();
      ChainCursor cw, cx, cp;  // next weights, next activations, next L2 prefetch (>= cw)
      chain_enter(g, cw, 0);
      cx = cw;
      cp = cw;
      int pf = 0;  // stages by which cp is ahead of cw
      const int pf_max = FG_L2_PREFETCH_BYTES / (cps * kChunkWBytes) > 0 ? FG_L2_PREFETCH_BYTES / (cps * kChunkWBytes) : 1;
      int fenced = -1;  // tensor maps of layers <= fenced have been acquired
      int ready = -1;   // activations of layers <= ready may be read
      int sw = 0, sx = 0, ahead = 0;
      uint32_t use_w = 0;
      unsigned long long t_idle = 0;
      bool dead = false;
      auto stage_chunks = [&](const ChainCursor& c) {
        const int nch = (c.K - static_cast<int>(c.kb) * k_per_stage + 63) / 64;
        return nch < cps ? nch : cps;
      };
      while (chain_valid(g, cx)) {
        bool progressed = false;
        // activations first: a stage whose weights are in flight must never wait for a ring slot
        while (ahead > 0) {
          if (cx.pi > ready) {
            const int dep = cx.e->dep;
            if (dep >= 0 && ld_acquire_gpu(g.done + dep) < g.table[dep].tiles) break;
            fence_proxy_async_global();
            ready = cx.pi;
            chain_stamp(g, cx.pi, 0);
          }
          const int nch = stage_chunks(cx);
          const uint32_t full = bar_base + 8 * sx;
          uint32_t dst = smem_base + sx * stage_bytes + kChunkWBytes;
          for (int ch = 0; ch < nch; ++ch) {
            tma_load_2d(dst, &cx.e->tmX, full, cx.kb * k_per_stage + ch * 64, 0, pol_x);
            dst += cbytes;
          }
          chain_advance(g, cx, 1);
          sx = (sx + 1 == S) ? 0 : sx + 1;
          --ahead;
          progressed = true;
        }
        if (chain_valid(g, cw) && ahead < S && mbar_test_wait(bar_base + 8 * (S + sw), (use_w & 1) ^ 1)) {
          if (cw.pi > fenced) {
            fence_tensormap_acquire(&cw.e->tmW);
            fence_tensormap_acquire(&cw.e->tmX);
            fenced = cw.pi;
          }
          const int nch = stage_chunks(cw);
          const uint32_t full = bar_base + 8 * sw;
          mbar_arrive_expect_tx(full, nch * cbytes);
          uint32_t dst = smem_base + sw * stage_bytes;
          for (int ch = 0; ch < nch; ++ch) {
            const int kc = cw.kb * k_per_stage + ch * 64;
            if constexpr (OP == kOpF16KN) {
              tma_load_2d(dst, &cw.e->tmW, full, cw.tile * kTileN, kc, pol_w);
              tma_load_2d(dst + 8192, &cw.e->tmW, full, cw.tile * kTileN + 64, kc, pol_w);
            } else {
              tma_load_2d(dst, &cw.e->tmW, full, kc, cw.tile * kTileN, pol_w);
            }
            dst += cbytes;
          }
          chain_advance(g, cw, 1);
          if (pf > 0) --pf; else cp = cw;
          if (++sw == S) {
            sw = 0;
            ++use_w;
          }
          ++ahead;
          progressed = true;
        } else if (ahead == S && pf < pf_max && chain_valid(g, cp)) {
          // the ring is full and the activations are not there yet: HBM would idle, so ask
          // for the next stages' weights to be brought into L2 meanwhile
          if (cp.pi > fenced) {
            fence_tensormap_acquire(&cp.e->tmW);
            fence_tensormap_acquire(&cp.e->tmX);
            fenced = cp.pi;
          }
          const int nch = stage_chunks(cp);
          for (int ch = 0; ch < nch; ++ch) {
            const int kc = cp.kb * k_per_stage + ch * 64;
            if constexpr (OP == kOpF16KN) {
              tma_prefetch_l2_2d(&cp.e->tmW, cp.tile * kTileN, kc);
              tma_prefetch_l2_2d(&cp.e->tmW, cp.tile * kTileN + 64, kc);
            } else {
              tma_prefetch_l2_2d(&cp.e->tmW, kc, cp.tile * kTileN);
            }
          }
          chain_advance(g, cp, 1);
          ++pf;
          progressed = true;
        }
        if (progressed) {
          t_idle = 0;
        } else {
          const unsigned long long now = globaltimer_ns();
          if (t_idle == 0) {
            t_idle = now;
          } else if (now - t_idle > kWaitBudgetNs) {
            dead = true;
            break;
          }
        }
      }
      if (dead) atomicExch(g.status, kStatusTimeout);
    }
    return;
  }

  if (warp >= 6) {
    // ------------------------------------ finishers ------------------------------------
    // Two teams of MT/4 warps take the CTA's partial segments in turn (team = index of the
    // partial & 1): the end of one layer and the start of the next often leave a CTA with two
    // partials in flight, and a reduction of the first must not hold back the ticket of the second.
    constexpr int FW = finisher_warps<MT>();
    const int team = (warp - 6) / FW;
    const int fin_warp = (warp - 6) % FW;
    const bool leader = (fin_warp == 0 && lane == 0);
    const uint32_t my_flush = bar_flush + 8 * team, my_fin = bar_fin + 8 * team;
    volatile uint32_t* prev_slot = prev_slots + team;
    const int bar_id = kFinBarrier + team;
    ChainCursor c;
    chain_enter(g, c, 0);
    uint32_t ev = 0;  // partial segments of this CTA so far (both teams count all of them)
    bool dead = false;
    while (chain_valid(g, c)) {
      const uint32_t len = chain_seg_len(c);
      const bool mine = (len != c.KB) && (ev & 1) == static_cast<uint32_t>(team);
      if (mine && !dead) {
        bool ok = mbar_wait_bounded(my_flush, (ev >> 1) & 1, kWaitBudgetNs * 4);
        ok = __all_sync(0xffffffffu, ok);
        // Everything the final store needs besides the partials is requested now, so that it
        // travels while the ticket does: the table entry, the bias of this lane's four columns
        // and the residual of its 4 x 4 outputs.  (Not earlier: the teams run ahead of the
        // layers, and only the partial's arrival says that this layer's inputs are complete.)
        const ChainEntry* e = c.e;
        const ChainEpilogue ep = chain_epilogue_of(e);
        __half* const Cb = e->C;
        const long long ldc = e->ldc;
        const int M = e->M;
        const int n0 = c.tile * kTileN + 4 * lane;
        const int m0 = 4 * fin_warp;
        __half bias4[4], res4[4][4];
#pragma unroll
        for (int q = 0; q < 4; ++q) bias4[q] = ep.bias != nullptr ? ld_half_now(ep.bias + n0 + q) : __half(0.f);
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int q = 0; q < 4; ++q)
            res4[i][q] = (ep.residual != nullptr && m0 + i < M)
                             ? ld_half_now(ep.residual + static_cast<size_t>(m0 + i) * ep.ldr + n0 + q)
                             : __half(0.f);
        const uint32_t t0 = c.tile * c.KB;  // first stage of this tile inside the layer
        const uint32_t c_first = cta_of_unit(t0, c.U, c.G);
        const uint32_t c_last = cta_of_unit(t0 + c.KB - 1, c.U, c.G);
        const uint32_t gtile = e->tile_begin + c.tile;
        const uint32_t parity = static_cast<uint32_t>(c.pi & 1) * 2u;
        if (leader) {
          uint32_t prev = 0xffffffffu;
          if (ok) {
            fence_acq_rel_gpu();
            prev = atomicAdd(g.tickets + gtile, 1u);
          } else {
            atomicExch(g.status, kStatusTimeout);
          }
          *prev_slot = prev;
          chain_stamp(g, c.pi, 5);
          chain_note(g, c.pi, 7, prev == c_last - c_first ? c_last - c_first + 1 : 0);
        }
        named_bar_sync(bar_id, FW * 32);
        const uint32_t prev = *prev_slot;
        if (prev == 0xffffffffu) dead = true;
        if (prev == c_last - c_first) {
          fence_acq_rel_gpu();
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
                  const uint32_t rb = range_begin(cc, c.U, c.G);
                  const uint32_t cslot = parity + ((rb >= t0 && rb < t0 + c.KB) ? 0u : 1u);
                  const float4* src = reinterpret_cast<const float4*>(
                      g.partials + (static_cast<size_t>(cc) * 4 + cslot) * (MT * kTileN));
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
            if (leader) chain_stamp(g, c.pi, 6);
            with_act(ep.any ? ep.act : kActNone, [&](auto tag) {
              constexpr int ACT = decltype(tag)::value;
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const int m = m0 + i;
                if (m < M) {
                  float o[4] = {sum[i].x, sum[i].y, sum[i].z, sum[i].w};
                  if (ep.any) {
#pragma unroll
                    for (int q = 0; q < 4; ++q)
                      o[q] = act_fn<ACT>(o[q] + __half2float(bias4[q])) + __half2float(res4[i][q]);
                  }
                  // one 8-byte store per row and lane: the number of stores, not their bytes, is what the
                  // layers waiting for this tile feel
                  const __half2 lo = __floats2half2_rn(o[0], o[1]), hi = __floats2half2_rn(o[2], o[3]);
                  uint2 w;
                  w.x = *reinterpret_cast<const uint32_t*>(&lo);
                  w.y = *reinterpret_cast<const uint32_t*>(&hi);
                  *reinterpret_cast<uint2*>(Cb + static_cast<size_t>(m) * ldc + n0) = w;
                }
              }
            });
          }
          __threadfence();  // the tile is visible before the layer's counter says so
        }
        named_bar_sync(bar_id, FW * 32);
        if (leader) {
          if (prev == c_last - c_first) {
            g.tickets[gtile] = 0;
            atomicAdd(g.done + c.pi, 1u);
          }
          mbar_arrive(my_fin);
          chain_stamp(g, c.pi, 3);
        }
      }
      if (len != c.KB) ++ev;
      chain_advance(g, c, len);
    }
    return;
  }

  if (warp == 5) {
    // ------------------------------------ MMA issue ------------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = umma_idesc(OP == kOpF16KN);
      constexpr uint64_t a_hi = (OP == kOpF16NK) ? umma_smem_desc(0, 1, 64) : umma_smem_desc(0, 512, 64);
      constexpr uint64_t b_hi = umma_smem_desc(0, 1, 64);
      constexpr uint64_t a_step = (OP == kOpF16NK) ? 2 : 128;
      ChainCursor c;
      chain_enter(g, c, 0);
      uint32_t sg = 0;
      bool dead = false;
      int s = 0;
      uint32_t ph = 0;
      while (chain_valid(g, c) && !dead) {
        const int kb0 = static_cast<int>(c.kb);
        const int len = static_cast<int>(chain_seg_len(c));
        const int K = c.K;
        const uint32_t b = sg & 1, use = sg >> 1;
        if (!mbar_wait_bounded(bar_acc_empty + 8 * b, (use & 1) ^ 1, kWaitBudgetNs * 2)) {
          dead = true;
          break;
        }
        tc_fence_after_sync();
        const uint32_t tmem_d = tmem_base + b * (kUmmaChains * kUmmaMT);
        for (int it = 0; it < len; ++it, s = (s + 1 == S) ? 0 : s + 1, ph ^= (s == 0)) {
          // the activations of this stage may be waiting for the previous layer's tail
          if (!mbar_wait_bounded(bar_base + 8 * s, ph, kWaitBudgetNs * 2)) {
            dead = true;
            break;
          }
          if (c.u == c.ub && it == 0) chain_stamp(g, c.pi, 1);
          const int k0 = (kb0 + it) * k_per_stage;
          int nch = (K - k0 + 63) / 64;
          nch = nch < cps ? nch : cps;
          uint32_t wb = smem_base + s * stage_bytes;
          uint32_t acc_flag = (it > 0) ? 1u : 0u;
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
        }
        if (dead) break;
        umma_commit(bar_acc_full + 8 * b);
        if (c.u + len == c.ue) chain_stamp(g, c.pi, 2);
        ++sg;
        chain_advance(g, c, len);
      }
      if (dead) atomicExch(g.status, kStatusTimeout);
    }
    __syncwarp();
  } else {
    // ------------------------------------ epilogue warps 0-3 ------------------------------------
    const int n_in_tile = warp * 32 + lane;
    ChainCursor c;
    chain_enter(g, c, 0);
    uint32_t sg = 0, ev = 0;
    int guarded = 1;  // partial slots of layers <= guarded are free for reuse
    bool dead = false;
    while (chain_valid(g, c)) {
      const uint32_t len = chain_seg_len(c);
      const bool whole = (len == c.KB);
      const ChainEntry* e = c.e;
      const uint32_t b = sg & 1, use = sg >> 1;
      uint32_t r[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) r[i] = 0;
      if (!dead) {
        bool ok = mbar_wait_bounded(bar_acc_full + 8 * b, use & 1, kWaitBudgetNs * 4);
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
      if (whole) {
        const int n = c.tile * kTileN + n_in_tile;
        const int M = e->M;
        const ChainEpilogue ep = chain_epilogue_of(e);
        __half* const Cb = e->C;
        const long long ldc = e->ldc;
        with_act(ep.any ? ep.act : kActNone, [&](auto tag) {
          constexpr int ACT = decltype(tag)::value;
#pragma unroll
          for (int m = 0; m < MT; ++m)
            if (m < M) {
              float v = __uint_as_float(r[m]);
              if (ep.any) v = chain_epilogue<ACT>(ep, m, n, v);
              Cb[static_cast<size_t>(m) * ldc + n] = __float2half_rn(v);
            }
        });
        __threadfence();
        named_bar_sync(1, 128);
        if (threadIdx.x == 0 && !dead) {
          atomicAdd(g.done + c.pi, 1u);
          chain_stamp(g, c.pi, 3);
        }
      } else {
        if (ev >= 2) {  // the team that takes this partial must be done with its previous one
          bool ok = mbar_wait_bounded(bar_fin + 8 * (ev & 1), ((ev >> 1) - 1) & 1, kWaitBudgetNs * 4);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok && !dead) {
            dead = true;
            if (lane == 0) atomicExch(g.status, kStatusTimeout);
          }
        }
        // The slots alternate with the layer's parity; the one about to be overwritten was last
        // used two layers back, whose split tiles may still be waiting for their last arriver.
        if (c.pi > guarded && !dead) {
          bool ok = chain_wait_done(g, c.pi - 2);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) {
            dead = true;
            if (lane == 0) atomicExch(g.status, kStatusTimeout);
          }
          guarded = c.pi;
        }
        const uint32_t slot = static_cast<uint32_t>(c.pi & 1) * 2u + ((c.u == c.ub) ? 0u : 1u);
        float* mypart = g.partials + (static_cast<size_t>(blockIdx.x) * 4 + slot) * (MT * kTileN);
#pragma unroll
        for (int m = 0; m < MT; ++m) mypart[m * kTileN + n_in_tile] = __uint_as_float(r[m]);
        mbar_arrive(bar_flush + 8 * (ev & 1));
        if (threadIdx.x == 0) chain_stamp(g, c.pi, 4);
        ++ev;
      }
      ++sg;
      chain_advance(g, c, len);
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
