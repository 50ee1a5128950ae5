// Launch heuristic: pure host code, no CUDA calls, so it can be unit-tested on a box
// without a GPU.  It replaces the reference's split-K choice
// (backend/cuda/hk/edgemm.cu:287-305: BZ from tile-count thresholds 64/32 tuned for a
// 108-SM part, clamped by K % {1024,512,256}); script/heuristics.py is empty there.
//
// Here there is no split-K factor to pick: the (tile, k-block) list is dealt evenly to
// one persistent CTA per SM, so the plan only fixes the pipeline shape.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "../../include/fastgate_b200.h"
#include "fg_layout.h"

static int plan_impl(int op, int M, int N, int K, int sm_count, int smem_optin_bytes, fg_plan_t* out,
                     bool force_mma_sync, bool allow_gemv);

extern "C" int fg_plan(int op, int M, int N, int K, int sm_count, int smem_optin_bytes,
                       fg_plan_t* out) {
  return plan_impl(op, M, N, K, sm_count, smem_optin_bytes, out, false, true);
}

// Internal (fg_layout.h): the plan of the mma.sync kernel for a quantized op whatever M is.
extern "C" int fg_plan_mma_sync(int op, int M, int N, int K, int sm_count, int smem_optin_bytes,
                                fg_plan_t* out) {
  return plan_impl(op, M, N, K, sm_count, smem_optin_bytes, out, true, false);
}

// Internal (fg_layout.h): the plan of a tiled kernel even where fg_plan would pick the row-split
// GEMV kernel (entry points that push tiles to other ranks or use the library's built-in scratch).
extern "C" int fg_plan_tiled(int op, int M, int N, int K, int sm_count, int smem_optin_bytes,
                             fg_plan_t* out) {
  return plan_impl(op, M, N, K, sm_count, smem_optin_bytes, out, false, false);
}

// The row-split GEMV kernel takes NxK fp16 weights with up to four token rows when x fits in
// 64 KB of shared memory, a weight row in one ring stage, and a row has a 16-byte piece for every
// consumer thread.  (int8 weights stay with the tensor-core kernels: dequantising costs more issue
// slots per byte than the CUDA cores have left at HBM speed.)
static int gemv_max_m() {
  // FASTGATE_GEMV_MAX_M=0|1|2 narrows the kernel's range (0: never), for A/B measurements
  static const int v = [] {
    const char* e = std::getenv("FASTGATE_GEMV_MAX_M");
    const int n = (e != nullptr && e[0] >= '0' && e[0] <= '9') ? e[0] - '0' : FG_GEMV_MAX_M;
    return n < FG_GEMV_MAX_M ? n : FG_GEMV_MAX_M;
  }();
  return v;
}

static bool gemv_eligible(int op, int M, int K) {
  if (op == FG_OP_W8A16_NK)  // int8 rows: one token row (the conversion triples the instructions per byte)
    return M == 1 && gemv_max_m() >= 1 && K >= 2 * FG_GEMV_MIN_K && K * 2 <= 65536 && (K % 16) == 0;
  return op == FG_OP_F16_NK && M <= gemv_max_m() && K >= FG_GEMV_MIN_K && static_cast<long long>(M) * K * 2 <= 65536 &&
         K * 2 <= FG_GEMV_MAX_STAGE_BYTES;
}

static int plan_gemv(int op, int M, int N, int K, int sm_count, int smem_optin_bytes, fg_plan_t* out) {
  fg_plan_t p;
  std::memset(&p, 0, sizeof(p));
  p.op = op;
  p.math = 4;
  p.m_tile = M;
  p.passes = 1;
  p.tiles = N / 128;
  p.pdl = 1;
  const int row_bytes = K * (op == FG_OP_W8A16_NK ? 1 : 2);
  int rows = FG_GEMV_MAX_OUT;
  while (rows > 1 && (rows * row_bytes > FG_GEMV_STAGE_TARGET_BYTES || rows * M > FG_GEMV_MAX_OUT)) rows >>= 1;
  p.rows_per_stage = rows;
  p.k_per_stage = K;       // a stage holds whole rows
  p.k_blocks = 1;
  const int stage_bytes = rows * row_bytes;
  const int fit = std::min((smem_optin_bytes - fg_gemv_fixed_smem_bytes(M, K)) / (stage_bytes + 24), FG_MAX_STAGES);
  if (fit < 3) return FG_ERR_PLAN;  // rows too long for a useful ring: the tiled kernels take over
  // ring depth: up to three slots are given up for a depth that more warps divide
  int best_s = fit, best_w = fg_gemv_warps(fit);
  for (int s2 = fit - 1; s2 >= 3 && s2 >= fit - 3; --s2)
    if (fg_gemv_warps(s2) > best_w) {
      best_w = fg_gemv_warps(s2);
      best_s = s2;
    }
  if (op == FG_OP_F16_NK && M == 1) {
    // One token row of fp16 weights: five to nine warps with two or three ring slots each beat twelve
    // warps with one slot each wherever the ring is deep enough to choose (measured on B200, us per call,
    // twelve warps against this rule: 8192 x 8192 22.7 / 21.7, 11008 x 4096 15.4 / 13.9, 4096 x 4096
    // 8.9 / 8.3, 8192 x 7168 20.0 / 18.5, 8192 x 2048 8.4 / 7.8; 8192 x 6144 and 8192 x 5120 are unchanged
    // at 16 slots / 8 warps and 21 / 7).  A warp multiplies about 12 GB/s, an SM receives 47 GB/s:
    // more warps than that needs only add contention for the issue slots and shared memory.
    for (int s2 = fit; s2 >= 3 && s2 >= fit - 3; --s2) {
      int w = 0;
      for (int c = FG_GEMV_PREF_WARPS_MAX; c >= FG_GEMV_PREF_WARPS_MIN; --c)
        if (s2 % c == 0) {
          w = c;
          break;
        }
      if (w != 0) {
        best_s = s2;
        best_w = w;
        break;
      }
    }
  }
  p.stages = best_s;
  p.consumer_warps = best_w;
  const int blocks = (N + rows - 1) / rows;
  p.grid = std::min(std::min(sm_count, FG_MAX_GRID), blocks);
  // a fixed share first (its first ring-full needs no counter), the rest dealt out on demand
  p.static_rows = static_cast<int>(static_cast<long long>(N) * FG_GEMV_STATIC_PCT / 100 / p.grid) / rows * rows;
  p.smem_bytes = fg_gemv_smem_bytes(M, K, stage_bytes, p.stages);
  *out = p;
  return FG_OK;
}

// Small fp16 problems: a grid of tiles x s CTAs, s a divisor of the stages per tile, gives every CTA
// exactly one segment of one tile (one partial tile, one ticket, a reduction over exactly s
// contributors) instead of two segments in two tiles for most CTAs of a grid that only balances
// bytes.  Measured on B200 (us per call, all SMs against the aligned grid): 4096 x 4096 M = 16 12.9 / 11.6,
// 3072 x 3072 10.8 / 9.6, 2048 x 8192 14.2 / 12.8, 4096 x 2048 9.9 / 9.0; KxN weights, M = 8: 4096 x 4096
// 12.6 / 11.4, 3072 x 3072 10.8 / 8.6, 1152 x 3072 11.3 / 8.8.  Above about 80 MB of weights a CTA streams so
// many stages that the balance of bytes matters more (8192 x 8192 loses 0.9 us on 128 CTAs).
// Preference: the largest such grid that leaves a CTA at least 192 KB of weights, else at least 96 KB;
// never fewer than 48 % of the SMs, and 60 % above 40 MB of weights (5120 x 5120 on 80 CTAs and 7168 x 4096
// on 112 are level with all SMs or slower; 6144 x 4096 on 96, 4096 x 8192 on 128 and 6144 x 6144 on 144
// gain 3-10 %).  Returns 0 when nothing qualifies.
static int aligned_grid(int tiles, int k_blocks, long long stage_bytes, int sm_count) {
  const long long weight_bytes = static_cast<long long>(tiles) * k_blocks * stage_bytes;
  if (weight_bytes > FG_ALIGNED_GRID_MAX_BYTES) return 0;
  const int limit = std::min(sm_count, FG_MAX_GRID);
  for (long long per_cta : {196608LL, 98304LL}) {
    int best = 0;
    for (int s = 2; s <= k_blocks; ++s) {
      if (k_blocks % s) continue;
      const long long g = static_cast<long long>(tiles) * s;
      if (g > limit || g * 100 < (weight_bytes > FG_ALIGNED_GRID_SMALL_BYTES ? 60LL : 48LL) * sm_count) continue;
      if ((k_blocks / s) * stage_bytes < per_cta) continue;
      if (g > best) best = static_cast<int>(g);
    }
    if (best) return best;
  }
  return 0;
}

static int plan_impl(int op, int M, int N, int K, int sm_count, int smem_optin_bytes, fg_plan_t* out,
                     bool force_mma_sync, bool allow_gemv) {
  if (out == nullptr) return FG_ERR_NULL;
  std::memset(out, 0, sizeof(*out));
  if (op < FG_OP_F16_KN || op > FG_OP_W4A16_NK) return FG_ERR_PLAN;
  if (M <= 0 || N <= 0 || K <= 0 || (N % 128) != 0 || (K % 128) != 0) return FG_ERR_SHAPE;
  if (sm_count <= 0) sm_count = 148;                 // B200
  if (smem_optin_bytes <= 0) smem_optin_bytes = 232448;  // 227 KB opt-in per CTA on sm_100

  // Two rows: the GEMV kernel wins on every shape measured up to 96 MB of weights (11008 x 4096: 17.0 us
  // against 17.8 tiled; 3072 x 12288: 17.7 / 18.1; 9216 x 3072: 12.3 / 12.8) and ties at 8192 x 8192
  // (24.1 / 24.0), where a step that alternates it with tiled calls loses 0.6 us per call.
  if (allow_gemv && gemv_eligible(op, M, K) && (M == 1 || static_cast<long long>(N) * K <= FG_GEMV_M2_MAX_ELEMS)) {
    const int st = plan_gemv(op, M, N, K, sm_count, smem_optin_bytes, out);
    if (st == FG_OK) return st;  // no room for a ring: fall through to the tiled kernels
  }

  fg_plan_t p;
  std::memset(&p, 0, sizeof(p));
  p.op = op;
  const bool quantized = (op == FG_OP_W8A16_NK || op == FG_OP_W4A16_NK);
  p.passes = (M + 15) / 16;
  // accumulator tile height of the (last) pass; earlier passes of a multi-pass call use 16
  const int m_last = M - (p.passes - 1) * 16;
  p.m_tile = (p.passes == 1 && m_last <= 8) ? 8 : 16;
  if (!quantized && M > 16) {
    // fp16 weights: the tcgen05 kernel takes up to 64 token rows per pass over the weight
    p.passes = (M + FG_MAX_M_TILE - 1) / FG_MAX_M_TILE;
    p.m_tile = (M <= 32) ? 32 : 64;
  }
  p.math = 0;
  p.tiles = N / 128;

  const int chunk_k = fg_chunk_k(op);
  // KxN weights up to 8 rows: the mma.sync kernel up to 40 MB of weights (measured at M = 8: 3072 x 3072 8.6 us against
  // 9.6 for the tcgen05 kernel, 4096 x 2048 8.7 / 9.0, 4096 x 4096 11.4 / 11.5), the tcgen05 kernel above (5120 x 5120
  // 17.7 / 14.9, 8192 x 4096 16.8 / 15.4, 11008 x 4096 20.0 / 18.4, 8192 x 8192 25.8 / 24.8)
  const bool kn_large = (op == FG_OP_F16_KN && static_cast<long long>(N) * K * 2 > FG_ALIGNED_GRID_SMALL_BYTES);
  if (!quantized && (p.m_tile >= 16 || op == FG_OP_F16_NK || kn_large)) {
    // NxK fp16 weights at every M, KxN above 8 token rows (measured: with 64 KB stages the tcgen05
    // kernel is 1.5-5 % faster than the mma.sync one for NxK at M = 1 and 8 on 8192^2, 11008 x 4096,
    // 4096 x 11008 and 3072^2, and 3 % slower for KxN at 4096^2): the tcgen05 kernel (accumulator in tensor memory,
    // no cross-warp reduction, the whole shared memory is ring).  Its single MMA-issuing
    // thread pays a fixed cost per stage, so stages are as large as the ring allows: measured
    // on B200 at M = 16, 64 KB stages (3 in the ring) beat 32 KB (6) beat 16 KB (12) for every
    // shape tried, from 8192 x 8192 (24.5 / 26.0 / 32.8 us) down to 1024 x 1024 (7.2 / 7.9 / 9.5)
    // and 9216 x 3072 (13.6 / 16.1 / 19.7), although small layers then get only two or three
    // stages per CTA.
    p.math = 2;
    if (p.m_tile < 16) p.m_tile = 16;  // rows beyond M are zero-filled by the TMA
    p.consumer_warps = 4;  // epilogue warps, fixed
    int chunks = 4;
    while (chunks > 1 && chunks * chunk_k > K) chunks >>= 1;  // a stage never spans more than K
    p.k_per_stage = chunks * chunk_k;
    p.k_blocks = (K + p.k_per_stage - 1) / p.k_per_stage;
    const long long units = static_cast<long long>(p.tiles) * p.k_blocks;
    p.grid = static_cast<int>(std::min<long long>(std::min(sm_count, FG_MAX_GRID), units));
    if (units * p.grid >= (1LL << 31)) return FG_ERR_SHAPE;
    int stage_bytes = chunks * fg_chunk_bytes(op, p.m_tile);
    p.stages = std::min((smem_optin_bytes - 1024 - 64) / (stage_bytes + 16), FG_MAX_STAGES);
    // Taller activation tiles: stages shrink one chunk at a time until the ring is three deep
    // (measured at M = 32 / 64, 8192 x 8192: three chunks x 3 stages 26.9 / 30.6 us, two chunks
    // x 5 / 4 stages 27.5 / 31.6 us, four chunks x 2 stages 27.0 / 30.7 us).
    while (p.stages < 3 && chunks > 1) {
      chunks -= 1;
      p.k_per_stage = chunks * chunk_k;
      p.k_blocks = (K + p.k_per_stage - 1) / p.k_per_stage;
      stage_bytes = chunks * fg_chunk_bytes(op, p.m_tile);
      p.stages = std::min((smem_optin_bytes - 1024 - 64) / (stage_bytes + 16), FG_MAX_STAGES);
    }
    if (p.stages < 2) return FG_ERR_PLAN;
    {
      const long long units2 = static_cast<long long>(p.tiles) * p.k_blocks;
      p.grid = static_cast<int>(std::min<long long>(std::min(sm_count, FG_MAX_GRID), units2));
      if (units2 * p.grid >= (1LL << 31)) return FG_ERR_SHAPE;
      const int g = aligned_grid(p.tiles, p.k_blocks, static_cast<long long>(chunks) * FG_CHUNK_W_BYTES, sm_count);
      if (g) p.grid = g;
    }
    p.pdl = 1;
    p.smem_bytes = fg_umma_smem_bytes_mt(op, p.m_tile, chunks, p.stages);
    *out = p;
    return FG_OK;
  }
  if (quantized && p.m_tile == 16 && !force_mma_sync) {
    // Quantized weights, more than 8 token rows: warps dequantise landed stages into fp16 staging
    // tiles for tcgen05.mma (fg_umma_q_kernel).  Measured on B200 at 28672 x 8192, M = 16: int8
    // 66 us against 70 us for the 16-row mma.sync kernel, int4 58 us against 86 us.  Up to 8 rows
    // the mma.sync kernel is as fast or faster (int8 follows HBM there).
    p.math = 2;
    p.m_tile = 16;
    p.consumer_warps = 4;
    const int chunks = 1;  // 16 KB of packed weights per stage: the ring is short (64 KB go to staging)
    p.k_per_stage = chunks * chunk_k;
    p.k_blocks = (K + p.k_per_stage - 1) / p.k_per_stage;
    const long long units = static_cast<long long>(p.tiles) * p.k_blocks;
    p.grid = static_cast<int>(std::min<long long>(std::min(sm_count, FG_MAX_GRID), units));
    if (units * p.grid >= (1LL << 31)) return FG_ERR_SHAPE;
    const int stage_bytes = chunks * fg_chunk_bytes(op, 16);
    p.stages = std::min((smem_optin_bytes - 1024 - 160 - FG_UMMA_Q_STAGING_BYTES) / (stage_bytes + 16), FG_MAX_STAGES);
    if (p.stages < 2) return FG_ERR_PLAN;
    p.pdl = 1;
    p.smem_bytes = fg_umma_q_smem_bytes(op, chunks, p.stages);
    *out = p;
    return FG_OK;
  }
  // One 16 KB weight chunk per stage: measured on B200, deeper rings of small stages beat
  // fewer large ones for every shape tried (the ring is what a dependent launch prefetches
  // while its predecessor drains).
  const int chunks = 1;
  p.k_per_stage = chunks * chunk_k;
  p.k_blocks = (K + p.k_per_stage - 1) / p.k_per_stage;
  const long long units = static_cast<long long>(p.tiles) * p.k_blocks;
  p.grid = static_cast<int>(std::min<long long>(std::min(sm_count, FG_MAX_GRID), units));
  if (units * p.grid >= (1LL << 31)) return FG_ERR_SHAPE;  // beyond the kernel's 32-bit index math
  if (!quantized) {
    const int g = aligned_grid(p.tiles, p.k_blocks, static_cast<long long>(chunks) * FG_CHUNK_W_BYTES, sm_count);
    if (g) p.grid = g;
  }

  // Consumer warps, from sweeps on B200: the int8 path is happiest with 3 (its dequantising
  // inner loop keeps the issue slots busy), int4 with 5 (28672 x 8192, M = 8: 61 / 55 / 52 / 54.5 us
  // with 3 / 4 / 5 / 6 warps), fp16 with 4 for an 8-row tile and 8 for 16 rows.
  // A ring stage is always consumed by the same warp (stage s belongs to warp s % warps),
  // which needs stages % warps == 0: a warp then sees every phase of the barriers it waits
  // on.  The ring takes all the shared memory that is left.
  int warps = (op == FG_OP_W8A16_NK) ? 3 : (op == FG_OP_W4A16_NK) ? (p.m_tile == 16 ? 3 : 5) : (p.m_tile == 16 ? 8 : 4);
  const int stage_bytes = chunks * fg_chunk_bytes(op, p.m_tile);
  int stages = 0;
  for (; warps >= 1; --warps) {
    const int fixed = fg_fixed_smem_bytes(warps, p.m_tile);
    stages = (smem_optin_bytes - fixed) / (stage_bytes + 16);
    stages = std::min(stages, FG_MAX_STAGES) / warps * warps;
    if (stages >= 2 && stages >= warps) break;
  }
  if (warps < 1) return FG_ERR_PLAN;
  p.consumer_warps = warps;
  p.stages = stages;
  p.pdl = 1;
  p.smem_bytes = fg_smem_bytes(op, p.m_tile, chunks, p.stages, p.consumer_warps);
  *out = p;
  return FG_OK;
}

// Checks a (possibly hand-edited) plan against the limits the kernel relies on.
extern "C" int fg_plan_validate(const fg_plan_t* p, int N, int K, int smem_optin_bytes) {
  if (p == nullptr) return FG_ERR_NULL;
  if (smem_optin_bytes <= 0) smem_optin_bytes = 232448;
  if (p->op < FG_OP_F16_KN || p->op > FG_OP_W4A16_NK) return FG_ERR_PLAN;
  if (p->math == 4) {
    // row-split GEMV kernel
    if (p->m_tile < 1 || p->m_tile > FG_GEMV_MAX_M || !gemv_eligible(p->op, p->m_tile, K)) return FG_ERR_PLAN;
    if (p->rows_per_stage != 1 && p->rows_per_stage != 2 && p->rows_per_stage != 4 && p->rows_per_stage != 8) return FG_ERR_PLAN;
    if (p->rows_per_stage * p->m_tile > FG_GEMV_MAX_OUT) return FG_ERR_PLAN;
    const int row_bytes = K * (p->op == FG_OP_W8A16_NK ? 1 : 2);
    const long long stage_bytes = static_cast<long long>(p->rows_per_stage) * row_bytes;
    if (stage_bytes > FG_GEMV_MAX_STAGE_BYTES) return FG_ERR_PLAN;
    if (p->stages < 2 || p->stages > FG_MAX_STAGES) return FG_ERR_PLAN;
    if (p->consumer_warps < 1 || p->consumer_warps > FG_GEMV_MAX_WARPS || p->stages % p->consumer_warps) return FG_ERR_PLAN;
    if (p->k_per_stage != K || p->k_blocks != 1 || p->tiles != N / 128 || p->passes != 1) return FG_ERR_PLAN;
    if (p->grid < 1 || p->grid > FG_MAX_GRID) return FG_ERR_PLAN;
    if (p->static_rows < 0 || p->static_rows % p->rows_per_stage ||
        static_cast<long long>(p->static_rows) * p->grid > N) return FG_ERR_PLAN;
    if (p->smem_bytes != fg_gemv_smem_bytes(p->m_tile, K, static_cast<int>(stage_bytes), p->stages)) return FG_ERR_PLAN;
    if (p->smem_bytes > smem_optin_bytes) return FG_ERR_PLAN;
    return FG_OK;
  }
  const bool quantized = (p->op == FG_OP_W8A16_NK || p->op == FG_OP_W4A16_NK);
  if (p->m_tile != 8 && p->m_tile != 16 && p->m_tile != 32 && p->m_tile != 64) return FG_ERR_PLAN;
  if (p->m_tile > 16 && (p->math != 2 || p->op > FG_OP_F16_NK)) return FG_ERR_PLAN;  // tall tiles: fp16 tcgen05 kernel only
  if (p->math != 0 && p->math != 2) return FG_ERR_PLAN;
  const int chunk_k = fg_chunk_k(p->op);
  if (p->k_per_stage <= 0 || p->k_per_stage % chunk_k) return FG_ERR_PLAN;
  const int chunks = p->k_per_stage / chunk_k;
  if (chunks < 1 || chunks > 4) return FG_ERR_PLAN;
  if (p->stages < 2 || p->stages > FG_MAX_STAGES) return FG_ERR_PLAN;
  if (p->math == 2) {
    // tcgen05 variants: 16-row accumulator in tensor memory, fixed warp roles
    if (p->m_tile < 16) return FG_ERR_PLAN;
    if (quantized && (chunks > 4 || p->m_tile != 16)) return FG_ERR_PLAN;
  } else {
    if (p->consumer_warps < 1 || p->consumer_warps > FG_MAX_CONSUMER_WARPS) return FG_ERR_PLAN;
    // the dequantising kernels are built for <= 6 consumer warps (<= 3 with a 16-row tile)
    if (quantized && p->consumer_warps > (p->m_tile == 16 ? 3 : 6)) return FG_ERR_PLAN;
    // each stage must always meet the same consumer warp (see fg_plan)
    if (p->stages % p->consumer_warps) return FG_ERR_PLAN;
  }
  if (p->tiles != N / 128) return FG_ERR_PLAN;
  if (p->k_blocks != (K + p->k_per_stage - 1) / p->k_per_stage) return FG_ERR_PLAN;
  const long long units = static_cast<long long>(p->tiles) * p->k_blocks;
  if (p->grid < 1 || p->grid > FG_MAX_GRID || p->grid > units) return FG_ERR_PLAN;
  if (units * p->grid >= (1LL << 31)) return FG_ERR_PLAN;  // the kernel's index math is 32-bit
  const int want_smem = (p->math == 2) ? (quantized ? fg_umma_q_smem_bytes(p->op, chunks, p->stages)
                                                    : fg_umma_smem_bytes_mt(p->op, p->m_tile, chunks, p->stages))
                                       : fg_smem_bytes(p->op, p->m_tile, chunks, p->stages, p->consumer_warps);
  if (p->smem_bytes != want_smem) return FG_ERR_PLAN;
  if (p->smem_bytes > smem_optin_bytes) return FG_ERR_PLAN;
  return FG_OK;
}
