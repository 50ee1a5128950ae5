// Launch heuristic: pure host code, no CUDA calls, so it can be unit-tested on a box
// without a GPU.  It replaces the reference's split-K choice
// (backend/cuda/hk/edgemm.cu:287-305: BZ from tile-count thresholds 64/32 tuned for a
// 108-SM part, clamped by K % {1024,512,256}); script/heuristics.py is empty there.
//
// Here there is no split-K factor to pick: the (tile, k-block) list is dealt evenly to
// one persistent CTA per SM, so the plan only fixes the pipeline shape.
#include <algorithm>
#include <cstring>

#include "../../include/fastgate_b200.h"
#include "fg_layout.h"

extern "C" int fg_plan(int op, int M, int N, int K, int sm_count, int smem_optin_bytes,
                       fg_plan_t* out) {
  if (out == nullptr) return FG_ERR_NULL;
  std::memset(out, 0, sizeof(*out));
  if (op < FG_OP_F16_KN || op > FG_OP_W8A16_NK) return FG_ERR_PLAN;
  if (M <= 0 || N <= 0 || K <= 0 || (N % 128) != 0 || (K % 128) != 0) return FG_ERR_SHAPE;
  if (sm_count <= 0) sm_count = 148;                 // B200
  if (smem_optin_bytes <= 0) smem_optin_bytes = 232448;  // 227 KB opt-in per CTA on sm_100

  fg_plan_t p;
  std::memset(&p, 0, sizeof(p));
  p.op = op;
  p.passes = (M + 15) / 16;
  // accumulator tile height of the (last) pass; earlier passes of a multi-pass call use 16
  const int m_last = M - (p.passes - 1) * 16;
  p.m_tile = (p.passes == 1 && m_last <= 8) ? 8 : 16;
  p.math = 0;
  p.tiles = N / 128;

  const int chunk_k = fg_chunk_k(op);
  // Two 16 KB weight chunks per stage halve the number of barrier round trips; one chunk
  // per stage keeps more, smaller stages in flight when a CTA has little work.
  int chunks = 2;
  const long long units1 = static_cast<long long>(p.tiles) * ((K + chunk_k - 1) / chunk_k);
  if (units1 < 8LL * sm_count) chunks = 1;
  p.consumer_warps = 4;

  p.k_per_stage = chunks * chunk_k;
  p.k_blocks = (K + p.k_per_stage - 1) / p.k_per_stage;
  const long long units = static_cast<long long>(p.tiles) * p.k_blocks;
  p.grid = static_cast<int>(std::min<long long>(std::min(sm_count, FG_MAX_GRID), units));

  const int stage_bytes = chunks * fg_chunk_bytes(op, p.m_tile);
  const int fixed = fg_fixed_smem_bytes(p.consumer_warps, p.m_tile);
  int stages = (smem_optin_bytes - fixed) / (stage_bytes + 16);
  stages = std::min(stages, FG_MAX_STAGES);
  // no point in a ring deeper than the work of one CTA
  const long long per_cta = (units + p.grid - 1) / p.grid;
  stages = static_cast<int>(std::min<long long>(stages, std::max<long long>(per_cta, 2)));
  if (stages < 2) return FG_ERR_PLAN;
  p.stages = stages;
  p.smem_bytes = fg_smem_bytes(op, p.m_tile, chunks, stages, p.consumer_warps);
  *out = p;
  return FG_OK;
}

// Checks a (possibly hand-edited) plan against the limits the kernel relies on.
extern "C" int fg_plan_validate(const fg_plan_t* p, int N, int K, int smem_optin_bytes) {
  if (p == nullptr) return FG_ERR_NULL;
  if (smem_optin_bytes <= 0) smem_optin_bytes = 232448;
  if (p->op < FG_OP_F16_KN || p->op > FG_OP_W8A16_NK) return FG_ERR_PLAN;
  if (p->m_tile != 8 && p->m_tile != 16) return FG_ERR_PLAN;
  const int chunk_k = fg_chunk_k(p->op);
  if (p->k_per_stage <= 0 || p->k_per_stage % chunk_k) return FG_ERR_PLAN;
  const int chunks = p->k_per_stage / chunk_k;
  if (chunks < 1 || chunks > 4) return FG_ERR_PLAN;
  if (p->consumer_warps < 1 || p->consumer_warps > FG_MAX_CONSUMER_WARPS) return FG_ERR_PLAN;
  if (p->stages < 2 || p->stages > FG_MAX_STAGES) return FG_ERR_PLAN;
  if (p->tiles != N / 128) return FG_ERR_PLAN;
  if (p->k_blocks != (K + p->k_per_stage - 1) / p->k_per_stage) return FG_ERR_PLAN;
  const long long units = static_cast<long long>(p->tiles) * p->k_blocks;
  if (p->grid < 1 || p->grid > FG_MAX_GRID || p->grid > units) return FG_ERR_PLAN;
  if (p->smem_bytes != fg_smem_bytes(p->op, p->m_tile, chunks, p->stages, p->consumer_warps))
    return FG_ERR_PLAN;
  if (p->smem_bytes > smem_optin_bytes) return FG_ERR_PLAN;
  return FG_OK;
}
