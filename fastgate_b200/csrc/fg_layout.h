// Sizes shared by the host-side planner and the device kernel: how a pipeline stage,
// the shared-memory carve-up and the workspace are laid out.
#pragma once
#include <stddef.h>

#define FG_MAX_GRID 256            /* persistent CTAs the workspace has room for        */
#define FG_MAX_STAGES 24           /* ring depth limit                                  */
#define FG_L2_PREFETCH_BYTES 98304 /* weights per CTA asked into L2 while it waits for the previous kernel */
#define FG_MAX_CONSUMER_WARPS 8
#define FG_TILE_N 128              /* output columns per tile                           */
#define FG_CHUNK_W_BYTES 16384     /* weight bytes per chunk                            */
#define FG_RED_STRIDE 132          /* floats per row of the cross-warp reduction buffer */

/* Workspace: [0,256) header (status word at 0, the GEMV kernel's counters at 64 and 128); then
 * FG_MAX_GRID x 2 partial tiles of up to 64 x 128 fp32; then one 32-bit arrival counter per
 * output tile. */
#define FG_WS_HEADER_BYTES 256
#define FG_MAX_M_TILE 64           /* tallest accumulator tile (tcgen05 fp16 kernel)    */
#define FG_WS_PARTIAL_TILE_BYTES (FG_MAX_M_TILE * FG_TILE_N * 4)
#define FG_WS_PARTIAL_TILE16_BYTES (16 * FG_TILE_N * 4) /* kernels that never exceed 16 rows */
#define FG_WS_PARTIALS_BYTES ((size_t)FG_MAX_GRID * 2 * FG_WS_PARTIAL_TILE_BYTES)
#define FG_WS_TICKETS_OFFSET (FG_WS_HEADER_BYTES + FG_WS_PARTIALS_BYTES)

/* op codes mirror FG_OP_* of the public header */
static inline int fg_chunk_k(int op) { return op == 3 ? 256 : op == 2 ? 128 : 64; }
/* activation boxes (64 k x m_tile rows, 128 B per row) that accompany one weight chunk */
static inline int fg_x_boxes(int op) { return op == 3 ? 4 : op == 2 ? 2 : 1; }
static inline int fg_chunk_bytes(int op, int m_tile) {
  return FG_CHUNK_W_BYTES + fg_x_boxes(op) * m_tile * 128;
}
/* reduction buffer + 1 KB alignment slack + two hand-off barriers and the finishers' ticket
 * word (the ring's barriers are counted per stage) */
static inline int fg_fixed_smem_bytes(int consumer_warps, int m_tile) {
  return 1024 + consumer_warps * m_tile * FG_RED_STRIDE * 4 + 32;
}
static inline int fg_smem_bytes(int op, int m_tile, int chunks, int stages, int consumer_warps) {
  return fg_fixed_smem_bytes(consumer_warps, m_tile) + stages * (chunks * fg_chunk_bytes(op, m_tile) + 16);
}

/* row-split GEMV kernel (math 4): x, ring of whole-row stages, cross-warp sums, stage table, barriers */
#define FG_GEMV_MAX_M 2
#define FG_GEMV_M2_MAX_ELEMS (48LL << 20) /* two rows: only up to this many weights (96 MB) */
#define FG_GEMV_MAX_OUT 8                /* rows per stage x token rows */
#define FG_GEMV_MAX_WARPS 12             /* consumer warps; each owns every warps-th stage */
#define FG_GEMV_PREF_WARPS_MIN 5         /* one row of fp16 weights: the planner looks for a ring depth that this many ... */
#define FG_GEMV_PREF_WARPS_MAX 9         /* ... to this many warps divide */
#define FG_GEMV_MIN_K 1024
#define FG_GEMV_STAGE_TARGET_BYTES 16384 /* as many rows per stage as fit in this */
#define FG_GEMV_MAX_STAGE_BYTES 65536    /* a stage holds at least one whole row */
#define FG_GEMV_STATIC_PCT 100           /* share of the rows dealt out up front (whole stages); the rest on demand */
#define FG_GEMV_L2_PREFETCH_BYTES 98304
/* workspace header words of the GEMV kernel's row-block counter and exit counter */
#define FG_WS_GEMV_NEXT_OFFSET 64
#define FG_WS_GEMV_EXITED_OFFSET 128
static inline int fg_gemv_fixed_smem_bytes(int M, int K) { return 127 + ((M * K * 2 + 127) & ~127) + 8; }
/* per stage: the rows, the stage's row range, two barriers */
static inline int fg_gemv_smem_bytes(int M, int K, int stage_bytes, int stages) {
  return fg_gemv_fixed_smem_bytes(M, K) + stages * (stage_bytes + 8 + 16);
}
/* Consumer warps for a ring of `stages` slots: the largest divisor of stages up to FG_GEMV_MAX_WARPS
 * (a slot must always meet the same warp). */
static inline int fg_gemv_warps(int stages) {
  int w = stages < FG_GEMV_MAX_WARPS ? stages : FG_GEMV_MAX_WARPS;
  while (w > 1 && stages % w) --w;
  return w;
}

/* tcgen05 variant for quantized weights: ring, 32 KB fp16 staging buffers, barriers */
#ifdef __cplusplus
struct fg_plan_t;
extern "C" int fg_plan_mma_sync(int op, int M, int N, int K, int sm_count, int smem_optin_bytes,
                                struct fg_plan_t* out); /* quantized ops: the mma.sync kernel's plan for any M */
extern "C" int fg_plan_tiled(int op, int M, int N, int K, int sm_count, int smem_optin_bytes,
                             struct fg_plan_t* out);    /* never the row-split GEMV kernel */
#endif
#define FG_UMMA_Q_STAGING_BYTES 98304 /* three 32 KB buffers */
static inline int fg_umma_q_smem_bytes(int op, int chunks, int stages);

/* fp16 weights up to this size get a grid of tiles x s CTAs (every CTA one segment of one tile) */
#define FG_ALIGNED_GRID_MAX_BYTES (80LL << 20)
/* ... and what counts as a small problem there (smaller grids allowed; KxN weights up to 8 rows stay on the mma.sync kernel) */
#define FG_ALIGNED_GRID_SMALL_BYTES (40LL << 20)
/* tcgen05 variant: ring + barriers only (the accumulators live in tensor memory) */
static inline int fg_umma_smem_bytes_mt(int op, int m_tile, int chunks, int stages) {
  return 1024 + stages * (chunks * fg_chunk_bytes(op, m_tile) + 16) + 64;
}
static inline int fg_umma_smem_bytes(int op, int chunks, int stages) {
  return fg_umma_smem_bytes_mt(op, 16, chunks, stages);
}
/* token rows one launch covers: 64 for the fp16 tcgen05 kernel, 16 otherwise */
static inline int fg_pass_rows(int op, int math) { return (math == 2 && op <= 1) ? FG_MAX_M_TILE : 16; }
static inline int fg_umma_q_smem_bytes(int op, int chunks, int stages) {
  return 1024 + stages * (chunks * fg_chunk_bytes(op, 16) + 16) + FG_UMMA_Q_STAGING_BYTES + 160;
}
