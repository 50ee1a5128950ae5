/*
 * fastgate_b200 — C ABI of the B200 (sm_100a) small-batch matmul library.
 *
 * Everything a non-PyTorch caller needs is here: plain pointers and sizes, an
 * explicit cudaStream_t, an explicit caller-owned workspace, int status codes.
 * No entry point throws, exits, synchronises the device or allocates device
 * memory, unless its comment says so.
 *
 * The library replaces the host launchers of chanzhennan/Fastgate
 * (reference paths below are relative to that project):
 *
 *   backend/cuda/hk/edgemm.cu:102-156    edgemm_m8n128k64x4      C[M,N] = A[M,K] . B[K,N]
 *   backend/cuda/hk/edgemm.cu:274-324    edgemm_m8n128k64x4_bt   C[M,N] = A[M,K] . W[N,K]^T
 *   backend/cuda/hk/fastgemv.cu:12-33    fastgemv                y[N]   = W[N,K] . x[K]
 *   backend/cuda/hk/fastgemv.cu:35-61    fastgemv_int8           y[N]   = s * W8[N,K] . x[K]
 *   backend/cuda/hk/fastgemv.cu:86-111   fastgemv_extend         C[M,N] = x[M,K] . W[N,K]^T
 *   backend/cuda/czn/fastgemm.cu:13-55   fastgemm                same, M in {1,2}
 *   backend/cuda/hk/flatgemm.cu:13-169   flat_gemm_*             KxN weights
 *   backend/cuda/hk/edgemm_tr.cu:19-139  gemm_*_bt               NxK weights
 *
 * All matrices are dense row-major.  fp16 is IEEE binary16 ("half").
 * Contract shared with the reference (hk/edgemm.cu:107-109): K % 128 == 0 and
 * N % 128 == 0, otherwise FG_ERR_SHAPE.  M may be any positive number: one pass
 * over the weight serves up to 64 token rows of fp16 weights and up to 16 rows of
 * quantized weights; a larger M takes fg_plan_t.passes launches.
 * Results overwrite C (C = A.B); accumulation is fp32, one rounding to fp16.
 */
#ifndef FASTGATE_B200_H_
#define FASTGATE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* cudaStream_t without pulling in the CUDA headers. */
typedef struct CUstream_st* fg_stream_t;

/* ---- status codes -------------------------------------------------------- */
enum {
  FG_OK = 0,
  FG_ERR_SHAPE = 1,     /* K or N not a multiple of 128, or a size <= 0        */
  FG_ERR_ALIGN = 2,     /* a pointer is not 16-byte aligned                    */
  FG_ERR_NULL = 3,      /* a required pointer is NULL                          */
  FG_ERR_WORKSPACE = 4, /* workspace missing, misaligned or too small          */
  FG_ERR_CUDA = 5,      /* a CUDA runtime/driver call failed (see fg_last_cuda_error) */
  FG_ERR_TIMEOUT = 6,   /* a bounded device-side wait gave up (read back with fg_workspace_status) */
  FG_ERR_PLAN = 7,      /* a caller-supplied plan is not launchable            */
  FG_ERR_NO_DEVICE = 8  /* no sm_100 device is current                         */
};

/* ---- operand layouts ------------------------------------------------------ */
enum {
  FG_OP_F16_KN = 0,  /* weight B[K,N] fp16  (edgemm_m8n128k64x4, flat_gemm_*)     */
  FG_OP_F16_NK = 1,  /* weight W[N,K] fp16  (edgemm_*_bt, gemm_*_bt, fastgemv*)   */
  FG_OP_W8A16_NK = 2, /* weight W8[N,K] int8 + optional fp16 scale per row of W8  */
  FG_OP_W4A16_NK = 3  /* weight W4[N,K/2] bytes, two unsigned 4-bit values each      */
};

/*
 * Launch plan: the replacement for the reference's split-K choice
 * (hk/edgemm.cu:287-305; script/heuristics.py is empty there).  The weight is cut
 * into 128-column output tiles times k_blocks stages; that list of units is dealt
 * out in equal contiguous ranges to `grid` persistent CTAs ("stream-K"), so every
 * SM streams the same number of bytes whatever N/128 is.
 */
typedef struct fg_plan_t {
  int op;            /* FG_OP_*                                               */
  int m_tile;        /* 8, 16, 32 or 64: token rows held per accumulator tile   */
  int k_per_stage;   /* K elements one (full) pipeline stage covers            */
  int stages;        /* depth of the shared-memory ring                        */
  int consumer_warps;/* warps doing the math (+1 warp issuing copies, + warps finishing split tiles) */
  int grid;          /* persistent CTAs                                        */
  int tiles;         /* N / 128                                                */
  int k_blocks;      /* ceil(K / k_per_stage): stages per output tile          */
  int smem_bytes;    /* dynamic shared memory per CTA                          */
  int passes;        /* launches per call: ceil(M / 64) for fp16 weights on the tcgen05 kernel,
                        ceil(M / 16) otherwise                                  */
  int math;          /* 0 = mma.sync tiles, accumulators in registers; 2 = tcgen05.mma, accumulator in
                        tensor memory; 4 = row-split GEMV kernel (mixed-precision FMA, whole weight
                        rows per CTA, no reduction between CTAs; fp16 NxK weights with M <= 2 or int8
                        weights with M = 1; then m_tile = M, k_per_stage = K, k_blocks = 1); 1 and 3
                        reserved                                                          */
  int pdl;           /* 1 = programmatic dependent launch: the kernel may start, and prefetch
                        weight tiles, while the previous kernel of the stream drains; it reads
                        activations and writes nothing before that kernel has completed       */
  int rows_per_stage;/* math 4: weight rows per ring stage (1, 2, 4 or 8); else 0         */
  int static_rows;   /* math 4: rows every CTA streams before it takes blocks of rows_per_stage
                        rows from the shared counter (a multiple of rows_per_stage); else 0 */
} fg_plan_t;

/* Pure host function (callable without a GPU): fills *out for a problem on a device
 * with sm_count SMs and smem_optin_bytes of opt-in shared memory per CTA (pass 0/0
 * for the B200 values 148 / 232448). */
int fg_plan(int op, int M, int N, int K, int sm_count, int smem_optin_bytes, fg_plan_t* out);
/* Checks a plan (e.g. one edited by a tuner) against the limits the kernel relies on. */
int fg_plan_validate(const fg_plan_t* plan, int N, int K, int smem_optin_bytes);

/* ---- workspace -------------------------------------------------------------
 * Split-K partial tiles and per-tile arrival counters live in caller-owned device
 * memory, 256-byte aligned.  fg_workspace_bytes() is an upper bound for any M and
 * K at the given N.  The workspace must be cleared once with fg_workspace_init()
 * before first use; after that every call leaves the counters at zero again,
 * so no memset is launched per call.  The exception is a call that reported
 * FG_ERR_TIMEOUT or FG_ERR_PLAN in the status word: a wait that gave up leaves its
 * counters as they were, so clear the workspace again with
 * fg_workspace_init() before the next call.  One workspace serves one stream at a
 * time: calls that may overlap on the GPU need separate workspaces. */
size_t fg_workspace_bytes(int N);
int fg_workspace_init(void* ws, size_t ws_bytes, fg_stream_t stream);
/* Synchronises `stream`, copies the device status word to *status_out (FG_OK,
 * FG_ERR_TIMEOUT, or FG_ERR_PLAN if a kernel refused a launch that did not fit its
 * parameters) and clears it. */
int fg_workspace_status(void* ws, int* status_out, fg_stream_t stream);

/* ---- compute entry points (device pointers) --------------------------------
 * replaces edgemm_m8n128k64x4 (hk/edgemm.cu:102-156) and the flat_gemm_* family
 * (hk/flatgemm.cu:13-169): A[M,K], B[K,N], C[M,N], all fp16. */
int fg_gemm_f16_kn(const void* A, const void* B, void* C, int M, int N, int K,
                   void* ws, size_t ws_bytes, fg_stream_t stream);

/* replaces edgemm_m8n128k64x4_bt (hk/edgemm.cu:274-324), gemm_*_bt
 * (hk/edgemm_tr.cu:19-139), fastgemv / fastgemv_extend (hk/fastgemv.cu:12-33,86-111)
 * and fastgemm (czn/fastgemm.cu:13-55): x[M,K], W[N,K], C[M,N], all fp16. */
int fg_gemm_f16_nk(const void* x, const void* W, void* C, int M, int N, int K,
                   void* ws, size_t ws_bytes, fg_stream_t stream);

/* replaces fastgemv_int8 (hk/fastgemv.cu:35-61): x[M,K] fp16, W8[N,K] int8,
 * scales[N] fp16 or NULL (NULL = the reference's effective scale 1, zero-point 0),
 * C[M,N] fp16 = (x . W8^T) * scales[n]. */
int fg_gemm_w8a16_nk(const void* x, const int8_t* W8, const void* scales, void* C,
                     int M, int N, int K, void* ws, size_t ws_bytes, fg_stream_t stream);

/* int4 weight-only GEMV/GEMM: x[M,K] fp16, W4[N,K/2] bytes, C[M,N] fp16 =
 *     sum over groups g of scales[n,g] * sum_{k in g} x[m,k] * (w4[n,k] - zero_point).
 * Byte j of a row holds k = 2j in its low and k = 2j+1 in its high nibble, unsigned 0..15: the
 * packing of uint4_2 (hk/utility.cuh:13-36) that gemv_quantized_int4 (hk/fastgemv.cuh:394-495)
 * reads.  That kernel has no host wrapper in the reference and takes ONE scale and zero point
 * for the whole matrix; here scales is [N, groups] fp16 with groups = 1 (one scale per output
 * channel) or K/128 (one per 128 consecutive k), or NULL (scale 1), and zero_point an integer
 * 0..15 (8 = symmetric).  The reference's scalar form is scales filled with one value. */
int fg_gemm_w4a16_nk(const void* x, const uint8_t* W4, const void* scales, int groups, int zero_point,
                     void* C, int M, int N, int K, void* ws, size_t ws_bytes, fg_stream_t stream);

/* Group-wise asymmetric-range quantiser for fg_gemm_w4a16_nk: W[N,K] fp16 -> W4[N,K/2] and
 * scales[N,groups] fp16, groups = 1 or K/128; per group scale = fp16(max|W| / 7) (1 for an
 * all-zero group), q = clamp(rint(W / scale) + 8, 0, 15), zero point 8.  No counterpart in the
 * reference (it only generates random nibbles, hk/utility.cu generate_random_int4_numbers). */
int fg_quantize_rows_w4(const void* W, uint8_t* W4, void* scales, int groups, int N, int K, fg_stream_t stream);

/* Same operation as fg_gemm_f16_nk for callers that cannot allocate device memory: a
 * plugin that is handed its buffers and nothing else, code running under a fixed memory
 * budget, a loop that may not enter the allocator.  It takes no workspace: the split-K
 * scratch (arrival counters and fp32 partial tiles, about 2.5 MB) is a static array inside
 * the library, present on every GPU that loads it until the process exits, and the call
 * itself allocates nothing (no cudaMalloc/cudaFree, no allocating library routine).
 *   - Limits: N <= 65536 and at most 160 persistent CTAs; beyond that FG_ERR_WORKSPACE.
 *   - The first call on a device looks up the array's device address; make that call
 *     before any stream capture involving this entry point.
 *   - All calls share the one array.  Each call first clears the status word and the
 *     counters on `stream`, so calls are correct back to back on one stream; calls that
 *     may overlap on the GPU (different streams, different host threads) race on it and
 *     must be serialised by the caller.
 * It has no counterpart in the reference, whose launchers allocate nothing and use
 * fp16 atomics on C instead of scratch (backend/cuda/hk/edgemm.cu:138-142). */
int fg_gemm_f16_nk_noalloc(const void* x, const void* W, void* C, int M, int N, int K,
                           fg_stream_t stream);
/* Synchronises `stream` and copies the status word that the last fg_gemm_f16_nk_noalloc call on the
 * current device left in the built-in scratch (FG_OK, FG_ERR_TIMEOUT or FG_ERR_PLAN) to *status_out.
 * The next call clears the word itself.  Allocates nothing; no counterpart in the reference. */
int fg_noalloc_status(int* status_out, fg_stream_t stream);

/* The fp16 and int8 operations with an explicit plan (from fg_plan, possibly edited):
 * used by the tuner and the tests that walk every plan the heuristic can emit.  int4 plans
 * are refused (FG_ERR_PLAN): that op needs its group count and zero point, which
 * fg_gemm_w4a16_nk takes. */
int fg_gemm_planned(const fg_plan_t* plan, const void* x, const void* W, const void* scales,
                    void* C, int M, int N, int K, void* ws, size_t ws_bytes, fg_stream_t stream);

/* ---- N-sharded layers over the GPUs of one box: fused all-gather ("push") --------------
 * The reference has no multi-GPU path.  Rank r of `world` holds rows [r*N_local,
 * (r+1)*N_local) of an NxK weight and computes C[:, r*N_local : (r+1)*N_local].  Instead of
 * a separate all-gather, the kernel's epilogue stores each finished 128-column tile straight
 * into the full output C[M, n_total] of EVERY rank (plain stores through NVLink peer
 * mappings: symmetric memory, CUDA IPC or cudaDeviceEnablePeerAccess) and then adds 1 to
 * counter [rank] of every rank's flag array (eight 64-bit counters, one per source rank).
 * A call by rank r adds N_local/128 * passes to counter [r] on every rank, where passes is
 * fg_plan(FG_OP_F16_NK, M, N_local, K, ...).passes = ceil(M/64) (every pass over the weight
 * delivers each of the rank's tiles once);
 * fg_push_wait enqueues a one-thread kernel that waits, for at most 2 s, until counters
 * [0, world) of the local flag array have all reached `target` (the caller keeps the running
 * total per rank), after which the full output is complete on this rank.  No rank's compute
 * kernel ever waits for another. */
typedef struct fg_peers_t {
  int world;                      /* 1..8 */
  int rank;
  long long n_total;              /* = world * N_local, row length of the full output */
  void* C[8];                     /* full output [M, n_total] fp16 of each rank, as mapped here */
  unsigned long long* flag[8];    /* flag array (8 x u64, zero at start) of each rank, as mapped here */
  /* Optional: the activations x are the pushed output of an earlier layer.  The kernel then
   * reads x only after counters [0, world) at wait_flags (this rank's flag array of that
   * layer) have reached wait_target; its weight tiles are already on their way by then.
   * NULL = x is ready when the call is enqueued. */
  const unsigned long long* wait_flags;
  unsigned long long wait_target;
  /* Optional: multicast mappings of the same two allocations (an NVLink multicast object bound
   * to every rank's output / flag array, e.g. the multicast_ptr of a torch symmetric-memory
   * handle).  When both are set, a finished tile is stored ONCE with multimem.st and signalled
   * with one multimem.red; the NVSwitch replicates them to all ranks (this one included), which
   * divides the NVLink egress of the push by world.  NULL = one store and one atomic per rank. */
  void* mc_C;
  unsigned long long* mc_flag;
  /* Optional: the running totals kept in device memory instead of by the caller, so that a stream
   * of pushes and waits can be captured in a CUDA graph and replayed (nothing in a launch then
   * changes from call to call).  target_dev: one 64-bit word of this rank's device memory, zero at
   * start, belonging to the output buffers this call pushes into; every launch of the call adds
   * N_local/128 to it (so it always holds what every source rank will have delivered once the
   * launches enqueued so far have run), for fg_push_wait_dev and for later calls that name it as
   * wait_target_dev.  wait_target_dev: with wait_flags set, the kernel reads its wait target from
   * this word (the target_dev of the layer that produced x) instead of wait_target, after the
   * launches before it in the stream have completed.  NULL = the caller counts (wait_target,
   * fg_push_wait). */
  unsigned long long* target_dev;
  const unsigned long long* wait_target_dev;
} fg_peers_t;

/* A layer's output buffers are written by every rank as soon as that rank's kernel runs: push
 * into the same buffers again only after every rank has finished reading the previous result
 * (the counters order a rank's reads after the pushes, not the next push after the reads); use
 * two alternating sets of buffers, or a barrier between rounds. */
int fg_gemm_f16_nk_push(const void* x, const void* W_shard, int M, int N_local, int K,
                        const fg_peers_t* peers, void* ws, size_t ws_bytes, fg_stream_t stream);
int fg_push_wait(const unsigned long long* my_flags, int world, unsigned long long target, void* ws,
                 fg_stream_t stream);
/* The same with the target read on the device from *target_dev (see fg_peers_t.target_dev) when the
 * wait runs. */
int fg_push_wait_dev(const unsigned long long* my_flags, int world, const unsigned long long* target_dev,
                     void* ws, fg_stream_t stream);
/* count (1..16) such waits as one launch: my_flags[i] / target_dev[i] are host arrays of device pointers. */
int fg_push_wait_dev_many(const unsigned long long* const* my_flags, const unsigned long long* const* target_dev,
                          int count, int world, void* ws, fg_stream_t stream);

/* ---- grouped launch: many independent problems, one kernel ---------------------------
 * count problems C_i[M_i,N_i] = x_i[M_i,K_i] . W_i^T (fp16, M_i <= 16, the usual 128
 * contract; op = FG_OP_F16_NK or FG_OP_F16_KN for all) run as ONE persistent launch: the
 * stages of all problems form one work list, so launch cost, DRAM ramp and the tail of split
 * tiles are paid once per group instead of once per problem.  For projections whose inputs do
 * not depend on each other (the DiT linear stack of the benchmark); layers that feed each
 * other stay separate calls.  No counterpart in the reference (one launch per operator).
 *
 * fg_group_create builds the tensor maps and uploads the problem table to table_dev (caller
 * owned device memory, 128-byte aligned, fg_group_table_bytes(count)); it synchronises (one
 * cudaMemcpy).  Pointers and shapes are frozen in the group; the data behind them may change
 * between runs.  With peers != NULL (world, rank and flag[] are used) every problem is one
 * rank's N-shard: finished tiles are pushed into peer_C[r] + column rank*N of every rank and
 * counter [rank] of every rank grows by fg_group_tiles() per run (see fg_gemm_f16_nk_push).
 * fg_group_run only launches (workspace as for the other entry points, with room for
 * fg_group_tiles() counters). */
typedef struct fg_problem_t {
  const void* x;       /* [M, K] fp16 */
  const void* W;       /* [N, K] (NK) or [K, N] (KN) fp16 */
  void* C;             /* [M, N] fp16; ignored when pushing */
  int M, N, K;
  void* peer_C[8];     /* pushing: full output [M, n_total] of every rank, as mapped here */
  long long n_total;   /* pushing: world * N */
  void* mc_C;          /* pushing: multicast mapping of the same outputs, or NULL (used only when
                          peers->mc_flag is set and every problem of the group has one) */
} fg_problem_t;
typedef struct fg_group fg_group_t;

size_t fg_group_table_bytes(int count);
int fg_group_create(int op, const fg_problem_t* problems, int count, const fg_peers_t* peers,
                    void* table_dev, size_t table_bytes, fg_group_t** out);
int fg_group_run(const fg_group_t* group, void* ws, size_t ws_bytes, fg_stream_t stream);
unsigned long long fg_group_tiles(const fg_group_t* group);
void fg_group_destroy(fg_group_t* group);

/* ---- dependent layer chain: a stack of projections that feed each other, one kernel ------
 * count layers C_i[M,N_i] = act(x_i[M,K_i] . W_i^T + bias_i) + residual_i (fp16, M <= 16, the
 * usual 128 contract, one op for all) run in order inside ONE persistent, cooperatively
 * launched kernel.  x_i may be the output of an earlier layer dep_i of the same chain, or a
 * column slice of it (row stride ldx): the kernel keeps streaming the next layer's weights
 * while the previous layer's last tiles drain and holds back only the activations, on a
 * per-layer counter of finished tiles (bounded wait, FG_ERR_TIMEOUT in the workspace status).
 * A launch per layer pays its fixed cost per layer; the chain pays it once.  No counterpart
 * in the reference (one launch per operator).
 *
 * Rules: dep < the layer's own index (or -1: x is ready when the launch starts); a layer may
 * overwrite a buffer only if it depends, directly or through its chain of dep, on every layer
 * that reads that buffer; residual may alias C (in place).  fg_chain_create builds the tensor
 * maps and uploads the layer table to table_dev (caller owned, 128-byte aligned,
 * fg_chain_table_bytes(count)); it synchronises.  fg_chain_run enqueues one small memset
 * (the per-layer counters) and the kernel; the workspace is the chain's own
 * (fg_chain_workspace_bytes, 256-byte aligned, cleared once with fg_workspace_init). */
typedef struct fg_layer_t {
  const void* x;         /* [M, K] fp16, row stride ldx elements (0: K) */
  const void* W;         /* [N, K] (NK) or [K, N] (KN) fp16, dense */
  void* C;               /* [M, N] fp16, row stride ldc elements (0: N) */
  const void* bias;      /* [N] fp16 or NULL */
  const void* residual;  /* [M, N] fp16, row stride ldr elements (0: N), or NULL */
  long long ldx, ldc, ldr;
  int M, N, K;
  int act;               /* FG_ACT_* */
  int dep;               /* index of the layer that produces x, or -1 */
} fg_layer_t;
typedef struct fg_chain fg_chain_t;

size_t fg_chain_table_bytes(int count);
int fg_chain_create(int op, const fg_layer_t* layers, int count, void* table_dev, size_t table_bytes,
                    fg_chain_t** out);
size_t fg_chain_workspace_bytes(const fg_chain_t* chain);
int fg_chain_run(const fg_chain_t* chain, void* ws, size_t ws_bytes, fg_stream_t stream);
/* With fg_trace_enable(1) a run also writes eight words per layer and CTA at
 * fg_chain_trace_offset() of the workspace, as unsigned long long [count][fg_chain_grid()][8]:
 * timestamps (ns) of activations ready, first stage landed, last stage committed, last tile or
 * partial handed on, last partial written, its ticket back, its reduction loaded; and the number
 * of contributors if this CTA reduced its last split tile (else 0). */
int fg_chain_grid(const fg_chain_t* chain);
size_t fg_chain_trace_offset(const fg_chain_t* chain);
void fg_chain_destroy(fg_chain_t* chain);

/* ---- fused epilogue ----------------------------------------------------------------------
 * The reference has no fused operator (no bias, activation or residual anywhere in
 * backend/cuda); at 10-25 us per call a separate elementwise kernel costs as much as the
 * GEMV itself, so the linear layers of its stated use (DiT / LLM inference) want
 *     C = act(x . W^T * scale + bias[n]) + residual[m, n]
 * evaluated in fp32 and rounded once.  Any of bias, residual may be NULL; ep == NULL is the
 * plain product.  op = FG_OP_*; scales only for FG_OP_W8A16_NK. */
enum { FG_ACT_NONE = 0, FG_ACT_GELU_ERF = 1, FG_ACT_GELU_TANH = 2, FG_ACT_SILU = 3, FG_ACT_SILU_GATE = 4 };
typedef struct fg_epilogue_t {
  const void* bias;      /* [N] fp16 */
  const void* residual;  /* [M, N] fp16 (row length = that of the output), added after the activation */
  int act;               /* FG_ACT_* */
  /* Output split (a fused QKV projection written straight into the consumer's three tensors):
   * with split1 > 0, columns [0, split1) go to C, [split1, split2) to C2 and [split2, N) to C3, each
   * a dense row-major tensor of its own width.  split1, split2 multiples of 8; split2 == N: two
   * outputs; all zero: one output. */
  int split1, split2;
  void* C2;
  void* C3;
} fg_epilogue_t;
/* FG_ACT_SILU_GATE (gated MLP, op FG_OP_F16_NK only): W is the [N, K] weight made by fg_prepack_gate_up
 * from a gate and an up projection of N/2 rows each; C and residual are [M, N/2], bias (optional) is
 * [N] in the order of W's rows:
 *     C[m, j] = silu(x . Wgate[j] + bias_gate[j]) * (x . Wup[j] + bias_up[j]) + residual[m, j]
 * One pass over both projections, no intermediate tensors. */
int fg_gemm_fused(int op, const void* x, const void* W, const void* scales, void* C, int M, int N, int K,
                  const fg_epilogue_t* ep, void* ws, size_t ws_bytes, fg_stream_t stream);

/* ---- one-time weight repacking ------------------------------------------------------------
 * fg_prepack_kn_to_nk: B[K, N] -> W[N, K] (fp16, N and K multiples of 64).  Callers of the KxN
 * operators (edgemm_m8n128k64x4, flat_gemm_*) whose weight is fixed can repack it once and use the
 * NxK entry points from then on.  The reference only sketches packed weight containers
 * (backend/cuda/hk/utility.cuh:13-46) and has no repacking routine.
 * fg_prepack_gate_up: Wg[Nh, K], Wu[Nh, K] -> Wgu[2 Nh, K] whose every 128 rows hold 64 gate rows
 * followed by the matching 64 up rows (Nh a multiple of 64): the weight FG_ACT_SILU_GATE takes. */
int fg_prepack_kn_to_nk(const void* B, void* W, int N, int K, fg_stream_t stream);
int fg_prepack_gate_up(const void* Wg, const void* Wu, void* Wgu, int Nh, int K, fg_stream_t stream);

/* ---- int8 weight producer ----------------------------------------------------------------
 * Per-output-channel symmetric quantiser for fg_gemm_w8a16_nk: W[N,K] fp16 -> W8[N,K] int8
 * and scales[N] fp16 with scale[n] = fp16(max_k|W[n,k]| / 127) (1 for an all-zero row) and
 * W8 = clamp(rint(W / scale), -127, 127).  K % 8 == 0.  The reference has no quantiser (its
 * int8 GEMV is fed hand-made data, script/fastgemv-int8.py:5-11). */
int fg_quantize_rows_w8(const void* W, int8_t* W8, void* scales, int N, int K, fg_stream_t stream);

/* ---- end-to-end convenience (HOST pointers) ---------------------------------
 * x_host and C_host are host buffers (pinned for full speed); W_dev, scales_dev,
 * x_stage_dev (M*K fp16) and C_stage_dev (M*N fp16) are device buffers the caller
 * owns.  Copies x in, runs the op, copies C out and synchronises `stream`.
 * The weight stays resident on the device, as at the reference's call sites. */
int fg_linear_host(int op, const void* x_host, const void* W_dev, const void* scales_dev,
                   void* C_host, void* x_stage_dev, void* C_stage_dev, int M, int N, int K,
                   void* ws, size_t ws_bytes, fg_stream_t stream);

/* ---- built-in tracer -----------------------------------------------------------
 * While enabled (process-wide), every launch records sixteen 64-bit words per CTA in a
 * spare corner of the workspace.  %globaltimer stamps (ns): [0] CTA start, [1] first copy
 * issued, [2] last copy issued, [3] first stage landed, [4] last tensor-core op of the last
 * segment issued, [7] last accumulator complete / read back, [5] finishers done;
 * [6] number of segments.  Accumulated waiting time (ns, tcgen05 kernel): [9] math waiting for a stage to land, [10] math issuing, [11] epilogue waiting for an
 * accumulator.  fg_trace_read synchronises `stream`, copies 16*ctas words to
 * `out` and clears them.  Costs one predicated branch per event when disabled. */
int fg_trace_enable(int on);
int fg_trace_read(void* ws, unsigned long long* out, int ctas, fg_stream_t stream);

/* ---- diagnostics -------------------------------------------------------------- */
const char* fg_status_str(int status);
/* cudaError_t / CUresult of the last failing call on this host thread (0 if none). */
int fg_last_cuda_error(void);
/* Number of kernel launches this library has issued from this process. */
unsigned long long fg_launch_count(void);
/* "fastgate_b200 <version> sm_100a" */
const char* fg_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FASTGATE_B200_H_ */
