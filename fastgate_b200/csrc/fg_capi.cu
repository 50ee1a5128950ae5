// C ABI of fastgate_b200: argument checks, tensor-map encoding, kernel launch.
// Host code only depends on the CUDA runtime; the driver's tensor-map encoder is
// looked up at run time, so the library loads (and fg_plan works) on a box without a GPU.
#include <cuda.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdint>
#include <cstring>
#include <mutex>
#include <new>
#include <vector>

#include "../../include/fastgate_b200.h"
#include "fg_kernels.cuh"
#include "fg_umma.cuh"
#include "fg_gemv.cuh"
#include "fg_umma_group.cuh"
#include "fg_umma_chain.cuh"
#include "fg_umma_q.cuh"
#include "fg_quant.cuh"
#include "fg_layout.h"

static_assert(FG_TILE_N == fg::kTileN, "layout mismatch");
static_assert(FG_RED_STRIDE == fg::kRedStride, "layout mismatch");
static_assert(FG_CHUNK_W_BYTES == fg::kChunkWBytes, "layout mismatch");
static_assert(FG_MAX_CONSUMER_WARPS == fg::kMaxConsumerWarps, "layout mismatch");
static_assert(int(FG_ERR_TIMEOUT) == int(fg::kStatusTimeout), "status mismatch");
static_assert(int(FG_ERR_PLAN) == int(fg::kStatusBadLaunch), "status mismatch");
static_assert(int(FG_ACT_GELU_ERF) == int(fg::kActGeluErf) && int(FG_ACT_GELU_TANH) == int(fg::kActGeluTanh) &&
                  int(FG_ACT_SILU) == int(fg::kActSilu) && int(FG_ACT_SILU_GATE) == int(fg::kActSiluGate),
              "activation code mismatch");
static_assert(int(FG_OP_F16_KN) == int(fg::kOpF16KN) && int(FG_OP_F16_NK) == int(fg::kOpF16NK) &&
                  int(FG_OP_W8A16_NK) == int(fg::kOpW8A16NK) && int(FG_OP_W4A16_NK) == int(fg::kOpW4A16NK),
              "op code mismatch");

extern "C" int fg_plan_validate(const fg_plan_t* p, int N, int K, int smem_optin_bytes);

namespace {

thread_local int g_last_cuda = 0;
std::atomic<int> g_trace{0};
// While tracing, consecutive launches of the single-problem kernels write to eight rotating blocks of
// kTraceBlockCtas CTAs each, so that a launch that overlaps its predecessor (programmatic dependent
// launch) does not overwrite its stamps; fg_trace_enable restarts the rotation at block 0.
std::atomic<unsigned int> g_trace_seq{0};
constexpr int kTraceBlocks = 8;
constexpr int kTraceBlockCtas = 256;
// The tracer borrows the partial-tile slots of CTAs 200.. (unused while grid <= 200).
constexpr int kTraceFirstCta = 200;
std::atomic<unsigned long long> g_launches{0};

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                   const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                   const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encoder() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

struct DeviceInfo {
  int sm_count = 0;
  int smem_optin = 0;
  int cc_major = 0;
  int smem_set[4][2] = {{0, 0}, {0, 0}, {0, 0}, {0, 0}};  // largest dynamic smem opted in per kernel
  int smem_set_umma[4][3] = {};
  int smem_set_gemv[FG_GEMV_MAX_M + 1] = {};  // fp16 with one and two rows, int8
  int smem_set_group[2] = {0, 0};
  int smem_set_chain[2] = {0, 0};
};

constexpr int kMaxDevices = 64;
DeviceInfo g_dev[kMaxDevices];
std::mutex g_dev_mu;

int device_info(DeviceInfo** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_NO_DEVICE;
  }
  if (dev < 0 || dev >= kMaxDevices) return FG_ERR_NO_DEVICE;
  DeviceInfo& d = g_dev[dev];
  std::lock_guard<std::mutex> lk(g_dev_mu);
  if (d.sm_count == 0) {
    int sm = 0, optin = 0, major = 0;
    if ((e = cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess) {
      g_last_cuda = static_cast<int>(e);
      return FG_ERR_CUDA;
    }
    d.smem_optin = optin;
    d.cc_major = major;
    d.sm_count = sm;
  }
  if (d.cc_major != 10) return FG_ERR_NO_DEVICE;  // the kernels are sm_100a only
  *out = &d;
  return FG_OK;
}

// 2-D row-major tensor: `inner` contiguous elements per row, `rows` rows, 128B swizzle.
int encode_2d(CUtensorMap* tm, CUtensorMapDataType dt, int elem_bytes, const void* base,
              uint64_t inner, uint64_t rows, uint32_t box_inner, uint32_t box_rows,
              uint64_t row_stride_elems = 0) {
  EncodeTiledFn enc = get_encoder();
  if (enc == nullptr) return FG_ERR_CUDA;
  const cuuint64_t gdim[2] = {inner, rows};
  const cuuint64_t gstride[1] = {(row_stride_elems ? row_stride_elems : inner) * static_cast<uint64_t>(elem_bytes)};
  const cuuint32_t box[2] = {box_inner, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult r = enc(tm, dt, 2, const_cast<void*>(base), gdim, gstride, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                         CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    g_last_cuda = static_cast<int>(r);
    return FG_ERR_CUDA;
  }
  return FG_OK;
}

using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const fg::KParams);

// Stages beyond the first ring-full whose weights a CTA asks into L2 while it waits for the
// previous kernel of the stream (programmatic dependent launch): about FG_L2_PREFETCH_BYTES per
// CTA.  Measured on the 8192 x 8192 sweep: 64-128 KB per CTA takes 2-3 % off a call, 256 KB and
// more cost time (the requests compete with the last loads of the kernel that is draining).
int l2_prefetch_stages(int chunks) {
  const int stage_w = chunks * 16384;  // every op moves 16 KB of weights per chunk
  const int n = FG_L2_PREFETCH_BYTES / stage_w;
  return n > 0 ? n : 1;
}

KernelFn pick_kernel(int op, int m_tile) {
  switch (op * 2 + (m_tile == 16)) {
    case 0: return fg::fg_streamk_kernel<fg::kOpF16KN, 8>;
    case 1: return fg::fg_streamk_kernel<fg::kOpF16KN, 16>;
    case 2: return fg::fg_streamk_kernel<fg::kOpF16NK, 8>;
    case 3: return fg::fg_streamk_kernel<fg::kOpF16NK, 16>;
    case 4: return fg::fg_streamk_kernel<fg::kOpW8A16NK, 8>;
    case 5: return fg::fg_streamk_kernel<fg::kOpW8A16NK, 16>;
    case 6: return fg::fg_streamk_kernel<fg::kOpW4A16NK, 8>;
    default: return fg::fg_streamk_kernel<fg::kOpW4A16NK, 16>;
  }
}

KernelFn pick_umma_kernel(int op, int m_tile) {
  if (op == FG_OP_W8A16_NK) return fg::fg_umma_q_kernel<fg::kOpW8A16NK>;
  if (op == FG_OP_W4A16_NK) return fg::fg_umma_q_kernel<fg::kOpW4A16NK>;
  if (op == FG_OP_F16_KN)
    return m_tile == 64 ? fg::fg_umma_kernel<fg::kOpF16KN, 64>
                        : m_tile == 32 ? fg::fg_umma_kernel<fg::kOpF16KN, 32> : fg::fg_umma_kernel<fg::kOpF16KN, 16>;
  return m_tile == 64 ? fg::fg_umma_kernel<fg::kOpF16NK, 64>
                      : m_tile == 32 ? fg::fg_umma_kernel<fg::kOpF16NK, 32> : fg::fg_umma_kernel<fg::kOpF16NK, 16>;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

int check_common(const void* x, const void* W, const void* C, int M, int N, int K, void* ws,
                 size_t ws_bytes) {
  if (x == nullptr || W == nullptr || C == nullptr) return FG_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0 || (N % 128) != 0 || (K % 128) != 0) return FG_ERR_SHAPE;
  if (!aligned16(x) || !aligned16(W) || !aligned16(C)) return FG_ERR_ALIGN;
  if (ws == nullptr || (reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return FG_ERR_WORKSPACE;
  if (ws_bytes < FG_WS_TICKETS_OFFSET + 4 * static_cast<size_t>(N / 128)) return FG_ERR_WORKSPACE;
  return FG_OK;
}

// The kernel a plan names, with its shared-memory opt-in done for this device.  Both the
// workspace entry points and the workspace-free one go through here and through launch_one,
// so a plan can never be launched with another kernel's thread count or memory layout.
int prepare_kernel(const fg_plan_t& pl, DeviceInfo* dev, KernelFn* out) {
  const bool umma = (pl.math == 2);
  const int tall = pl.m_tile == 64 ? 2 : pl.m_tile == 32 ? 1 : 0;
  KernelFn kern = umma ? pick_umma_kernel(pl.op, pl.m_tile) : pick_kernel(pl.op, pl.m_tile);
  std::lock_guard<std::mutex> lk(g_dev_mu);  // the opt-in bookkeeping is shared by all host threads
  int& set = umma ? dev->smem_set_umma[pl.op][tall] : dev->smem_set[pl.op][pl.m_tile == 16];
  if (pl.smem_bytes > set) {
    const cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kern),
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, pl.smem_bytes);
    if (e != cudaSuccess) {
      g_last_cuda = static_cast<int>(e);
      return FG_ERR_CUDA;
    }
    set = pl.smem_bytes;
  }
  *out = kern;
  return FG_OK;
}

// One warp, launched so that it overlaps its neighbours in the stream (see fg_push_wait_kernel).
template <typename... Params, typename... Args>
cudaError_t launch_wait(void (*kern)(Params...), cudaStream_t stream, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(1);
  cfg.blockDim = dim3(32);
  cfg.dynamicSmemBytes = 0;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<Params>(args)...);
}

int launch_one(const fg_plan_t& pl, KernelFn kern, const CUtensorMap& tmW, const CUtensorMap& tmX,
               const fg::KParams& p, cudaStream_t stream) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pl.grid);
  // tcgen05 kernel: fixed warp roles; mma.sync kernel: consumers + one copy-issuing warp +
  // m_tile/4 warps that finish split tiles
  const bool quantized = (pl.op == FG_OP_W8A16_NK || pl.op == FG_OP_W4A16_NK);
  cfg.blockDim = dim3(pl.math == 2 ? (quantized ? fg::kUmmaQThreads : fg::kUmmaThreads)
                                   : (pl.consumer_warps + 1 + 2 * (pl.m_tile / 4)) * 32);
  cfg.dynamicSmemBytes = pl.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pl.pdl && p.pdl) ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tmW, tmX, p);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return FG_OK;
}

// ---- row-split GEMV kernel (plan.math == 4) -------------------------------------------------
using GemvFn = void (*)(const fg::GemvParams);

GemvFn pick_gemv_kernel(int M, bool int8) {
  if (int8) return fg::fg_gemv_kernel<1, 1>;
  return M == 1 ? fg::fg_gemv_kernel<1> : fg::fg_gemv_kernel<2>;
}

int run_gemv(const fg_plan_t& pl, DeviceInfo* dev, const void* x, const void* W, const void* scales, void* C, int M,
             int N, int K, void* ws, cudaStream_t stream, const fg_epilogue_t* ep) {
  if (M != pl.m_tile || M < 1 || M > FG_GEMV_MAX_M) return FG_ERR_PLAN;
  const bool int8 = (pl.op == FG_OP_W8A16_NK);
  if (pl.op != FG_OP_F16_NK && !(int8 && M == 1)) return FG_ERR_PLAN;
  GemvFn kern = pick_gemv_kernel(M, int8);
  {
    std::lock_guard<std::mutex> lk(g_dev_mu);
    int& set = dev->smem_set_gemv[int8 ? 2 : M - 1];
    if (pl.smem_bytes > set) {
      const cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kern),
                                                 cudaFuncAttributeMaxDynamicSharedMemorySize, pl.smem_bytes);
      if (e != cudaSuccess) {
        g_last_cuda = static_cast<int>(e);
        return FG_ERR_CUDA;
      }
      set = pl.smem_bytes;
    }
  }
  uint8_t* wsb = static_cast<uint8_t*>(ws);
  fg::GemvParams p = {};
  p.W = W;
  p.x = static_cast<const __half*>(x);
  p.C = static_cast<__half*>(C);
  p.scales = int8 ? static_cast<const __half*>(scales) : nullptr;
  p.bias = ep ? static_cast<const __half*>(ep->bias) : nullptr;
  p.residual = ep ? static_cast<const __half*>(ep->residual) : nullptr;
  p.act = ep ? ep->act : 0;
  p.split1 = ep ? ep->split1 : 0;
  p.split2 = ep ? ep->split2 : 0;
  p.C2 = ep ? static_cast<__half*>(ep->C2) : nullptr;
  p.C3 = ep ? static_cast<__half*>(ep->C3) : nullptr;
  p.M = M;
  p.N = N;
  p.K = K;
  p.rows_per_stage = pl.rows_per_stage;
  p.stage_bytes = pl.rows_per_stage * K * (int8 ? 1 : 2);
  p.stages = pl.stages;
  p.static_rows = pl.static_rows;
  p.l2_prefetch_bytes = pl.pdl ? FG_GEMV_L2_PREFETCH_BYTES : 0;
  p.next = reinterpret_cast<unsigned int*>(wsb + FG_WS_GEMV_NEXT_OFFSET);
  p.exited = reinterpret_cast<unsigned int*>(wsb + FG_WS_GEMV_EXITED_OFFSET);
  p.status = reinterpret_cast<int*>(wsb);
  p.trace = nullptr;
  if (g_trace.load(std::memory_order_relaxed) && pl.grid <= kTraceFirstCta)
    p.trace = reinterpret_cast<unsigned long long*>(wsb + FG_WS_HEADER_BYTES +
                                                    static_cast<size_t>(kTraceFirstCta) * 2 * FG_WS_PARTIAL_TILE_BYTES) +
              static_cast<size_t>(g_trace_seq.fetch_add(1, std::memory_order_relaxed) % kTraceBlocks) * kTraceBlockCtas *
                  fg::kTraceSlots;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pl.grid);
  cfg.blockDim = dim3((pl.consumer_warps + 1) * 32);
  cfg.dynamicSmemBytes = pl.smem_bytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = pl.pdl ? 1 : 0;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, p);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return FG_OK;
}

// int4 op: scales per row and the zero point
struct QuantArgs {
  int groups;
  int zero_point;
};

int run_planned(const fg_plan_t& pl, DeviceInfo* dev, const void* x, const void* W,
                const void* scales, void* C, int M, int N, int K, void* ws, cudaStream_t stream,
                const fg_peers_t* peers = nullptr, const fg_epilogue_t* ep = nullptr,
                const QuantArgs* qa = nullptr) {
  const int op = pl.op;
  if (pl.math == 4) {
    if (peers != nullptr || qa != nullptr) return FG_ERR_PLAN;  // the row-split kernel neither pushes nor takes int4
    return run_gemv(pl, dev, x, W, scales, C, M, N, K, ws, stream, ep);
  }
  const int chunks = pl.k_per_stage / fg_chunk_k(op);
  KernelFn kern = nullptr;
  {
    const int pst = prepare_kernel(pl, dev, &kern);
    if (pst != FG_OK) return pst;
  }

  CUtensorMap tmW;
  int st;
  if (op == FG_OP_F16_KN)
    st = encode_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, W, N, K, 64, 64);
  else if (op == FG_OP_F16_NK)
    st = encode_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, W, K, N, 64, 128);
  else if (op == FG_OP_W8A16_NK)
    st = encode_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, W, K, N, 128, 128);
  else
    st = encode_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, W, K / 2, N, 128, 128);  // packed nibbles
  if (st != FG_OK) return st;

  uint8_t* wsb = static_cast<uint8_t*>(ws);
  fg::KParams p = {};
  p.scales = static_cast<const __half*>(scales);
  p.scale_groups = qa ? qa->groups : 1;
  {
    const unsigned int h = __half_as_ushort(__float2half_rn(1024.f + static_cast<float>(qa ? qa->zero_point : 0)));
    p.w4_magic = h | (h << 16);
  }
  p.partials = reinterpret_cast<float*>(wsb + FG_WS_HEADER_BYTES);
  p.tickets = reinterpret_cast<unsigned int*>(wsb + FG_WS_TICKETS_OFFSET);
  p.status = reinterpret_cast<int*>(wsb);
  p.trace = nullptr;
  if (g_trace.load(std::memory_order_relaxed) && pl.grid <= kTraceFirstCta)
    p.trace = reinterpret_cast<unsigned long long*>(wsb + FG_WS_HEADER_BYTES +
                                                    static_cast<size_t>(kTraceFirstCta) * 2 * FG_WS_PARTIAL_TILE_BYTES) +
              static_cast<size_t>(g_trace_seq.fetch_add(1, std::memory_order_relaxed) % kTraceBlocks) * kTraceBlockCtas *
                  fg::kTraceSlots;
  p.N = N;
  p.K = K;
  p.tiles = pl.tiles;
  p.k_blocks = pl.k_blocks;
  p.chunks_per_stage = chunks;
  p.stages = pl.stages;
  p.consumer_warps = pl.consumer_warps;
  p.pdl = pl.pdl ? 1 : 0;
  p.l2_prefetch = pl.pdl ? l2_prefetch_stages(chunks) : 0;
  p.bias = ep ? static_cast<const __half*>(ep->bias) : nullptr;
  p.residual = nullptr;
  p.act = ep ? ep->act : 0;
  p.split1 = ep ? ep->split1 : 0;
  p.split2 = ep ? ep->split2 : 0;
  p.C2 = ep ? static_cast<__half*>(ep->C2) : nullptr;
  p.C3 = ep ? static_cast<__half*>(ep->C3) : nullptr;
  if (peers != nullptr && (p.split1 != 0 || p.act == FG_ACT_SILU_GATE)) return FG_ERR_PLAN;  // a pushed output is one plain tensor
  p.world = 0;
  p.rank = 0;
  p.col0 = 0;
  p.ldc = N;
  p.wait_flags = nullptr;
  p.wait_world = 0;
  p.wait_target = 0;
  p.mc_C = nullptr;
  p.mc_flag = nullptr;
  p.target_dev = nullptr;
  p.wait_target_dev = nullptr;
  if (peers != nullptr) {
    p.target_dev = peers->target_dev;
    p.wait_target_dev = peers->wait_target_dev;
    if (peers->mc_C != nullptr && peers->mc_flag != nullptr) {
      p.mc_C = static_cast<__half*>(peers->mc_C);
      p.mc_flag = peers->mc_flag;
    }
    p.wait_flags = peers->wait_flags;
    p.wait_world = peers->world;
    p.wait_target = peers->wait_target;
    p.world = peers->world;
    p.rank = peers->rank;
    p.col0 = peers->rank * N;
    p.ldc = peers->n_total;
    for (int q = 0; q < peers->world; ++q) {
      p.peer_C[q] = static_cast<__half*>(peers->C[q]);
      p.peer_flag[q] = peers->flag[q];
    }
  }

  const int rows = fg_pass_rows(op, pl.math);  // token rows per launch
  for (int m0 = 0; m0 < M; m0 += rows) {
    const int mp = (M - m0) < rows ? (M - m0) : rows;
    if (mp > pl.m_tile) return FG_ERR_PLAN;
    const __half* xp = static_cast<const __half*>(x) + static_cast<size_t>(m0) * K;
    CUtensorMap tmX;
    st = encode_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xp, K, mp, 64, pl.m_tile);
    if (st != FG_OK) return st;
    const int width = (p.act == FG_ACT_SILU_GATE) ? N / 2 : N;  // row length of the output (and of the residual)
    p.C = static_cast<__half*>(C) + static_cast<size_t>(m0) * (p.split1 ? p.split1 : width);
    if (p.split1) {
      p.C2 = static_cast<__half*>(ep->C2) + static_cast<size_t>(m0) * (p.split2 - p.split1);
      p.C3 = static_cast<__half*>(ep->C3) + static_cast<size_t>(m0) * (N - p.split2);
    }
    p.M = mp;
    if (ep != nullptr && ep->residual != nullptr)
      p.residual = static_cast<const __half*>(ep->residual) + static_cast<size_t>(m0) * width;
    if (peers != nullptr) {
      for (int q = 0; q < peers->world; ++q)
        p.peer_C[q] = static_cast<__half*>(peers->C[q]) + static_cast<size_t>(m0) * peers->n_total;
      if (p.mc_C != nullptr) p.mc_C = static_cast<__half*>(peers->mc_C) + static_cast<size_t>(m0) * peers->n_total;
    }
    if ((st = launch_one(pl, kern, tmW, tmX, p, stream)) != FG_OK) return st;
  }
  return FG_OK;
}

int run_op(int op, const void* x, const void* W, const void* scales, void* C, int M, int N, int K,
           void* ws, size_t ws_bytes, fg_stream_t stream, const QuantArgs* qa = nullptr) {
  int st = check_common(x, W, C, M, N, K, ws, ws_bytes);
  if (st != FG_OK) return st;
  if (scales != nullptr && (reinterpret_cast<uintptr_t>(scales) & 3u) != 0) return FG_ERR_ALIGN;
  DeviceInfo* dev = nullptr;
  if ((st = device_info(&dev)) != FG_OK) return st;
  fg_plan_t pl;
  if ((st = fg_plan(op, M, N, K, dev->sm_count, dev->smem_optin, &pl)) != FG_OK) return st;
  return run_planned(pl, dev, x, W, scales, C, M, N, K, ws, reinterpret_cast<cudaStream_t>(stream), nullptr, nullptr,
                     qa);
}

// ---- scratch for fg_gemm_f16_nk_noalloc -------------------------------------------------
// Callers that must not (or cannot) call cudaMalloc -- code running inside someone else's
// memory budget, a plugin that is handed buffers but no allocator, a latency-critical loop
// that may not touch the allocator -- get the split-K scratch from this file-scope array
// instead of a workspace.  Every GPU that loads the library carries it until the process
// exits.  Layout: [0,256) status word | 4 B arrival counter per output tile | two fp32
// partial tiles of 16 x 128 per persistent CTA.
constexpr int kNoAllocMaxN = 65536;   // at most 512 output tiles
constexpr int kNoAllocMaxGrid = 160;  // persistent CTAs (a B200 has 148 SMs)
constexpr size_t kNoAllocTicketsOffset = 256;
constexpr size_t kNoAllocPartialsOffset = kNoAllocTicketsOffset + 4 * (kNoAllocMaxN / 128);
constexpr size_t kNoAllocBytes =
    kNoAllocPartialsOffset + static_cast<size_t>(kNoAllocMaxGrid) * 2 * FG_WS_PARTIAL_TILE16_BYTES;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocBytes];

// In host code `g_noalloc_scratch` is only a handle for the symbol, not a device address;
// the address is looked up once per device, with that device current.
unsigned char* g_noalloc_ptr[kMaxDevices] = {};
std::mutex g_noalloc_mu;

int noalloc_scratch(int dev_index, unsigned char** out) {
  std::lock_guard<std::mutex> lk(g_noalloc_mu);
  if (g_noalloc_ptr[dev_index] == nullptr) {
    void* ptr = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      g_last_cuda = static_cast<int>(e);
      return FG_ERR_CUDA;
    }
    g_noalloc_ptr[dev_index] = static_cast<unsigned char*>(ptr);
  }
  *out = g_noalloc_ptr[dev_index];
  return FG_OK;
}

}  // namespace

extern "C" {

size_t fg_workspace_bytes(int N) {
  const size_t tiles = N > 0 ? static_cast<size_t>((N + 127) / 128) : 0;
  return FG_WS_TICKETS_OFFSET + ((4 * tiles + 255) / 256) * 256;
}

int fg_workspace_init(void* ws, size_t ws_bytes, fg_stream_t stream) {
  if (ws == nullptr || (reinterpret_cast<uintptr_t>(ws) & 255u) != 0 || ws_bytes < FG_WS_TICKETS_OFFSET)
    return FG_ERR_WORKSPACE;
  const cudaError_t e = cudaMemsetAsync(ws, 0, ws_bytes, reinterpret_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  return FG_OK;
}

int fg_workspace_status(void* ws, int* status_out, fg_stream_t stream) {
  if (ws == nullptr || status_out == nullptr) return FG_ERR_NULL;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int v = 0;
  cudaError_t e = cudaMemcpyAsync(&v, ws, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e == cudaSuccess && v != 0) e = cudaMemsetAsync(ws, 0, sizeof(int), s);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  *status_out = v;
  return FG_OK;
}

int fg_gemm_f16_kn(const void* A, const void* B, void* C, int M, int N, int K, void* ws,
                   size_t ws_bytes, fg_stream_t stream) {
  return run_op(FG_OP_F16_KN, A, B, nullptr, C, M, N, K, ws, ws_bytes, stream);
}

int fg_gemm_f16_nk(const void* x, const void* W, void* C, int M, int N, int K, void* ws,
                   size_t ws_bytes, fg_stream_t stream) {
  return run_op(FG_OP_F16_NK, x, W, nullptr, C, M, N, K, ws, ws_bytes, stream);
}

int fg_gemm_w8a16_nk(const void* x, const int8_t* W8, const void* scales, void* C, int M, int N,
                     int K, void* ws, size_t ws_bytes, fg_stream_t stream) {
  return run_op(FG_OP_W8A16_NK, x, W8, scales, C, M, N, K, ws, ws_bytes, stream);
}

int fg_gemm_w4a16_nk(const void* x, const uint8_t* W4, const void* scales, int groups, int zero_point, void* C,
                     int M, int N, int K, void* ws, size_t ws_bytes, fg_stream_t stream) {
  if (zero_point < 0 || zero_point > 15) return FG_ERR_PLAN;
  if (K > 0 && groups != 1 && groups != K / 128) return FG_ERR_SHAPE;
  if (scales != nullptr && groups > 1 && (reinterpret_cast<uintptr_t>(scales) & 1u) != 0) return FG_ERR_ALIGN;
  QuantArgs qa{scales != nullptr ? groups : 1, zero_point};
  if (groups > 1 && scales != nullptr) {
    // group-wise scales are read two bytes at a time: only the common checks apply
    int st = check_common(x, W4, C, M, N, K, ws, ws_bytes);
    if (st != FG_OK) return st;
    DeviceInfo* dev = nullptr;
    if ((st = device_info(&dev)) != FG_OK) return st;
    fg_plan_t pl;
    if ((st = fg_plan(FG_OP_W4A16_NK, M, N, K, dev->sm_count, dev->smem_optin, &pl)) != FG_OK) return st;
    return run_planned(pl, dev, x, W4, scales, C, M, N, K, ws, reinterpret_cast<cudaStream_t>(stream), nullptr,
                       nullptr, &qa);
  }
  return run_op(FG_OP_W4A16_NK, x, W4, scales, C, M, N, K, ws, ws_bytes, stream, &qa);
}

int fg_gemm_planned(const fg_plan_t* plan, const void* x, const void* W, const void* scales, void* C,
                    int M, int N, int K, void* ws, size_t ws_bytes, fg_stream_t stream) {
  if (plan == nullptr) return FG_ERR_NULL;
  int st = check_common(x, W, C, M, N, K, ws, ws_bytes);
  if (st != FG_OK) return st;
  DeviceInfo* dev = nullptr;
  if ((st = device_info(&dev)) != FG_OK) return st;
  if ((st = fg_plan_validate(plan, N, K, dev->smem_optin)) != FG_OK) return st;
  if (plan->op == FG_OP_W4A16_NK) return FG_ERR_PLAN;  // needs groups and zero point: fg_gemm_w4a16_nk
  {
    const int rows = fg_pass_rows(plan->op, plan->math);
    if (plan->passes != (M + rows - 1) / rows) return FG_ERR_PLAN;
  }
  return run_planned(*plan, dev, x, W, plan->op == FG_OP_W8A16_NK ? scales : nullptr, C, M, N, K, ws,
                     reinterpret_cast<cudaStream_t>(stream));
}

int fg_gemm_f16_nk_push(const void* x, const void* W_shard, int M, int N_local, int K,
                        const fg_peers_t* peers, void* ws, size_t ws_bytes, fg_stream_t stream) {
  if (peers == nullptr) return FG_ERR_NULL;
  if (peers->world < 1 || peers->world > fg::kMaxPeers || peers->rank < 0 || peers->rank >= peers->world)
    return FG_ERR_PLAN;
  if (peers->n_total != static_cast<long long>(peers->world) * N_local) return FG_ERR_SHAPE;
  for (int q = 0; q < peers->world; ++q) {
    if (peers->C[q] == nullptr || peers->flag[q] == nullptr) return FG_ERR_NULL;
    if (!aligned16(peers->C[q]) || (reinterpret_cast<uintptr_t>(peers->flag[q]) & 7u) != 0) return FG_ERR_ALIGN;
  }
  if ((reinterpret_cast<uintptr_t>(peers->wait_flags) & 7u) != 0) return FG_ERR_ALIGN;
  if ((reinterpret_cast<uintptr_t>(peers->target_dev) & 7u) != 0 || (reinterpret_cast<uintptr_t>(peers->wait_target_dev) & 7u) != 0)
    return FG_ERR_ALIGN;
  if ((peers->mc_C == nullptr) != (peers->mc_flag == nullptr)) return FG_ERR_NULL;  // both multicast mappings or none
  if (!aligned16(peers->mc_C) || (reinterpret_cast<uintptr_t>(peers->mc_flag) & 7u) != 0) return FG_ERR_ALIGN;
  int st = check_common(x, W_shard, peers->C[peers->rank], M, N_local, K, ws, ws_bytes);
  if (st != FG_OK) return st;
  DeviceInfo* dev = nullptr;
  if ((st = device_info(&dev)) != FG_OK) return st;
  fg_plan_t pl;
  if ((st = fg_plan_tiled(FG_OP_F16_NK, M, N_local, K, dev->sm_count, dev->smem_optin, &pl)) != FG_OK) return st;
  return run_planned(pl, dev, x, W_shard, nullptr, peers->C[peers->rank], M, N_local, K, ws,
                     reinterpret_cast<cudaStream_t>(stream), peers);
}

int fg_push_wait(const unsigned long long* my_flags, int world, unsigned long long target, void* ws,
                 fg_stream_t stream) {
  if (my_flags == nullptr || ws == nullptr) return FG_ERR_NULL;
  if (world < 1 || world > fg::kMaxPeers) return FG_ERR_PLAN;
  const cudaError_t e = launch_wait(fg::fg_push_wait_kernel, reinterpret_cast<cudaStream_t>(stream), my_flags, world, target,
                                    static_cast<int*>(ws));
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return FG_OK;
}

int fg_push_wait_dev(const unsigned long long* my_flags, int world, const unsigned long long* target_dev, void* ws,
                     fg_stream_t stream) {
  if (my_flags == nullptr || target_dev == nullptr || ws == nullptr) return FG_ERR_NULL;
  if (world < 1 || world > fg::kMaxPeers) return FG_ERR_PLAN;
  if ((reinterpret_cast<uintptr_t>(target_dev) & 7u) != 0) return FG_ERR_ALIGN;
  const cudaError_t e = launch_wait(fg::fg_push_wait_dev_kernel, reinterpret_cast<cudaStream_t>(stream), my_flags, world,
                                    target_dev, static_cast<int*>(ws));
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return FG_OK;
}

int fg_push_wait_dev_many(const unsigned long long* const* my_flags, const unsigned long long* const* target_dev, int count,
                          int world, void* ws, fg_stream_t stream) {
  if (my_flags == nullptr || target_dev == nullptr || ws == nullptr) return FG_ERR_NULL;
  if (world < 1 || world > fg::kMaxPeers || count < 1 || count > fg::kMaxWaits) return FG_ERR_PLAN;
  fg::WaitList w = {};
  w.count = count;
  for (int i = 0; i < count; ++i) {
    if (my_flags[i] == nullptr || target_dev[i] == nullptr) return FG_ERR_NULL;
    if ((reinterpret_cast<uintptr_t>(my_flags[i]) & 7u) != 0 || (reinterpret_cast<uintptr_t>(target_dev[i]) & 7u) != 0)
      return FG_ERR_ALIGN;
    w.flags[i] = my_flags[i];
    w.target_dev[i] = target_dev[i];
  }
  const cudaError_t e = launch_wait(fg::fg_push_wait_many_kernel, reinterpret_cast<cudaStream_t>(stream), w, world,
                                    static_cast<int*>(ws));
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return FG_OK;
}

// ---- grouped launch ------------------------------------------------------------------
struct fg_group {
  int op;
  int count;
  int device;
  const fg::GroupEntry* table_dev;
  uint32_t total_units;
  uint32_t total_tiles;
  int chunks, stages, grid, smem_bytes;
  int world, rank;
  unsigned long long* flag[8];
  unsigned long long* mc_flag;
  unsigned long long* target_dev;
};

size_t fg_group_table_bytes(int count) {
  return count > 0 ? static_cast<size_t>(count) * sizeof(fg::GroupEntry) : 0;
}

int fg_group_create(int op, const fg_problem_t* problems, int count, const fg_peers_t* peers, void* table_dev,
                    size_t table_bytes, fg_group_t** out) {
  if (problems == nullptr || out == nullptr || table_dev == nullptr) return FG_ERR_NULL;
  *out = nullptr;
  if (op != FG_OP_F16_KN && op != FG_OP_F16_NK) return FG_ERR_PLAN;
  if (count < 1 || count > 65536) return FG_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(table_dev) & 127u) != 0 || table_bytes < fg_group_table_bytes(count))
    return FG_ERR_WORKSPACE;
  int world = 0, rank = 0;
  if (peers != nullptr) {
    world = peers->world;
    rank = peers->rank;
    if (world < 1 || world > fg::kMaxPeers || rank < 0 || rank >= world) return FG_ERR_PLAN;
    for (int q = 0; q < world; ++q) {
      if (peers->flag[q] == nullptr) return FG_ERR_NULL;
      if ((reinterpret_cast<uintptr_t>(peers->flag[q]) & 7u) != 0) return FG_ERR_ALIGN;
    }
  }
  DeviceInfo* dev = nullptr;
  int st = device_info(&dev);
  if (st != FG_OK) return st;
  int dev_index = 0;
  cudaError_t e = cudaGetDevice(&dev_index);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  for (int i = 0; i < count; ++i) {
    const fg_problem_t& q = problems[i];
    if (q.x == nullptr || q.W == nullptr) return FG_ERR_NULL;
    if (q.M <= 0 || q.M > 16 || q.N <= 0 || q.K <= 0 || (q.N % 128) != 0 || (q.K % 128) != 0) return FG_ERR_SHAPE;
    if (!aligned16(q.x) || !aligned16(q.W)) return FG_ERR_ALIGN;
    if (world == 0) {
      if (q.C == nullptr) return FG_ERR_NULL;
      if (!aligned16(q.C)) return FG_ERR_ALIGN;
    } else {
      if (q.n_total != static_cast<long long>(world) * q.N) return FG_ERR_SHAPE;
      for (int r = 0; r < world; ++r) {
        if (q.peer_C[r] == nullptr) return FG_ERR_NULL;
        if (!aligned16(q.peer_C[r])) return FG_ERR_ALIGN;
      }
    }
  }
  // stage size: as large as still leaves every CTA at least six stages (see fg_plan)
  const int sms = dev->sm_count < FG_MAX_GRID ? dev->sm_count : FG_MAX_GRID;
  int chunks = 4;
  long long units = 0;
  for (;; chunks >>= 1) {
    units = 0;
    for (int i = 0; i < count; ++i)
      units += static_cast<long long>(problems[i].N / 128) * ((problems[i].K + chunks * 64 - 1) / (chunks * 64));
    if (chunks == 1 || units >= 6LL * sms) break;
  }
  const int grid = static_cast<int>(units < sms ? units : sms);
  if (units * grid >= (1LL << 31)) return FG_ERR_SHAPE;
  const int stage_bytes = chunks * fg_chunk_bytes(op, 16);
  int stages = (dev->smem_optin - 1024 - 64) / (stage_bytes + 16);
  if (stages > FG_MAX_STAGES) stages = FG_MAX_STAGES;
  if (stages < 2) return FG_ERR_PLAN;

  std::vector<fg::GroupEntry> host(count);
  uint32_t unit = 0, tile = 0;
  for (int i = 0; i < count; ++i) {
    const fg_problem_t& q = problems[i];
    fg::GroupEntry& en = host[i];
    std::memset(&en, 0, sizeof(en));
    if (op == FG_OP_F16_KN)
      st = encode_2d(&en.tmW, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, q.W, q.N, q.K, 64, 64);
    else
      st = encode_2d(&en.tmW, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, q.W, q.K, q.N, 64, 128);
    if (st != FG_OK) return st;
    if ((st = encode_2d(&en.tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, q.x, q.K, q.M, 64, 16)) != FG_OK) return st;
    en.C = static_cast<__half*>(q.C);
    for (int r = 0; r < world; ++r) en.peer_C[r] = static_cast<__half*>(q.peer_C[r]);
    en.mc_C = static_cast<__half*>(q.mc_C);
    en.ldc = world ? q.n_total : q.N;
    en.col0 = world ? rank * q.N : 0;
    en.M = q.M;
    en.N = q.N;
    en.K = q.K;
    en.KB = static_cast<uint32_t>((q.K + chunks * 64 - 1) / (chunks * 64));
    en.tiles = static_cast<uint32_t>(q.N / 128);
    en.unit_begin = unit;
    en.tile_begin = tile;
    unit += en.tiles * en.KB;
    tile += en.tiles;
  }
  e = cudaMemcpy(table_dev, host.data(), fg_group_table_bytes(count), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  fg_group* grp = new (std::nothrow) fg_group();
  if (grp == nullptr) return FG_ERR_CUDA;
  grp->op = op;
  grp->count = count;
  grp->device = dev_index;
  grp->table_dev = static_cast<const fg::GroupEntry*>(table_dev);
  grp->total_units = unit;
  grp->total_tiles = tile;
  grp->chunks = chunks;
  grp->stages = stages;
  grp->grid = grid;
  grp->smem_bytes = fg_umma_smem_bytes(op, chunks, stages);
  grp->world = world;
  grp->rank = rank;
  for (int q = 0; q < 8; ++q) grp->flag[q] = (q < world) ? peers->flag[q] : nullptr;
  // multicast only if the flag array and every problem's output have a multicast mapping
  grp->mc_flag = (world > 0) ? peers->mc_flag : nullptr;
  grp->target_dev = (world > 0) ? peers->target_dev : nullptr;
  for (int i = 0; i < count && grp->mc_flag != nullptr; ++i)
    if (problems[i].mc_C == nullptr || !aligned16(problems[i].mc_C)) grp->mc_flag = nullptr;
  *out = grp;
  return FG_OK;
}

int fg_group_run(const fg_group_t* grp, void* ws, size_t ws_bytes, fg_stream_t stream) {
  if (grp == nullptr) return FG_ERR_NULL;
  if (ws == nullptr || (reinterpret_cast<uintptr_t>(ws) & 255u) != 0) return FG_ERR_WORKSPACE;
  if (ws_bytes < FG_WS_TICKETS_OFFSET + 4 * static_cast<size_t>(grp->total_tiles)) return FG_ERR_WORKSPACE;
  DeviceInfo* dev = nullptr;
  int st = device_info(&dev);
  if (st != FG_OK) return st;
  int dev_index = -1;
  if (cudaGetDevice(&dev_index) != cudaSuccess || dev_index != grp->device) return FG_ERR_NO_DEVICE;
  using GroupFn = void (*)(const fg::GParams);
  GroupFn kern = grp->op == FG_OP_F16_KN ? fg::fg_umma_group_kernel<fg::kOpF16KN> : fg::fg_umma_group_kernel<fg::kOpF16NK>;
  std::unique_lock<std::mutex> lk(g_dev_mu);
  int& set = dev->smem_set_group[grp->op == FG_OP_F16_NK];
  if (grp->smem_bytes > set) {
    const cudaError_t e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kern),
                                               cudaFuncAttributeMaxDynamicSharedMemorySize, grp->smem_bytes);
    if (e != cudaSuccess) {
      g_last_cuda = static_cast<int>(e);
      return FG_ERR_CUDA;
    }
    set = grp->smem_bytes;
  }
  lk.unlock();
  uint8_t* wsb = static_cast<uint8_t*>(ws);
  fg::GParams g = {};
  g.table = grp->table_dev;
  g.count = grp->count;
  g.total_units = grp->total_units;
  g.partials = reinterpret_cast<float*>(wsb + FG_WS_HEADER_BYTES);
  g.tickets = reinterpret_cast<unsigned int*>(wsb + FG_WS_TICKETS_OFFSET);
  g.status = reinterpret_cast<int*>(wsb);
  g.trace = nullptr;
  if (g_trace.load(std::memory_order_relaxed) && grp->grid <= kTraceFirstCta)
    g.trace = reinterpret_cast<unsigned long long*>(wsb + FG_WS_HEADER_BYTES +
                                                    static_cast<size_t>(kTraceFirstCta) * 2 * FG_WS_PARTIAL_TILE_BYTES);
  g.chunks_per_stage = grp->chunks;
  g.stages = grp->stages;
  g.world = grp->world;
  g.rank = grp->rank;
  for (int q = 0; q < 8; ++q) g.peer_flag[q] = grp->flag[q];
  g.mc_flag = grp->mc_flag;
  g.target_dev = grp->target_dev;
  g.total_tiles = grp->total_tiles;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grp->grid);
  cfg.blockDim = dim3(fg::kUmmaGroupThreads);
  cfg.dynamicSmemBytes = grp->smem_bytes;
  cfg.stream = reinterpret_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, g);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return FG_OK;
}

unsigned long long fg_group_tiles(const fg_group_t* grp) { return grp ? grp->total_tiles : 0; }

void fg_group_destroy(fg_group_t* grp) { delete grp; }

// ---- dependent layer chain -------------------------------------------------------------
struct fg_chain {
  int op;
  int count;
  int device;
  const fg::ChainEntry* table_dev;
  uint32_t total_tiles;
  int chunks, stages, grid, smem_bytes;
  size_t off_tickets, off_done, off_trace, ws_bytes;
};

size_t fg_chain_table_bytes(int count) {
  return count > 0 ? static_cast<size_t>(count) * sizeof(fg::ChainEntry) : 0;
}

int fg_chain_create(int op, const fg_layer_t* layers, int count, void* table_dev, size_t table_bytes,
                    fg_chain_t** out) {
  if (layers == nullptr || out == nullptr || table_dev == nullptr) return FG_ERR_NULL;
  *out = nullptr;
  if (op != FG_OP_F16_KN && op != FG_OP_F16_NK) return FG_ERR_PLAN;
  if (count < 1 || count > 65536) return FG_ERR_SHAPE;
  if ((reinterpret_cast<uintptr_t>(table_dev) & 127u) != 0 || table_bytes < fg_chain_table_bytes(count))
    return FG_ERR_WORKSPACE;
  DeviceInfo* dev = nullptr;
  int st = device_info(&dev);
  if (st != FG_OK) return st;
  int dev_index = 0;
  cudaError_t e = cudaGetDevice(&dev_index);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  for (int i = 0; i < count; ++i) {
    const fg_layer_t& q = layers[i];
    if (q.x == nullptr || q.W == nullptr || q.C == nullptr) return FG_ERR_NULL;
    if (q.M <= 0 || q.M > 16 || q.N <= 0 || q.K <= 0 || (q.N % 128) != 0 || (q.K % 128) != 0) return FG_ERR_SHAPE;
    if (q.ldx < 0 || q.ldc < 0 || q.ldr < 0) return FG_ERR_SHAPE;
    if ((q.ldx != 0 && q.ldx < q.K) || (q.ldc != 0 && q.ldc < q.N) || (q.ldr != 0 && q.ldr < q.N)) return FG_ERR_SHAPE;
    if (!aligned16(q.x) || !aligned16(q.W) || !aligned16(q.C) || (q.ldx % 8) != 0 || (q.ldc % 8) != 0)
      return FG_ERR_ALIGN;
    if (q.residual != nullptr && (reinterpret_cast<uintptr_t>(q.residual) & 1u) != 0) return FG_ERR_ALIGN;
    if (q.bias != nullptr && (reinterpret_cast<uintptr_t>(q.bias) & 1u) != 0) return FG_ERR_ALIGN;
    if (q.act < FG_ACT_NONE || q.act > FG_ACT_SILU) return FG_ERR_PLAN;
    if (q.dep < -1 || q.dep >= i) return FG_ERR_PLAN;
  }
  // stage size: as large as still leaves every CTA about six stages per layer on average.  (Unlike
  // the single-layer kernel, the chain did not gain from 64 KB stages on the DiT stack: 15.0 us per
  // layer against 14.7 us with 32 KB stages, which leave the ring six deep across a layer boundary.)
  const int sms = dev->sm_count < FG_MAX_GRID ? dev->sm_count : FG_MAX_GRID;
  int chunks = 4;
  long long units = 0, max_units = 0;
  for (;; chunks >>= 1) {
    units = 0;
    max_units = 0;
    for (int i = 0; i < count; ++i) {
      const long long u = static_cast<long long>(layers[i].N / 128) * ((layers[i].K + chunks * 64 - 1) / (chunks * 64));
      units += u;
      max_units = u > max_units ? u : max_units;
    }
    if (chunks == 1 || units >= 6LL * sms * count) break;
  }
  const int grid = static_cast<int>(max_units < sms ? max_units : sms);
  if (max_units * grid >= (1LL << 31)) return FG_ERR_SHAPE;
  const int stage_bytes = chunks * fg_chunk_bytes(op, 16);
  int stages = (dev->smem_optin - 1024 - 96) / (stage_bytes + 16);  // 32 bytes more than the plain kernel: two finisher teams
  if (stages > FG_MAX_STAGES) stages = FG_MAX_STAGES;
  if (stages < 2) return FG_ERR_PLAN;

  std::vector<fg::ChainEntry> host(count);
  uint32_t tile = 0;
  for (int i = 0; i < count; ++i) {
    const fg_layer_t& q = layers[i];
    fg::ChainEntry& en = host[i];
    std::memset(&en, 0, sizeof(en));
    if (op == FG_OP_F16_KN)
      st = encode_2d(&en.tmW, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, q.W, q.N, q.K, 64, 64);
    else
      st = encode_2d(&en.tmW, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, q.W, q.K, q.N, 64, 128);
    if (st != FG_OK) return st;
    st = encode_2d(&en.tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, q.x, q.K, q.M, 64, 16, static_cast<uint64_t>(q.ldx));
    if (st != FG_OK) return st;
    en.C = static_cast<__half*>(q.C);
    en.bias = static_cast<const __half*>(q.bias);
    en.residual = static_cast<const __half*>(q.residual);
    en.ldc = q.ldc ? q.ldc : q.N;
    en.ldr = q.ldr ? q.ldr : q.N;
    en.M = q.M;
    en.N = q.N;
    en.K = q.K;
    en.act = q.act;
    en.dep = q.dep;
    en.KB = static_cast<uint32_t>((q.K + chunks * 64 - 1) / (chunks * 64));
    en.tiles = static_cast<uint32_t>(q.N / 128);
    en.tile_begin = tile;
    tile += en.tiles;
  }
  e = cudaMemcpy(table_dev, host.data(), fg_chain_table_bytes(count), cudaMemcpyHostToDevice);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  fg_chain* ch = new (std::nothrow) fg_chain();
  if (ch == nullptr) return FG_ERR_CUDA;
  ch->op = op;
  ch->count = count;
  ch->device = dev_index;
  ch->table_dev = static_cast<const fg::ChainEntry*>(table_dev);
  ch->total_tiles = tile;
  ch->chunks = chunks;
  ch->stages = stages;
  ch->grid = grid;
  ch->smem_bytes = fg_umma_smem_bytes(op, chunks, stages) + 32;
  // header | grid x 4 partial tiles | one ticket per tile | one counter per layer | timestamps
  ch->off_tickets = FG_WS_HEADER_BYTES + static_cast<size_t>(grid) * 4 * FG_WS_PARTIAL_TILE16_BYTES;
  ch->off_done = (ch->off_tickets + 4 * static_cast<size_t>(tile) + 255) & ~static_cast<size_t>(255);
  ch->off_trace = (ch->off_done + 4 * static_cast<size_t>(count) + 255) & ~static_cast<size_t>(255);
  ch->ws_bytes = (ch->off_trace + 64 * static_cast<size_t>(count) * grid + 255) & ~static_cast<size_t>(255);
  *out = ch;
  return FG_OK;
}

size_t fg_chain_workspace_bytes(const fg_chain_t* ch) { return ch ? ch->ws_bytes : 0; }

int fg_chain_run(const fg_chain_t* ch, void* ws, size_t ws_bytes, fg_stream_t stream) {
  if (ch == nullptr) return FG_ERR_NULL;
  if (ws == nullptr || (reinterpret_cast<uintptr_t>(ws) & 255u) != 0 || ws_bytes < ch->ws_bytes) return FG_ERR_WORKSPACE;
  DeviceInfo* dev = nullptr;
  int st = device_info(&dev);
  if (st != FG_OK) return st;
  int dev_index = -1;
  if (cudaGetDevice(&dev_index) != cudaSuccess || dev_index != ch->device) return FG_ERR_NO_DEVICE;
  using ChainFn = void (*)(const fg::CParams);
  ChainFn kern = ch->op == FG_OP_F16_KN ? fg::fg_umma_chain_kernel<fg::kOpF16KN> : fg::fg_umma_chain_kernel<fg::kOpF16NK>;
  std::unique_lock<std::mutex> lk(g_dev_mu);
  int& set = dev->smem_set_chain[ch->op == FG_OP_F16_NK];
  cudaError_t e;
  if (ch->smem_bytes > set) {
    e = cudaFuncSetAttribute(reinterpret_cast<const void*>(kern), cudaFuncAttributeMaxDynamicSharedMemorySize,
                             ch->smem_bytes);
    if (e != cudaSuccess) {
      g_last_cuda = static_cast<int>(e);
      return FG_ERR_CUDA;
    }
    set = ch->smem_bytes;
  }
  lk.unlock();
  uint8_t* wsb = static_cast<uint8_t*>(ws);
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  e = cudaMemsetAsync(wsb + ch->off_done, 0, 4 * static_cast<size_t>(ch->count), s);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  fg::CParams g = {};
  g.table = ch->table_dev;
  g.count = ch->count;
  g.partials = reinterpret_cast<float*>(wsb + FG_WS_HEADER_BYTES);
  g.tickets = reinterpret_cast<unsigned int*>(wsb + ch->off_tickets);
  g.done = reinterpret_cast<unsigned int*>(wsb + ch->off_done);
  g.status = reinterpret_cast<int*>(wsb);
  g.trace = g_trace.load(std::memory_order_relaxed) ? reinterpret_cast<unsigned long long*>(wsb + ch->off_trace) : nullptr;
  g.chunks_per_stage = ch->chunks;
  g.stages = ch->stages;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(ch->grid);
  cfg.blockDim = dim3(fg::kUmmaThreads);
  cfg.dynamicSmemBytes = ch->smem_bytes;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;  // the CTAs wait on one another: all must be resident
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kern, g);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return FG_OK;
}

int fg_chain_grid(const fg_chain_t* ch) { return ch ? ch->grid : 0; }

size_t fg_chain_trace_offset(const fg_chain_t* ch) { return ch ? ch->off_trace : 0; }

void fg_chain_destroy(fg_chain_t* ch) { delete ch; }

int fg_quantize_rows_w8(const void* W, int8_t* W8, void* scales, int N, int K, fg_stream_t stream) {
  if (W == nullptr || W8 == nullptr || scales == nullptr) return FG_ERR_NULL;
  if (N <= 0 || K <= 0 || (K % 8) != 0) return FG_ERR_SHAPE;
  if (!aligned16(W) || (reinterpret_cast<uintptr_t>(W8) & 7u) != 0 || (reinterpret_cast<uintptr_t>(scales) & 1u) != 0)
    return FG_ERR_ALIGN;
  fg::fg_quantize_rows_kernel<<<N, fg::kQuantThreads, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(W), W8, static_cast<__half*>(scales), K);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return FG_OK;
}

int fg_quantize_rows_w4(const void* W, uint8_t* W4, void* scales, int groups, int N, int K, fg_stream_t stream) {
  if (W == nullptr || W4 == nullptr || scales == nullptr) return FG_ERR_NULL;
  if (N <= 0 || K <= 0 || (K % 128) != 0 || (groups != 1 && groups != K / 128)) return FG_ERR_SHAPE;
  if (!aligned16(W) || (reinterpret_cast<uintptr_t>(W4) & 3u) != 0 || (reinterpret_cast<uintptr_t>(scales) & 1u) != 0)
    return FG_ERR_ALIGN;
  const long long segments = static_cast<long long>(N) * groups;
  const int per_cta = fg::kQuantThreads / 32;
  const long long grid = (segments + per_cta - 1) / per_cta;
  if (grid > 0x7fffffffLL) return FG_ERR_SHAPE;
  fg::fg_quantize_rows_w4_kernel<<<static_cast<unsigned int>(grid), fg::kQuantThreads, 0,
                                   reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(W), W4, static_cast<__half*>(scales), K, K / groups, segments);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return FG_OK;
}

int fg_gemm_fused(int op, const void* x, const void* W, const void* scales, void* C, int M, int N, int K,
                  const fg_epilogue_t* ep, void* ws, size_t ws_bytes, fg_stream_t stream) {
  if (op < FG_OP_F16_KN || op > FG_OP_W8A16_NK) return FG_ERR_PLAN;
  int st = check_common(x, W, C, M, N, K, ws, ws_bytes);
  if (st != FG_OK) return st;
  bool gate = false;
  if (ep != nullptr) {
    if (ep->act < FG_ACT_NONE || ep->act > FG_ACT_SILU_GATE) return FG_ERR_PLAN;
    if ((reinterpret_cast<uintptr_t>(ep->bias) & 1u) != 0 || (reinterpret_cast<uintptr_t>(ep->residual) & 1u) != 0)
      return FG_ERR_ALIGN;
    gate = (ep->act == FG_ACT_SILU_GATE);
    if (gate && (op != FG_OP_F16_NK || ep->split1 != 0)) return FG_ERR_PLAN;  // interleaved NxK fp16 weights, one output
    if (ep->split1 != 0 || ep->split2 != 0) {
      if (ep->split1 <= 0 || ep->split2 < ep->split1 || ep->split2 > N || (ep->split1 % 8) != 0 || (ep->split2 % 8) != 0)
        return FG_ERR_SHAPE;
      if ((ep->split2 > ep->split1 && ep->C2 == nullptr) || (N > ep->split2 && ep->C3 == nullptr)) return FG_ERR_NULL;
      if (!aligned16(ep->C2) || !aligned16(ep->C3)) return FG_ERR_ALIGN;
    }
  }
  if (scales != nullptr && (reinterpret_cast<uintptr_t>(scales) & 3u) != 0) return FG_ERR_ALIGN;
  DeviceInfo* dev = nullptr;
  if ((st = device_info(&dev)) != FG_OK) return st;
  fg_plan_t pl;
  if (gate) {
    // the tcgen05 kernel, whose epilogue warps swap gate and up sums through 8 KB more of shared memory
    if ((st = fg_plan_tiled(op, M, N, K, dev->sm_count, dev->smem_optin, &pl)) != FG_OK) return st;
    if (pl.math != 2) return FG_ERR_PLAN;
    pl.smem_bytes += static_cast<int>(fg::kGateXchBytes);
    if (pl.smem_bytes > dev->smem_optin) return FG_ERR_PLAN;
  } else if ((st = fg_plan(op, M, N, K, dev->sm_count, dev->smem_optin, &pl)) != FG_OK) {
    return st;
  }
  return run_planned(pl, dev, x, W, op == FG_OP_W8A16_NK ? scales : nullptr, C, M, N, K, ws,
                     reinterpret_cast<cudaStream_t>(stream), nullptr, ep);
}

// ---- one-time weight repacking ---------------------------------------------------------------
int fg_prepack_kn_to_nk(const void* B, void* W, int N, int K, fg_stream_t stream) {
  if (B == nullptr || W == nullptr) return FG_ERR_NULL;
  if (N <= 0 || K <= 0 || (N % 64) != 0 || (K % 64) != 0) return FG_ERR_SHAPE;
  if (!aligned16(B) || !aligned16(W)) return FG_ERR_ALIGN;
  const dim3 grid(N / 64, K / 64);
  fg::fg_transpose_kn_to_nk_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(B), static_cast<__half*>(W), N, K);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return FG_OK;
}

int fg_prepack_gate_up(const void* Wg, const void* Wu, void* Wgu, int N, int K, fg_stream_t stream) {
  if (Wg == nullptr || Wu == nullptr || Wgu == nullptr) return FG_ERR_NULL;
  if (N <= 0 || K <= 0 || (N % 64) != 0 || (K % 128) != 0) return FG_ERR_SHAPE;
  if (!aligned16(Wg) || !aligned16(Wu) || !aligned16(Wgu)) return FG_ERR_ALIGN;
  // blocks of 64 rows are contiguous in all three matrices: 2 * N / 64 plain copies as one kernel
  const long long chunks16 = static_cast<long long>(64) * K * 2 / 16;  // 16-byte pieces per block of rows
  const dim3 grid(static_cast<unsigned>((chunks16 + 1023) / 1024), 2 * (N / 64));
  fg::fg_interleave_gate_up_kernel<<<grid, 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(Wg), static_cast<const uint4*>(Wu), static_cast<uint4*>(Wgu), static_cast<int>(chunks16));
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return FG_OK;
}

int fg_linear_host(int op, const void* x_host, const void* W_dev, const void* scales_dev, void* C_host,
                   void* x_stage_dev, void* C_stage_dev, int M, int N, int K, void* ws,
                   size_t ws_bytes, fg_stream_t stream) {
  if (x_host == nullptr || C_host == nullptr || x_stage_dev == nullptr || C_stage_dev == nullptr)
    return FG_ERR_NULL;
  if (op < FG_OP_F16_KN || op > FG_OP_W8A16_NK) return FG_ERR_PLAN;
  if (M <= 0 || N <= 0 || K <= 0) return FG_ERR_SHAPE;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemcpyAsync(x_stage_dev, x_host, static_cast<size_t>(M) * K * 2,
                                  cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  const int st = run_op(op, x_stage_dev, W_dev, op == FG_OP_W8A16_NK ? scales_dev : nullptr,
                        C_stage_dev, M, N, K, ws, ws_bytes, stream);
  if (st != FG_OK) return st;
  e = cudaMemcpyAsync(C_host, C_stage_dev, static_cast<size_t>(M) * N * 2, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  return FG_OK;
}

int fg_trace_enable(int on) {
  g_trace.store(on ? 1 : 0, std::memory_order_relaxed);
  g_trace_seq.store(0, std::memory_order_relaxed);
  return FG_OK;
}

int fg_trace_read(void* ws, unsigned long long* out, int ctas, fg_stream_t stream) {
  if (ws == nullptr || out == nullptr) return FG_ERR_NULL;
  if (ctas < 1 || ctas > kTraceFirstCta) return FG_ERR_PLAN;  // 64 B per CTA, far below the borrowed slots
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  uint8_t* src = static_cast<uint8_t*>(ws) + FG_WS_HEADER_BYTES +
                 static_cast<size_t>(kTraceFirstCta) * 2 * FG_WS_PARTIAL_TILE_BYTES;
  const size_t bytes = static_cast<size_t>(ctas) * fg::kTraceSlots * sizeof(unsigned long long);
  cudaError_t e = cudaMemcpyAsync(out, src, bytes, cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e == cudaSuccess) e = cudaMemsetAsync(src, 0, bytes, s);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  return FG_OK;
}

int fg_gemm_f16_nk_noalloc(const void* x, const void* W, void* C, int M, int N, int K,
                           fg_stream_t stream) {
  if (x == nullptr || W == nullptr || C == nullptr) return FG_ERR_NULL;
  if (M <= 0 || N <= 0 || K <= 0 || (N % 128) != 0 || (K % 128) != 0) return FG_ERR_SHAPE;
  if (N > kNoAllocMaxN) return FG_ERR_WORKSPACE;  // more output tiles than the built-in scratch has counters for
  if (!aligned16(x) || !aligned16(W) || !aligned16(C)) return FG_ERR_ALIGN;
  DeviceInfo* dev = nullptr;
  int st = device_info(&dev);
  if (st != FG_OK) return st;
  int dev_index = 0;
  cudaError_t e = cudaGetDevice(&dev_index);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  unsigned char* scratch = nullptr;
  if ((st = noalloc_scratch(dev_index, &scratch)) != FG_OK) return st;

  fg_plan_t pl;
  const int sms = dev->sm_count < kNoAllocMaxGrid ? dev->sm_count : kNoAllocMaxGrid;
  // The built-in scratch holds 16-row partial tiles: plan (and run) in passes of at most 16 rows.
  if ((st = fg_plan_tiled(FG_OP_F16_NK, M < 16 ? M : 16, N, K, sms, dev->smem_optin, &pl)) != FG_OK) return st;
  if (pl.grid > kNoAllocMaxGrid || pl.m_tile > 16 || pl.math >= 4) return FG_ERR_WORKSPACE;
  pl.pdl = 0;  // a memset precedes every launch, so there is no kernel to overlap with

  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  KernelFn kern = nullptr;
  if ((st = prepare_kernel(pl, dev, &kern)) != FG_OK) return st;
  CUtensorMap tmW;
  if ((st = encode_2d(&tmW, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, W, K, N, 64, 128)) != FG_OK) return st;

  fg::KParams p = {};
  p.scales = nullptr;
  p.status = reinterpret_cast<int*>(scratch);
  p.tickets = reinterpret_cast<unsigned int*>(scratch + kNoAllocTicketsOffset);
  p.partials = reinterpret_cast<float*>(scratch + kNoAllocPartialsOffset);
  p.trace = nullptr;
  p.N = N;
  p.K = K;
  p.tiles = pl.tiles;
  p.k_blocks = pl.k_blocks;
  p.chunks_per_stage = pl.k_per_stage / fg_chunk_k(FG_OP_F16_NK);
  p.stages = pl.stages;
  p.consumer_warps = pl.consumer_warps;
  p.pdl = 0;
  p.l2_prefetch = 0;
  p.bias = nullptr;
  p.residual = nullptr;
  p.act = 0;
  p.split1 = p.split2 = 0;
  p.C2 = p.C3 = nullptr;
  p.mc_C = nullptr;
  p.mc_flag = nullptr;
  p.scale_groups = 1;
  p.w4_magic = 0;
  p.world = 0;
  p.rank = 0;
  p.col0 = 0;
  p.ldc = N;
  p.wait_flags = nullptr;
  p.wait_world = 0;
  p.wait_target = 0;
  for (int m0 = 0; m0 < M; m0 += 16) {
    const int mp = (M - m0) < 16 ? (M - m0) : 16;
    // The array is shared by every call and keeps what the last one left: the status word
    // and the arrival counters must read zero when the kernel starts.
    e = cudaMemsetAsync(scratch, 0, kNoAllocPartialsOffset, s);
    if (e != cudaSuccess) {
      g_last_cuda = static_cast<int>(e);
      return FG_ERR_CUDA;
    }
    CUtensorMap tmX;
    const __half* xp = static_cast<const __half*>(x) + static_cast<size_t>(m0) * K;
    if ((st = encode_2d(&tmX, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, xp, K, mp, 64, pl.m_tile)) != FG_OK) return st;
    p.C = static_cast<__half*>(C) + static_cast<size_t>(m0) * N;
    p.M = mp;
    if ((st = launch_one(pl, kern, tmW, tmX, p, s)) != FG_OK) return st;
  }
  return FG_OK;
}

int fg_noalloc_status(int* status_out, fg_stream_t stream) {
  if (status_out == nullptr) return FG_ERR_NULL;
  DeviceInfo* dev = nullptr;
  int st = device_info(&dev);
  if (st != FG_OK) return st;
  int dev_index = 0;
  cudaError_t e = cudaGetDevice(&dev_index);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  unsigned char* scratch = nullptr;
  if ((st = noalloc_scratch(dev_index, &scratch)) != FG_OK) return st;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int v = 0;
  e = cudaMemcpyAsync(&v, scratch, sizeof(int), cudaMemcpyDeviceToHost, s);
  if (e == cudaSuccess) e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) {
    g_last_cuda = static_cast<int>(e);
    return FG_ERR_CUDA;
  }
  *status_out = v;
  return FG_OK;
}

const char* fg_status_str(int status) {
  switch (status) {
    case FG_OK: return "ok";
    case FG_ERR_SHAPE: return "K(input column) & N(output column) must be multiple of 128!";
    case FG_ERR_ALIGN: return "pointer is not 16-byte aligned";
    case FG_ERR_NULL: return "required pointer is NULL";
    case FG_ERR_WORKSPACE: return "workspace missing, misaligned or too small";
    case FG_ERR_CUDA: return "CUDA call failed";
    case FG_ERR_TIMEOUT: return "bounded device-side wait gave up";
    case FG_ERR_PLAN: return "plan is not launchable";
    case FG_ERR_NO_DEVICE: return "no sm_100 device is current";
    default: return "unknown status";
  }
}

int fg_last_cuda_error(void) { return g_last_cuda; }
unsigned long long fg_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
const char* fg_version(void) { return "fastgate_b200 0.1 sm_100a"; }

}  // extern "C"
