// pybind11 / torch-extension surface of fastgate_b200.
//
// Same operator names, positional argument order and in-place-output convention as the
// reference's host launchers (chanzhennan/Fastgate: backend/cuda/hk/edgemm.h:4-14,
// edgemm_tr.h:7-11, flatgemm.h:4-10, fastgemv.h:4-7, backend/cuda/czn/fastgemm.h:4; bound
// the way backend/pybind.cpp:21-27 binds free functions taking at::Tensor by value).
// Every op is a thin layer over the C ABI (include/fastgate_b200.h): it validates the
// tensors, picks the current CUDA stream and a cached per-(device, stream) workspace, and
// turns status codes into exceptions.  There is no CPU path.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>
#include <mutex>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include "../../include/fastgate_b200.h"

namespace {

struct Workspace {
  at::Tensor buf;
  size_t bytes = 0;
};
std::mutex g_ws_mu;
std::map<std::pair<int, int64_t>, Workspace> g_ws;

// One workspace per (device, stream): calls on one stream are ordered, calls on different
// streams may overlap and must not share partial tiles or arrival counters.  Returned by value
// (a tensor handle and its size): the handle keeps the memory alive for the caller even if
// another thread replaces the map entry with a larger buffer meanwhile.
Workspace workspace_for(int device, cudaStream_t stream, int N) {
  const size_t need = fg_workspace_bytes(N);
  std::lock_guard<std::mutex> lk(g_ws_mu);
  Workspace& w = g_ws[{device, reinterpret_cast<int64_t>(stream)}];
  if (w.bytes < need) {
    const size_t bytes = std::max<size_t>(need, fg_workspace_bytes(65536));
    w.buf = at::empty({static_cast<int64_t>(bytes)},
                      at::TensorOptions().dtype(at::kByte).device(at::kCUDA, device));
    const int st = fg_workspace_init(w.buf.data_ptr(), bytes, reinterpret_cast<fg_stream_t>(stream));
    if (st != FG_OK) throw std::runtime_error(std::string("fastgate_b200: ") + fg_status_str(st));
    w.bytes = bytes;
  }
  return w;
}

void check_tensor(const at::Tensor& t, const char* name, at::ScalarType dt) {
  if (!t.is_cuda()) throw std::runtime_error(std::string("fastgate_b200: ") + name + " must be a CUDA tensor (there is no CPU path)");
  if (t.scalar_type() != dt) throw std::runtime_error(std::string("fastgate_b200: ") + name + " has the wrong dtype");
  if (!t.is_contiguous()) throw std::runtime_error(std::string("fastgate_b200: ") + name + " must be contiguous");
}

[[noreturn]] void raise(int st, bool transposed_weight) {
  if (st == FG_ERR_SHAPE) {
    // texts of backend/cuda/hk/edgemm.cu:108 and :280
    throw std::invalid_argument(transposed_weight
                                    ? "K(input column) & N(transposed output row) must be multiple of 128!"
                                    : "K(input column) & N(output column) must be multiple of 128!");
  }
  throw std::runtime_error(std::string("fastgate_b200: ") + fg_status_str(st) + " (cuda error " +
                           std::to_string(fg_last_cuda_error()) + ")");
}

// x[M,K] (fp16), weight in the given layout, C with M*N elements (fp16), scales[N] or undefined.
void linear(int op, const at::Tensor& x, const at::Tensor& W, at::Tensor& C, const c10::optional<at::Tensor>& scales) {
  check_tensor(x, "activation", at::kHalf);
  check_tensor(W, "weight", op == FG_OP_W8A16_NK ? at::kChar : at::kHalf);
  check_tensor(C, "output", at::kHalf);
  if (x.dim() != 2 || W.dim() != 2) throw std::runtime_error("fastgate_b200: activation and weight must be 2-D");
  const int64_t M = x.size(0), K = x.size(1);
  const int64_t N = (op == FG_OP_F16_KN) ? W.size(1) : W.size(0);
  const int64_t Kw = (op == FG_OP_F16_KN) ? W.size(0) : W.size(1);
  if (Kw != K) throw std::runtime_error("fastgate_b200: activation and weight disagree on K");
  if (C.numel() != M * N) throw std::runtime_error("fastgate_b200: output must hold M*N elements");
  if (W.get_device() != x.get_device() || C.get_device() != x.get_device())
    throw std::runtime_error("fastgate_b200: all tensors must live on one device");
  const void* sp = nullptr;
  if (scales.has_value() && scales->defined()) {
    if (op != FG_OP_W8A16_NK) throw std::runtime_error("fastgate_b200: scales only apply to int8 weights");
    check_tensor(*scales, "scales", at::kHalf);
    if (scales->numel() != N) throw std::runtime_error("fastgate_b200: scales must hold N elements");
    sp = scales->data_ptr();
  }
  if (M == 0) return;
  if ((N % 128) != 0 || (K % 128) != 0 || N <= 0 || K <= 0) raise(FG_ERR_SHAPE, op != FG_OP_F16_KN);

  const c10::cuda::CUDAGuard guard(x.device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(x.get_device()).stream();
  const Workspace ws = workspace_for(x.get_device(), stream, static_cast<int>(N));
  int st;
  {
    pybind11::gil_scoped_release nogil;
    fg_stream_t s = reinterpret_cast<fg_stream_t>(stream);
    if (op == FG_OP_F16_KN)
      st = fg_gemm_f16_kn(x.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, ws.buf.data_ptr(), ws.bytes, s);
    else if (op == FG_OP_F16_NK)
      st = fg_gemm_f16_nk(x.data_ptr(), W.data_ptr(), C.data_ptr(), M, N, K, ws.buf.data_ptr(), ws.bytes, s);
    else
      st = fg_gemm_w8a16_nk(x.data_ptr(), static_cast<const int8_t*>(W.data_ptr()), sp, C.data_ptr(), M, N, K,
                            ws.buf.data_ptr(), ws.bytes, s);
  }
  if (st != FG_OK) raise(st, op != FG_OP_F16_KN);
}

// ---- the three calling conventions of the reference ---------------------------------------
// (A[M,K], B[K,N], C)                     edgemm*, edgemv*, flat_gemm_*
void op_kn(at::Tensor A, at::Tensor B, at::Tensor C) { linear(FG_OP_F16_KN, A, B, C, c10::nullopt); }
// the reference's bz argument chose the split-K factor by hand; here it is accepted and ignored
void op_kn_bz(at::Tensor A, at::Tensor B, at::Tensor C, int /*bz*/) { linear(FG_OP_F16_KN, A, B, C, c10::nullopt); }
// (A[M,K], W[N,K], C)                     edgemm_*_bt, *_tr_amd, gemm_*_bt
void op_nk(at::Tensor A, at::Tensor W, at::Tensor C) { linear(FG_OP_F16_NK, A, W, C, c10::nullopt); }
void op_nk_bz(at::Tensor A, at::Tensor W, at::Tensor C, int /*bz*/) { linear(FG_OP_F16_NK, A, W, C, c10::nullopt); }
// (W[N,K], x[M,K], C)  weight first        fastgemv*, fastgemm
void op_wfirst(at::Tensor W, at::Tensor x, at::Tensor C) { linear(FG_OP_F16_NK, x, W, C, c10::nullopt); }
void op_wfirst_int8(at::Tensor W8, at::Tensor x, at::Tensor C, c10::optional<at::Tensor> scales) {
  linear(FG_OP_W8A16_NK, x, W8, C, scales);
}

// (W4[N,K/2] uint8, x[M,K], C)  int4 weight-only: two unsigned 4-bit values per byte, low nibble
// first (uint4_2, backend/cuda/hk/utility.cuh:13-36); scales [N] / [N,1] or [N,K/128] or None.
void op_wfirst_int4(at::Tensor W4, at::Tensor x, at::Tensor C, c10::optional<at::Tensor> scales, int zero_point) {
  check_tensor(x, "activation", at::kHalf);
  check_tensor(W4, "weight", at::kByte);
  check_tensor(C, "output", at::kHalf);
  if (x.dim() != 2 || W4.dim() != 2) throw std::runtime_error("fastgate_b200: activation and weight must be 2-D");
  const int64_t M = x.size(0), K = x.size(1), N = W4.size(0);
  if (W4.size(1) * 2 != K) throw std::runtime_error("fastgate_b200: activation and weight disagree on K");
  if (C.numel() != M * N) throw std::runtime_error("fastgate_b200: output must hold M*N elements");
  if (W4.get_device() != x.get_device() || C.get_device() != x.get_device())
    throw std::runtime_error("fastgate_b200: all tensors must live on one device");
  if (zero_point < 0 || zero_point > 15) throw std::invalid_argument("fastgate_b200: zero_point must be 0..15");
  const void* sp = nullptr;
  int groups = 1;
  if (scales.has_value() && scales->defined()) {
    check_tensor(*scales, "scales", at::kHalf);
    if (N > 0 && scales->numel() % N == 0) groups = static_cast<int>(scales->numel() / N);
    if (scales->numel() != N * groups || (groups != 1 && groups != K / 128))
      throw std::runtime_error("fastgate_b200: scales must hold N or N * K/128 elements");
    sp = scales->data_ptr();
  }
  if (M == 0) return;
  if ((N % 128) != 0 || (K % 128) != 0 || N <= 0 || K <= 0) raise(FG_ERR_SHAPE, true);
  const c10::cuda::CUDAGuard guard(x.device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(x.get_device()).stream();
  const Workspace ws = workspace_for(x.get_device(), stream, static_cast<int>(N));
  int st;
  {
    pybind11::gil_scoped_release nogil;
    st = fg_gemm_w4a16_nk(x.data_ptr(), static_cast<const uint8_t*>(W4.data_ptr()), sp, groups, zero_point,
                          C.data_ptr(), M, N, K, ws.buf.data_ptr(), ws.bytes, reinterpret_cast<fg_stream_t>(stream));
  }
  if (st != FG_OK) raise(st, true);
}

// ---- N-sharded layer with the all-gather fused into the epilogue --------------------------
// x[M,K] fp16 (replicated), W[N_local,K] fp16 (this rank's rows); c_ptrs / flag_ptrs are the
// device addresses, as mapped into this process, of every rank's full output [M, n_total]
// and arrival counter (e.g. buffer_ptrs of a torch symmetric-memory allocation).
void linear_nk_push(at::Tensor x, at::Tensor W, std::vector<int64_t> c_ptrs, std::vector<int64_t> flag_ptrs,
                    int64_t rank, int64_t n_total, int64_t wait_flag_ptr, int64_t wait_target, int64_t mc_c_ptr,
                    int64_t mc_flag_ptr, int64_t target_dev_ptr, int64_t wait_target_dev_ptr) {
  check_tensor(x, "activation", at::kHalf);
  check_tensor(W, "weight", at::kHalf);
  if (x.dim() != 2 || W.dim() != 2 || x.size(1) != W.size(1))
    throw std::runtime_error("fastgate_b200: activation [M,K] and weight [N_local,K] expected");
  if (c_ptrs.size() != flag_ptrs.size() || c_ptrs.empty() || c_ptrs.size() > 8)
    throw std::runtime_error("fastgate_b200: 1..8 peers expected");
  const int64_t M = x.size(0), K = x.size(1), N = W.size(0);
  if (M == 0) return;
  if ((N % 128) != 0 || (K % 128) != 0) raise(FG_ERR_SHAPE, true);
  fg_peers_t peers = {};
  peers.world = static_cast<int>(c_ptrs.size());
  peers.rank = static_cast<int>(rank);
  peers.n_total = n_total;
  peers.wait_flags = reinterpret_cast<const unsigned long long*>(wait_flag_ptr);
  peers.wait_target = static_cast<unsigned long long>(wait_target);
  peers.mc_C = reinterpret_cast<void*>(mc_c_ptr);                       // multicast mappings, 0 = none
  peers.mc_flag = reinterpret_cast<unsigned long long*>(mc_flag_ptr);
  // running totals kept on the device (0 = the caller counts): what makes the call replayable in a graph
  peers.target_dev = reinterpret_cast<unsigned long long*>(target_dev_ptr);
  peers.wait_target_dev = reinterpret_cast<const unsigned long long*>(wait_target_dev_ptr);
  for (size_t q = 0; q < c_ptrs.size(); ++q) {
    peers.C[q] = reinterpret_cast<void*>(c_ptrs[q]);
    peers.flag[q] = reinterpret_cast<unsigned long long*>(flag_ptrs[q]);
  }
  const c10::cuda::CUDAGuard guard(x.device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(x.get_device()).stream();
  const Workspace ws = workspace_for(x.get_device(), stream, static_cast<int>(N));
  int st;
  {
    pybind11::gil_scoped_release nogil;
    st = fg_gemm_f16_nk_push(x.data_ptr(), W.data_ptr(), M, N, K, &peers, ws.buf.data_ptr(), ws.bytes,
                             reinterpret_cast<fg_stream_t>(stream));
  }
  if (st != FG_OK) raise(st, true);
}

// Enqueues the bounded wait for this rank's arrival counter on the current stream.
void push_wait(int64_t flag_ptr, int64_t world, int64_t target, int64_t device) {
  const c10::cuda::CUDAGuard guard(c10::Device(c10::kCUDA, static_cast<c10::DeviceIndex>(device)));
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(device).stream();
  const Workspace ws = workspace_for(static_cast<int>(device), stream, 128);
  const int st = fg_push_wait(reinterpret_cast<const unsigned long long*>(flag_ptr), static_cast<int>(world),
                              static_cast<unsigned long long>(target), ws.buf.data_ptr(),
                              reinterpret_cast<fg_stream_t>(stream));
  if (st != FG_OK) raise(st, true);
}

// The same wait with its target read on the device from the running total at target_dev_ptr.
void push_wait_dev(int64_t flag_ptr, int64_t world, int64_t target_dev_ptr, int64_t device) {
  const c10::cuda::CUDAGuard guard(c10::Device(c10::kCUDA, static_cast<c10::DeviceIndex>(device)));
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(device).stream();
  const Workspace ws = workspace_for(static_cast<int>(device), stream, 128);
  const int st = fg_push_wait_dev(reinterpret_cast<const unsigned long long*>(flag_ptr), static_cast<int>(world),
                                  reinterpret_cast<const unsigned long long*>(target_dev_ptr), ws.buf.data_ptr(),
                                  reinterpret_cast<fg_stream_t>(stream));
  if (st != FG_OK) raise(st, true);
}

// Several such waits as one launch.
void push_wait_dev_many(std::vector<int64_t> flag_ptrs, std::vector<int64_t> target_dev_ptrs, int64_t world, int64_t device) {
  if (flag_ptrs.size() != target_dev_ptrs.size() || flag_ptrs.empty()) throw std::runtime_error("fastgate_b200: one total per flag array expected");
  const c10::cuda::CUDAGuard guard(c10::Device(c10::kCUDA, static_cast<c10::DeviceIndex>(device)));
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(device).stream();
  const Workspace ws = workspace_for(static_cast<int>(device), stream, 128);
  std::vector<const unsigned long long*> f, t;
  for (size_t i = 0; i < flag_ptrs.size(); ++i) {
    f.push_back(reinterpret_cast<const unsigned long long*>(flag_ptrs[i]));
    t.push_back(reinterpret_cast<const unsigned long long*>(target_dev_ptrs[i]));
  }
  const int st = fg_push_wait_dev_many(f.data(), t.data(), static_cast<int>(f.size()), static_cast<int>(world), ws.buf.data_ptr(),
                                       reinterpret_cast<fg_stream_t>(stream));
  if (st != FG_OK) raise(st, true);
}

// Device status word of the current stream's workspace (synchronises the stream).
int64_t workspace_status(int64_t device) {
  const c10::cuda::CUDAGuard guard(c10::Device(c10::kCUDA, static_cast<c10::DeviceIndex>(device)));
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(device).stream();
  const Workspace ws = workspace_for(static_cast<int>(device), stream, 128);
  int v = -1;
  const int st = fg_workspace_status(ws.buf.data_ptr(), &v, reinterpret_cast<fg_stream_t>(stream));
  if (st != FG_OK) raise(st, true);
  return v;
}

// Linear layer with a fused epilogue: C = act(x . W^T * scales + bias) + residual.
// layout "nk": W[N,K] (fp16, or int8 with optional scales); "kn": W[K,N] fp16.
// act "silu_gate": W is the interleaved gate/up weight of prepack_gate_up, C and residual are [M, N/2].
// C2, C3: the output columns are split over C, C2 and C3 in that order (their widths add up to N).
void linear_fused(at::Tensor x, at::Tensor W, at::Tensor C, c10::optional<at::Tensor> scales,
                  c10::optional<at::Tensor> bias, c10::optional<at::Tensor> residual, const std::string& act,
                  const std::string& layout, c10::optional<at::Tensor> C2, c10::optional<at::Tensor> C3) {
  int act_code;
  if (act == "none") act_code = FG_ACT_NONE;
  else if (act == "gelu" || act == "gelu_erf") act_code = FG_ACT_GELU_ERF;
  else if (act == "gelu_tanh") act_code = FG_ACT_GELU_TANH;
  else if (act == "silu") act_code = FG_ACT_SILU;
  else if (act == "silu_gate") act_code = FG_ACT_SILU_GATE;
  else throw std::invalid_argument("fastgate_b200: act must be none, gelu, gelu_tanh, silu or silu_gate");
  const bool gate = act_code == FG_ACT_SILU_GATE;
  if (layout != "nk" && layout != "kn") throw std::invalid_argument("fastgate_b200: layout must be nk or kn");
  const bool int8w = W.scalar_type() == at::kChar;
  if (int8w && layout == "kn") throw std::invalid_argument("fastgate_b200: int8 weights are stored NxK");
  const int op = layout == "kn" ? FG_OP_F16_KN : (int8w ? FG_OP_W8A16_NK : FG_OP_F16_NK);
  check_tensor(x, "activation", at::kHalf);
  check_tensor(W, "weight", int8w ? at::kChar : at::kHalf);
  check_tensor(C, "output", at::kHalf);
  if (x.dim() != 2 || W.dim() != 2) throw std::runtime_error("fastgate_b200: activation and weight must be 2-D");
  const int64_t M = x.size(0), K = x.size(1);
  const int64_t N = (op == FG_OP_F16_KN) ? W.size(1) : W.size(0);
  if (((op == FG_OP_F16_KN) ? W.size(0) : W.size(1)) != K) throw std::runtime_error("fastgate_b200: activation and weight disagree on K");
  if (gate && (layout != "nk" || int8w)) throw std::invalid_argument("fastgate_b200: silu_gate takes fp16 NxK weights (prepack_gate_up)");
  const int64_t n_out = gate ? N / 2 : N;  // columns of the result
  fg_epilogue_t ep = {nullptr, nullptr, act_code, 0, 0, nullptr, nullptr};
  const bool has2 = C2.has_value() && C2->defined(), has3 = C3.has_value() && C3->defined();
  if (has2 || has3) {
    if (gate) throw std::invalid_argument("fastgate_b200: silu_gate writes one output");
    if (!has2) throw std::invalid_argument("fastgate_b200: C3 without C2");
    check_tensor(*C2, "output C2", at::kHalf);
    if (has3) check_tensor(*C3, "output C3", at::kHalf);
    if (M > 0 && (C.numel() % M || C2->numel() % M || (has3 && C3->numel() % M)))
      throw std::runtime_error("fastgate_b200: split outputs must hold M rows each");
    const int64_t n1 = M > 0 ? C.numel() / M : 0, n2 = M > 0 ? C2->numel() / M : 0, n3 = (has3 && M > 0) ? C3->numel() / M : 0;
    if (M > 0 && n1 + n2 + n3 != N) throw std::runtime_error("fastgate_b200: widths of the split outputs must add up to N");
    ep.split1 = static_cast<int>(n1);
    ep.split2 = static_cast<int>(n1 + n2);
    ep.C2 = C2->data_ptr();
    ep.C3 = has3 ? C3->data_ptr() : nullptr;
  } else if (C.numel() != M * n_out) {
    throw std::runtime_error("fastgate_b200: output must hold M*N elements (M*N/2 with silu_gate)");
  }
  const void* sp = nullptr;
  if (scales.has_value() && scales->defined()) {
    if (!int8w) throw std::runtime_error("fastgate_b200: scales only apply to int8 weights");
    check_tensor(*scales, "scales", at::kHalf);
    if (scales->numel() != N) throw std::runtime_error("fastgate_b200: scales must hold N elements");
    sp = scales->data_ptr();
  }
  if (bias.has_value() && bias->defined()) {
    check_tensor(*bias, "bias", at::kHalf);
    if (bias->numel() != N) throw std::runtime_error("fastgate_b200: bias must hold N elements");
    ep.bias = bias->data_ptr();
  }
  if (residual.has_value() && residual->defined()) {
    check_tensor(*residual, "residual", at::kHalf);
    if (residual->numel() != M * n_out) throw std::runtime_error("fastgate_b200: residual must hold as many elements as the output");
    ep.residual = residual->data_ptr();
  }
  if (M == 0) return;
  if ((N % 128) != 0 || (K % 128) != 0) raise(FG_ERR_SHAPE, op != FG_OP_F16_KN);
  const c10::cuda::CUDAGuard guard(x.device());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(x.get_device()).stream();
  const Workspace ws = workspace_for(x.get_device(), stream, static_cast<int>(N));
  int st;
  {
    pybind11::gil_scoped_release nogil;
    st = fg_gemm_fused(op, x.data_ptr(), W.data_ptr(), sp, C.data_ptr(), M, N, K, &ep, ws.buf.data_ptr(), ws.bytes,
                       reinterpret_cast<fg_stream_t>(stream));
  }
  if (st != FG_OK) raise(st, op != FG_OP_F16_KN);
}

// B[K,N] fp16 -> W[N,K] fp16.
at::Tensor prepack_kn_to_nk(at::Tensor B) {
  check_tensor(B, "weight", at::kHalf);
  if (B.dim() != 2 || (B.size(0) % 64) != 0 || (B.size(1) % 64) != 0)
    throw std::invalid_argument("fastgate_b200: weight [K,N] with K and N multiples of 64 expected");
  const c10::cuda::CUDAGuard guard(B.device());
  at::Tensor W = at::empty({B.size(1), B.size(0)}, B.options());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(B.get_device()).stream();
  const int st = fg_prepack_kn_to_nk(B.data_ptr(), W.data_ptr(), static_cast<int>(B.size(1)), static_cast<int>(B.size(0)),
                                     reinterpret_cast<fg_stream_t>(stream));
  if (st != FG_OK) raise(st, true);
  return W;
}

// Wg[N,K], Wu[N,K] fp16 -> Wgu[2N,K] fp16, blocks of 64 rows interleaved (gate first).
at::Tensor prepack_gate_up(at::Tensor Wg, at::Tensor Wu) {
  check_tensor(Wg, "gate weight", at::kHalf);
  check_tensor(Wu, "up weight", at::kHalf);
  if (Wg.dim() != 2 || Wg.sizes() != Wu.sizes() || (Wg.size(0) % 64) != 0 || (Wg.size(1) % 128) != 0)
    throw std::invalid_argument("fastgate_b200: gate and up weights [N,K] of one shape, N % 64 == 0, K % 128 == 0 expected");
  const c10::cuda::CUDAGuard guard(Wg.device());
  at::Tensor Wgu = at::empty({2 * Wg.size(0), Wg.size(1)}, Wg.options());
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(Wg.get_device()).stream();
  const int st = fg_prepack_gate_up(Wg.data_ptr(), Wu.data_ptr(), Wgu.data_ptr(), static_cast<int>(Wg.size(0)),
                                    static_cast<int>(Wg.size(1)), reinterpret_cast<fg_stream_t>(stream));
  if (st != FG_OK) raise(st, true);
  return Wgu;
}

// W[N,K] fp16 -> (W8[N,K] int8, scales[N] fp16), one scale per output channel.
std::pair<at::Tensor, at::Tensor> quantize_int8(at::Tensor W) {
  check_tensor(W, "weight", at::kHalf);
  if (W.dim() != 2 || (W.size(1) % 8) != 0) throw std::invalid_argument("fastgate_b200: weight [N,K] with K % 8 == 0 expected");
  const c10::cuda::CUDAGuard guard(W.device());
  at::Tensor W8 = at::empty(W.sizes(), W.options().dtype(at::kChar));
  at::Tensor scales = at::empty({W.size(0)}, W.options());
  if (W.numel() == 0) return {W8, scales};
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(W.get_device()).stream();
  const int st = fg_quantize_rows_w8(W.data_ptr(), static_cast<int8_t*>(W8.data_ptr()), scales.data_ptr(),
                                     static_cast<int>(W.size(0)), static_cast<int>(W.size(1)),
                                     reinterpret_cast<fg_stream_t>(stream));
  if (st != FG_OK) raise(st, true);
  return {W8, scales};
}

// W[N,K] fp16 -> (W4[N,K/2] uint8, scales[N,groups] fp16), zero point 8; group_size 128 or 0 (whole row).
std::pair<at::Tensor, at::Tensor> quantize_int4(at::Tensor W, int group_size) {
  check_tensor(W, "weight", at::kHalf);
  if (W.dim() != 2 || (W.size(1) % 128) != 0) throw std::invalid_argument("fastgate_b200: weight [N,K] with K % 128 == 0 expected");
  if (group_size != 0 && group_size != 128) throw std::invalid_argument("fastgate_b200: group_size must be 128 or 0 (one scale per row)");
  const int groups = group_size == 0 ? 1 : static_cast<int>(W.size(1) / 128);
  const c10::cuda::CUDAGuard guard(W.device());
  at::Tensor W4 = at::empty({W.size(0), W.size(1) / 2}, W.options().dtype(at::kByte));
  at::Tensor scales = at::empty({W.size(0), groups}, W.options());
  if (W.numel() == 0) return {W4, scales};
  cudaStream_t stream = at::cuda::getCurrentCUDAStream(W.get_device()).stream();
  const int st = fg_quantize_rows_w4(W.data_ptr(), static_cast<uint8_t*>(W4.data_ptr()), scales.data_ptr(), groups,
                                     static_cast<int>(W.size(0)), static_cast<int>(W.size(1)),
                                     reinterpret_cast<fg_stream_t>(stream));
  if (st != FG_OK) raise(st, true);
  return {W4, scales};
}

// cuBLAS comparators of the reference (backend/cuda/hk/hgemm.cu:29-74, hgemm_tr.cu:30-75):
// library calls, kept only so that scripts which import them keep working.
void hgemm(at::Tensor A, at::Tensor B, at::Tensor C) {
  auto out = C.view({A.size(0), B.size(1)});
  at::matmul_out(out, A, B);
}
void hgemm_tr(at::Tensor A, at::Tensor W, at::Tensor C) {
  auto out = C.view({A.size(0), W.size(0)});
  at::matmul_out(out, A, W.t());
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "fastgate_b200: B200 (sm_100a) small-batch matmul operators with the SPEEDGATE surface";
  namespace py = pybind11;
  // KxN weight: backend/cuda/hk/edgemm.h:4-14
  for (const char* n : {"edgemm", "edgemm_m8n256k64", "edgemm_m8n128k64", "edgemm_m8n128k128",
                        "edgemv_m1n128k64x4", "edgemm_m8n128k64x4", "edgemv_m1n256k64x4",
                        "edgemm_m8n128k64x4_amd", "edgemm_m8n256k32x8"})
    m.def(n, &op_kn, py::arg("A"), py::arg("B"), py::arg("C"));
  // backend/cuda/hk/flatgemm.h:4-10
  for (const char* n : {"flat_gemm_m8n256k32x8_bz1", "flat_gemm_m8n256k32x16"})
    m.def(n, &op_kn, py::arg("A"), py::arg("B"), py::arg("C"));
  for (const char* n : {"flat_gemm_m8n128k64x4_bz1", "flat_gemm_m8n256k64x8", "flat_gemm_m8n512k32x16",
                        "flat_gemm_m8n64k128x8", "flat_gemm_m8n32k256x8"})
    m.def(n, &op_kn_bz, py::arg("A"), py::arg("B"), py::arg("C"), py::arg("bz") = 1);
  // NxK weight, activation first: backend/cuda/hk/edgemm.h:10,14 and edgemm_tr.h:7-11
  for (const char* n : {"edgemm_m8n128k64x4_bt", "edgemm_m8n128k64x4_tr_amd", "gemm_m8n128k64x4_bt",
                        "gemm_m8n32k128x8_bt", "gemm_m8n32k256x8_bt"})
    m.def(n, &op_nk, py::arg("A"), py::arg("B"), py::arg("C"));
  for (const char* n : {"gemm_m8n32k256x8_bt_bz2", "gemm_m8n64k128x8_bt_exp"})
    m.def(n, &op_nk_bz, py::arg("A"), py::arg("B"), py::arg("C"), py::arg("bz") = 1);
  // NxK weight, weight first: backend/cuda/hk/fastgemv.h:4-7, backend/cuda/czn/fastgemm.h:4
  for (const char* n : {"fastgemv", "fastgemv_tuned", "fastgemv_extend", "fastgemm"})
    m.def(n, &op_wfirst, py::arg("A"), py::arg("B"), py::arg("C"));
  m.def("fastgemv_int8", &op_wfirst_int8, py::arg("A"), py::arg("B"), py::arg("C"),
        py::arg("scales") = py::none(),
        "int8 weight W8[N,K], fp16 x[M,K]; scales[N] (fp16) optional: None = scale 1, zero-point 0 "
        "as the reference launches it (backend/cuda/hk/fastgemv.cu:50-59)");
  m.def("hgemm", &hgemm);
  m.def("hgemm_tr", &hgemm_tr);
  m.def("linear_nk_push", &linear_nk_push, py::arg("x"), py::arg("W"), py::arg("c_ptrs"), py::arg("flag_ptrs"),
        py::arg("rank"), py::arg("n_total"), py::arg("wait_flag_ptr") = 0, py::arg("wait_target") = 0,
        py::arg("mc_c_ptr") = 0, py::arg("mc_flag_ptr") = 0, py::arg("target_dev_ptr") = 0, py::arg("wait_target_dev_ptr") = 0);
  m.def("push_wait", &push_wait, py::arg("flag_ptr"), py::arg("world"), py::arg("target"), py::arg("device"));
  m.def("push_wait_dev", &push_wait_dev, py::arg("flag_ptr"), py::arg("world"), py::arg("target_dev_ptr"), py::arg("device"));
  m.def("push_wait_dev_many", &push_wait_dev_many, py::arg("flag_ptrs"), py::arg("target_dev_ptrs"), py::arg("world"), py::arg("device"));
  m.def("workspace_status", &workspace_status, py::arg("device"));
  m.def("prepack_kn_to_nk", &prepack_kn_to_nk, py::arg("B"), "B[K,N] fp16 -> W[N,K] fp16 (one-time repack for the NxK operators)");
  m.def("prepack_gate_up", &prepack_gate_up, py::arg("Wg"), py::arg("Wu"),
        "Wg[N,K], Wu[N,K] fp16 -> Wgu[2N,K]: 64 gate rows, then the matching 64 up rows, per 128 rows (for act='silu_gate')");
  m.def("linear_fused", &linear_fused, py::arg("x"), py::arg("W"), py::arg("C"), py::arg("scales") = py::none(),
        py::arg("bias") = py::none(), py::arg("residual") = py::none(), py::arg("act") = "none", py::arg("layout") = "nk",
        py::arg("C2") = py::none(), py::arg("C3") = py::none(),
        "C = act(x . W^T * scales + bias) + residual in one kernel (fp32 until the final rounding); act='silu_gate': "
        "C[M,N/2] = silu(x.Wgate^T) * (x.Wup^T) on a weight from prepack_gate_up; C2/C3: the output columns are split over "
        "C, C2, C3 (a fused QKV projection written into three tensors)");
  m.def("fastgemv_int4", &op_wfirst_int4, py::arg("W4"), py::arg("x"), py::arg("C"), py::arg("scales") = py::none(),
        py::arg("zero_point") = 8,
        "C[M,N] = sum_g scales[n,g] * sum_k x[m,k] * (w4[n,k] - zero_point): W4 [N,K/2] uint8, low nibble = even k");
  m.def("quantize_int4", &quantize_int4, py::arg("W"), py::arg("group_size") = 128,
        "W[N,K] fp16 -> (W4 [N,K/2] uint8, scales [N, K/group_size] fp16), zero point 8, for fastgemv_int4");
  m.def("quantize_int8", &quantize_int8, py::arg("W"),
        "W[N,K] fp16 -> (W8 int8, scales fp16): symmetric, one scale per output channel, for fastgemv_int8");
  m.def("launch_count", []() { return fg_launch_count(); });
  m.def("version", []() { return std::string(fg_version()); });
}
