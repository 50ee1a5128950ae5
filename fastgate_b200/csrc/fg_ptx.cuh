// Thin inline-PTX wrappers for sm_100a: mbarrier, bulk-tensor (TMA) loads without
// cluster multicast, ldmatrix, mma.sync and cache-policy helpers.
#pragma once
#include <cuda_fp16.h>
#include <stdint.h>

namespace fg {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t dynamic_smem_size() {
  uint32_t v;
  asm volatile("mov.u32 %0, %%dynamic_smem_size;" : "=r"(v));
  return v;
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Non-blocking probe of a phase (try_wait may suspend the thread for a while before it says no).
__device__ __forceinline__ uint32_t mbar_test_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Multicast ("multimem") store / reduction: one instruction, delivered by the NVSwitch to the
// copy of the address in every GPU of the multicast group.
__device__ __forceinline__ void multimem_st_b32(void* mc_ptr, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.b32 [%0], %1;" ::"l"(mc_ptr), "r"(v) : "memory");
}
// Eight fp16 values (16 bytes, 16-byte aligned) as one multicast store.
__device__ __forceinline__ void multimem_st_v4_f16x2(void* mc_ptr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc_ptr), "r"(a), "r"(b), "r"(c), "r"(d)
               : "memory");
}
// Four fp16 values (8 bytes, 8-byte aligned) as one multicast store.
__device__ __forceinline__ void multimem_st_v2_f16x2(void* mc_ptr, uint32_t a, uint32_t b) {
  asm volatile("multimem.st.relaxed.sys.global.v2.f16x2 [%0], {%1,%2};" ::"l"(mc_ptr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ void multimem_red_release_add_u64(unsigned long long* mc_ptr, unsigned long long v) {
  asm volatile("multimem.red.release.sys.global.add.u64 [%0], %1;" ::"l"(mc_ptr), "l"(v) : "memory");
}
// Release/acquire fence at GPU scope (__threadfence() is the sequentially consistent one).
__device__ __forceinline__ void fence_acq_rel_gpu() { asm volatile("fence.acq_rel.gpu;" ::: "memory"); }
// The same at system scope (other GPUs).  Cumulative: it also orders what other threads of the CTA
// wrote before a barrier this thread has passed.
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ uint32_t smid() {
  uint32_t v;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(v));
  return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: gives up after ~budget_ns of wall time and returns false.  Every
// wait in the library goes through here, so no kernel can spin forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  unsigned long long budget_ns) {
  if (mbar_try_wait(bar, parity)) return true;
  unsigned long long t0 = 0;
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 0x3ffu) == 0) {
      unsigned long long now = globaltimer_ns();
      if (t0 == 0) t0 = now;
      else if (now - t0 > budget_ns) return false;
    }
  }
  return true;
}

// ---- L2 cache policies --------------------------------------------------------
__device__ __forceinline__ uint64_t policy_evict_first() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ uint64_t policy_evict_last() {
  uint64_t p;
  asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}

// ---- TMA: 2-D tiled bulk tensor load, this CTA's shared memory only ------------
// c0 is the innermost coordinate; c0 * element size must be a multiple of 16 bytes.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, uint32_t bar, int c0,
                                            int c1, uint64_t policy) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
      " [%0], [%1, {%3, %4}], [%2], %5;" ::"r"(dst),
      "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "l"(policy)
      : "memory");
}
// Ask for one box of a tensor map to be brought into L2 (no shared-memory destination, no barrier).
__device__ __forceinline__ void tma_prefetch_l2_2d(const void* tmap, int x, int y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global.tile [%0, {%1, %2}];" ::"l"(tmap), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}

// ---- ldmatrix / mma.sync --------------------------------------------------------
__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                        uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1,
                                              uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void lds_v2(uint32_t addr, uint32_t& r0, uint32_t& r1) {
  asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(r0), "=r"(r1) : "r"(addr));
}
// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Programmatic dependent launch (no-ops when the kernel was launched without the attribute).
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void griddep_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Four signed bytes -> two half2 registers, exact.  XOR 0x80 makes each byte b+128;
// placing it under the exponent byte 0x64 gives the half 1024 + (b+128); subtracting
// 1152 leaves b.  lo holds bytes 0,1 and hi holds bytes 2,3.
__device__ __forceinline__ void dequant_s8x4(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t u = w ^ 0x80808080u;
  uint32_t l, h;
  asm("prmt.b32 %0, %1, %2, 0x5140;" : "=r"(l) : "r"(u), "r"(0x64646464u));
  asm("prmt.b32 %0, %1, %2, 0x5342;" : "=r"(h) : "r"(u), "r"(0x64646464u));
  const uint32_t bias = 0x64806480u;  // half2(1152, 1152)
  asm("sub.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(l), "r"(bias));
  asm("sub.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(h), "r"(bias));
}

// Eight unsigned 4-bit weights of one 32-bit word (nibble i = element i) to four half2, minus the
// zero point: nibbles (0,4), (1,5), (2,6), (3,7).  A nibble placed under the exponent pattern
// 0x6400 is the half 1024 + nibble; `magic` is half2(1024 + zero_point), so one subtraction
// leaves nibble - zero_point exactly (integers well inside the half's 11 significand bits).
__device__ __forceinline__ void dequant_u4x8(uint32_t w, uint32_t magic, uint32_t (&out)[4]) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t v;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(v) : "r"(w >> (4 * i)), "r"(0x000F000Fu), "r"(0x64006400u));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(out[i]) : "r"(v), "r"(magic));
  }
}
__device__ __forceinline__ void lds_v4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}

}  // namespace fg
