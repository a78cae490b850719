// PTX wrappers and the shared-memory map used by the tensor-core decode kernel.
#pragma once

#include <cuda_fp16.h>

#include <cstdint>

namespace bkv {
namespace mma {

constexpr int kTile = 16;  // tokens of one tile: the M of the QK MMA and the K of the PV MMA

// ---- shared-memory map of a CTA that owns the SM ---------------------------------------
constexpr uint32_t kSmemBase = 0x400;              // dynamic shared memory starts after the 1 KB the system reserves
constexpr uint32_t kSmemEnd = kSmemBase + 232448;  // 227 KB opt-in maximum
constexpr uint32_t kLutAddr = 0x10000;  // table block P at kLutAddr + P*kLutBlock: address = block | byte << 8 | slot
constexpr uint32_t kLutBlock = 0x10000;
constexpr uint32_t kRingHi = kLutAddr + 2 * kLutBlock;

constexpr unsigned long long kWaitLimitNs = 2000000000ull;  // a wait that lasts 2 s gives up
constexpr float kRescaleThreshold = 8.f;                     // log2 units: p stays below 2^8

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ void bulk_copy_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
// true in exactly one lane of a converged warp; the compiler treats the guarded region as
// single-threaded, which is what the uniform-datapath bulk-copy instructions want
__device__ __forceinline__ bool elect_one_sync() {
  uint32_t pred;
  asm volatile(
      "{\n"
      ".reg .pred P;\n"
      "elect.sync _|P, 0xffffffff;\n"
      "selp.b32 %0, 1, 0, P;\n"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}
// 16-byte asynchronous copies (per thread, generic proxy), grouped per tile
__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait_group() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ unsigned long long global_timer_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait bookkeeping: true once kWaitLimitNs have passed since the first failed
// poll (the clock is only read every 256 polls).
struct WaitBudget {
  uint32_t polls = 0;
  unsigned long long start = 0;
  __device__ __forceinline__ bool expired() {
    if ((++polls & 255u) != 0) return false;
    const unsigned long long now = global_timer_ns();
    if (start == 0) {
      start = now;
      return false;
    }
    return now - start > kWaitLimitNs;
  }
};
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mma16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma16816_zero(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                              uint32_t b0, uint32_t b1) {  // c = a*b (no accumulator input)
  asm("{\n"
      ".reg .f32 z;\n"
      "mov.f32 z, 0f00000000;\n"
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {z,z,z,z};\n"
      "}\n"
      : "=f"(c[0]), "=f"(c[1]), "=f"(c[2]), "=f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ float fast_exp2(float x) {  // ex2.approx: 2 ulp, exp2(-inf) = 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  uint32_t r;
  asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
  return r;
}
__device__ __forceinline__ uint32_t hfma2_u32(uint32_t a, uint32_t b, uint32_t c) {  // a*b + c, rounded once
  uint32_t r;
  asm("fma.rn.f16x2 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
  return r;
}
// Makes a value opaque to the optimiser at this point: it is neither recomputed from its
// definition later nor folded into the expressions that use it; it simply lives in a register.
__device__ __forceinline__ void keep_in_register(uint32_t& v) { asm volatile("" : "+r"(v)); }
// Table look-up: the address is complete, no base is added.  Not volatile: the table is
// constant once built, so the compiler may schedule these freely.
__device__ __forceinline__ uint32_t lut_load(uint32_t addr) {
  uint32_t v;
  asm("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
// Ring loads are volatile: they stay, in program order, between the full-barrier wait of
// their tile and the bulk copies that later refill the same ring stage.
template <int IMM>
__device__ __forceinline__ uint4 ring_load128i(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4+%5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr), "n"(IMM));
  return v;
}
template <int IMM>
__device__ __forceinline__ uint2 ring_load64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.b32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(IMM));
  return v;
}
template <int IMM>
__device__ __forceinline__ uint32_t ring_load32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.b32 %0, [%1+%2];" : "=r"(v) : "r"(addr), "n"(IMM));
  return v;
}
template <bool BF16>
__device__ __forceinline__ float2 stat_word_to_f32(uint32_t w) {  // (scale, minimum)
  if (BF16) return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
  return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

// registers a thread may use when one CTA of NW warps owns the SM: the register file is
// split over the four schedulers (16 K registers each) and a CTA's warps are dealt to them
// round-robin
constexpr int max_regs_for(int nw) {
  const int per_thread = 16384 / (((nw + 3) / 4) * 32) / 8 * 8;
  return per_thread > 255 ? 255 : per_thread;
}

}  // namespace mma
}  // namespace bkv
