// Shared device helpers for the sm_100a mixed-precision linear kernels:
// format decode (E2M1 / E4M3 -> f16 through the hardware converters), mbarrier
// and bulk-async-copy wrappers, ldmatrix / mma.sync wrappers, and the host
// side error plumbing of the C ABI.
#pragma once

#include <cstdint>
#include <cstdio>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include "../../include/rdq_b200.h"

namespace rdq {

// ---------------------------------------------------------------------------
// host side error plumbing
// ---------------------------------------------------------------------------
void set_error(const char *fmt, ...);

#define RDQ_REQUIRE(cond, code, ...)                 \
  do {                                               \
    if (!(cond)) {                                   \
      ::rdq::set_error(__VA_ARGS__);                 \
      return (code);                                 \
    }                                                \
  } while (0)

#define RDQ_CUDA(call)                                                     \
  do {                                                                     \
    cudaError_t e__ = (call);                                              \
    if (e__ != cudaSuccess) {                                              \
      ::rdq::set_error("%s failed: %s", #call, cudaGetErrorString(e__));   \
      return RDQ_E_CUDA;                                                   \
    }                                                                      \
  } while (0)

static inline bool aligned16(const void *p) {
  return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

int sm_count();  // multiprocessors of the current device (cached per device)

// ---------------------------------------------------------------------------
// format decode.  All conversions are exact: every E2M1 / E4M3 value is an
// f16 value.  E4M3 follows torch.float8_e4m3fn (subnormals mant * 2^-9, 0x7f /
// 0xff NaN, no inf), which is what the oracle uses
// (rdquant/core/formats.py:52-66).
// ---------------------------------------------------------------------------

// four packed bytes (8 E2M1 codes; low nibble = even k) -> four half2
// (k0,k1) (k2,k3) (k4,k5) (k6,k7)
__device__ __forceinline__ void cvt_e2m1x8(uint32_t w, uint32_t &h01, uint32_t &h23,
                                           uint32_t &h45, uint32_t &h67) {
  asm("{\n"
      ".reg .b8 b0, b1, b2, b3;\n"
      "mov.b32 {b0, b1, b2, b3}, %4;\n"
      "cvt.rn.f16x2.e2m1x2 %0, b0;\n"
      "cvt.rn.f16x2.e2m1x2 %1, b1;\n"
      "cvt.rn.f16x2.e2m1x2 %2, b2;\n"
      "cvt.rn.f16x2.e2m1x2 %3, b3;\n"
      "}\n"
      : "=r"(h01), "=r"(h23), "=r"(h45), "=r"(h67)
      : "r"(w));
}

// four E4M3 bytes -> two half2 (e0,e1) (e2,e3)
__device__ __forceinline__ void cvt_e4m3x4(uint32_t w, uint32_t &h01, uint32_t &h23) {
  asm("{\n"
      ".reg .b16 lo, hi;\n"
      "mov.b32 {lo, hi}, %2;\n"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n"
      "cvt.rn.f16x2.e4m3x2 %1, hi;\n"
      "}\n"
      : "=r"(h01), "=r"(h23)
      : "r"(w));
}

// two E4M3 bytes (low 16 bits of w) -> half2
__device__ __forceinline__ uint32_t cvt_e4m3x2(uint32_t w) {
  uint32_t out;
  asm("{\n"
      ".reg .b16 lo, hi;\n"
      "mov.b32 {lo, hi}, %1;\n"
      "cvt.rn.f16x2.e4m3x2 %0, lo;\n"
      "}\n"
      : "=r"(out)
      : "r"(w));
  return out;
}

__device__ __forceinline__ float e4m3_to_float(uint32_t byte) {
  uint32_t h2 = cvt_e4m3x2(byte & 0xffu);
  return __half2float(__ushort_as_half(static_cast<unsigned short>(h2 & 0xffffu)));
}

__device__ __forceinline__ uint32_t hmul2_u32(uint32_t a, uint32_t b) {
  __half2 r = __hmul2(*reinterpret_cast<__half2 *>(&a), *reinterpret_cast<__half2 *>(&b));
  return *reinterpret_cast<uint32_t *>(&r);
}

__device__ __forceinline__ float2 h2_to_f2(uint32_t h) {
  return __half22float2(*reinterpret_cast<__half2 *>(&h));
}

// ---------------------------------------------------------------------------
// mbarrier / bulk async copy (TMA, non-tensor form) / PDL
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_init_fence() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Has the barrier phase completed?  Returns at once.
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// One suspended wait on the barrier phase: the thread sleeps in hardware (it takes no
// issue slots from the working warps) until the phase completes or about `ns`
// nanoseconds have passed.
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile(
      "{\n.reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n"
      "selp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(ok)
      : "r"(bar), "r"(parity), "r"(ns)
      : "memory");
  return ok != 0;
}
// Bounded wait: gives up after `limit` suspended waits of up to 0.1 ms each (about a
// second) and reports false, so a lost copy or a logic error cannot hang the device.
// (Spinning on mbar_test before suspending was measured: the decode GEMV loses 8 % to the
// issue slots the spinning warps take from the working ones.)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit = 10000u) {
#pragma unroll 1
  for (uint32_t i = 0; i < limit; ++i) {
    if (mbar_try(bar, parity, 100000u)) return true;
  }
  return false;
}
// global -> shared bulk copy; src, dst 16-byte aligned, bytes % 16 == 0.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes,
                                         uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::
          "r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---------------------------------------------------------------------------
// warp matrix helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t &r0, uint32_t &r1,
                                            uint32_t &r2, uint32_t &r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                          uint32_t a3, uint32_t b0, uint32_t b1) {
  asm(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// A CTA without work stays resident for a few microseconds instead of returning at once.  The
// decode chain relies on every SM holding exactly one CTA of each launch: the CTAs of the GEMV
// after this kernel are placed, one per SM, into the slots the GEMV before it frees.  A CTA of
// this kernel that returned at the same moment would free a second slot on its SM, two CTAs of
// that GEMV would land there, run at half speed each, and the whole launch would wait for them
// (measured: 52 of 148 SMs doubled, +60 % on the following GEMVs).  After the linger all pending
// CTAs of that GEMV are placed and the freed slot goes to the launch after it.
__device__ __forceinline__ void linger(unsigned int ns) {
  unsigned long long t0, t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
  for (int i = 0; i < 64; ++i) {  // bounded: 64 naps of at most 0.25 us
    __nanosleep(250);
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    if (t - t0 > ns) break;
  }
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace rdq
