// SPDX-License-Identifier: Apache-2.0
/**
 * @file  pipeline.cuh
 * @brief Device primitives shared by the streaming kernels: mbarriers with
 *        bounded waits, bulk copies into shared memory, explicit shared-space
 *        accesses by 32-bit address.
 *
 * Every wait on another agent (a bulk copy, another warp, the tensor pipe) goes
 * through mbar_wait_bounded: a fixed number of polls, after which the caller's
 * abort flag and the translation unit's status word are raised and the wait
 * returns false, so a lost signal ends the kernel instead of hanging the GPU.
 */
#pragma once

#include "common.cuh"

namespace nntr {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\t"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok)
               : "r"(bar), "r"(parity)
               : "memory");
  return ok != 0;
}
/** try_wait that lets the hardware park the thread for up to `ns` nanoseconds per try */
__device__ __forceinline__ bool mbar_try_wait_hint(uint32_t bar, uint32_t parity, uint32_t ns) {
  uint32_t ok;
  asm volatile("{\n\t.reg .pred p;\n\t"
               "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
               "selp.u32 %0, 1, 0, p;\n\t}"
               : "=r"(ok)
               : "r"(bar), "r"(parity), "r"(ns)
               : "memory");
  return ok != 0;
}

/** Bounded wait for the phase with `parity` of an mbarrier. After `spin` polls it also watches the CTA's abort flag and
 *  backs off. False when the CTA is aborting, or (after `polls` polls) when the phase never completed: then the abort
 *  flag and *status are raised. hint_ns != 0 uses the parked form of try_wait. */
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status,
                                                  uint32_t polls, uint32_t spin, uint32_t hint_ns = 0) {
  for (uint32_t it = 0; it < polls; ++it) {
    if (hint_ns ? mbar_try_wait_hint(bar, parity, hint_ns) : mbar_try_wait(bar, parity))
      return true;
    if (it > spin) {
      if (*abort_flag)
        return false;
      __nanosleep(32);
    }
  }
  *abort_flag = 1;
  atomicExch(status, NNTR_CUDA_ERR_TIMEOUT);
  return false;
}

/** Bulk copy global -> shared memory of this CTA, completion counted in bytes on an mbarrier. Both addresses 16-byte
 *  aligned, size a multiple of 16. Local memory only (no multicast). */
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

/** 4-way dot product of unsigned bytes (a) with signed bytes (b), accumulated in c */
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
  int d;
  asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
  return d;
}

/* explicit shared-space accesses by 32-bit address */
__device__ __forceinline__ uint32_t lds32(uint32_t a) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(a));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t a) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(a));
  return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t a) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(a));
  return v;
}
__device__ __forceinline__ void sts32(uint32_t a, uint32_t v) {
  asm volatile("st.shared.u32 [%0], %1;" ::"r"(a), "r"(v) : "memory");
}
__device__ __forceinline__ void sts64(uint32_t a, uint32_t v0, uint32_t v1) {
  asm volatile("st.shared.v2.u32 [%0], {%1, %2};" ::"r"(a), "r"(v0), "r"(v1) : "memory");
}

} // namespace nntr
