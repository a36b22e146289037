// Shared-memory staging and element access helpers for the persistent work-list kernels.
#pragma once

#include "kaon_device.cuh"
#include "kaon_plan.h"

namespace kaon {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

// ---- mbarrier + 1-D bulk copy (TMA engine, no tensor map): global -> shared ----

__device__ __forceinline__ void mbar_init(uint64_t* bar, unsigned count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, unsigned bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

// dst, src 16-byte aligned; bytes a non-zero multiple of 16
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, unsigned bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
          smem_u32(dst)),
      "l"(src), "r"(bytes), "r"(smem_u32(bar))
      : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, unsigned parity) {
  unsigned ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait for a bulk copy; on timeout records `code` and returns false.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, unsigned parity, unsigned* status,
                                          unsigned code) {
  for (unsigned i = 0; i < (1u << 22); ++i)
    if (mbar_try_wait(bar, parity)) return true;
  atomicCAS(status, 0u, code);
  return false;
}

// Orders this thread's earlier generic-proxy accesses to shared memory before later async-proxy
// (bulk copy) writes to it.
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Copy `bytes` from global to shared.  Source 16-byte aligned: the 16-byte-multiple head goes through
// the bulk engine (the caller's thread 0 issues it; completion lands on the barrier) and the tail of
// < 16 bytes is copied with plain loads.  Source only 8-byte aligned (a run of int8 / bf16 momentum that
// starts on an odd 8-element group): everything is copied with plain 8-byte loads.  Call with all
// threads; returns the bytes the bulk engine must move (0 if none).
__device__ __forceinline__ unsigned stage_tail(unsigned char* dst, const unsigned char* src,
                                               unsigned bytes, int tid) {
  if (reinterpret_cast<uintptr_t>(src) & 15) {
    const unsigned words = bytes >> 3;
    for (unsigned i = tid; i < words; i += blockDim.x)
      reinterpret_cast<uint2*>(dst)[i] = reinterpret_cast<const uint2*>(src)[i];
    const unsigned done = words << 3;
    if ((unsigned)tid < bytes - done) dst[done + tid] = src[done + tid];
    return 0u;
  }
  unsigned head = bytes & ~15u;
  unsigned tail = bytes - head;
  if ((unsigned)tid < tail) dst[head + tid] = src[head + tid];
  return head;
}

// ---- eight consecutive elements as fp32 ----

template <typename PT>
struct Elems;

template <>
struct Elems<__nv_bfloat16> {
  static constexpr int BYTES = 2;
  static constexpr bool IS_BF16 = true;
  __device__ static __forceinline__ void load8(const void* base, float out[8]) {
    uint4 v = *reinterpret_cast<const uint4*>(base);
    out[0] = bf16lo(v.x); out[1] = bf16hi(v.x); out[2] = bf16lo(v.y); out[3] = bf16hi(v.y);
    out[4] = bf16lo(v.z); out[5] = bf16hi(v.z); out[6] = bf16lo(v.w); out[7] = bf16hi(v.w);
  }
  __device__ static __forceinline__ float load1(const void* base, int i) {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(base)[i]);
  }
};

template <>
struct Elems<float> {
  static constexpr int BYTES = 4;
  static constexpr bool IS_BF16 = false;
  __device__ static __forceinline__ void load8(const void* base, float out[8]) {
    float4 a = reinterpret_cast<const float4*>(base)[0];
    float4 b = reinterpret_cast<const float4*>(base)[1];
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
    out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  }
  __device__ static __forceinline__ float load1(const void* base, int i) {
    return reinterpret_cast<const float*>(base)[i];
  }
};

// cnt valid elements (1..8); the rest read as zero
template <typename PT>
__device__ __forceinline__ void load8_guard(const void* base, int cnt, float out[8]) {
  if (cnt >= 8) {
    Elems<PT>::load8(base, out);
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) out[k] = (k < cnt) ? Elems<PT>::load1(base, k) : 0.0f;
  }
}

// ---- work claiming ----

// Persistent-CTA claim of the next work item.  Thread 0 fetches; everyone reads it after the barrier
// the caller places.
__device__ __forceinline__ void claim(unsigned* counter, int* slot, int tid) {
  if (tid == 0) *slot = (int)atomicAdd(counter, 1u);
}

}  // namespace kaon
