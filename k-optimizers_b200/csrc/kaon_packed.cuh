// Packed-pair arithmetic and bit-gather helpers shared by the fast paths of the step kernels (sm_100a).
#pragma once

#include "kaon_device.cuh"

namespace kaon {

// ---- packed fp32 pairs (f32x2 arithmetic of sm_100: each lane is an independent IEEE fp32 operation,
//      so results are those of the scalar instructions; two lanes cost one issue slot) ----
typedef float2 f32x2;
__device__ __forceinline__ f32x2 pack2(float lo, float hi) { return make_float2(lo, hi); }
__device__ __forceinline__ void unpack2(f32x2 v, float& lo, float& hi) { lo = v.x; hi = v.y; }
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) { return __ffma2_rn(a, b, c); }
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) { return __fmul2_rn(a, b); }
__device__ __forceinline__ f32x2 add2(f32x2 a, f32x2 b) { return __fadd2_rn(a, b); }
__device__ __forceinline__ f32x2 sub2(f32x2 a, f32x2 b) { return __fadd2_rn(a, make_float2(-b.x, -b.y)); }
// max / min of three (sm_100 takes three inputs in one instruction)
__device__ __forceinline__ float max3f(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float min3f(float a, float b, float c) {
  float d;
  asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Byte permute with the full selector: bit 3 of a selector nibble replicates the selected byte's top bit
// over the whole result byte (the __byte_perm intrinsic documents only the three index bits).
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t d;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(sel));
  return d;
}
// a - b on two packed bf16 values, one rounding to bf16 per lane.  Equal to bf16(fp32(a) - fp32(b)): the
// fp32 difference of two 8-bit significands is inexact only when one operand is below 2^-16 of the other,
// and then it lies nowhere near a bf16 rounding boundary.
__device__ __forceinline__ uint32_t sub_bf16x2(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("sub.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// maximum over the 16 lanes of this thread's half warp (every lane of the warp calls it; v >= 0, so
// the ordering of the bit patterns is that of the values): two whole-warp reductions, one per half
__device__ __forceinline__ float half_warp_max(float v, int tid) {
  const bool upper = (tid & 16) != 0;
  const uint32_t b = __float_as_uint(v);
  uint32_t lo, hi;
  asm volatile("redux.sync.max.u32 %0, %1, 0xffffffff;" : "=r"(lo) : "r"(upper ? 0u : b));
  asm volatile("redux.sync.max.u32 %0, %1, 0xffffffff;" : "=r"(hi) : "r"(upper ? b : 0u));
  return __uint_as_float(upper ? hi : lo);
}
// Stores to global memory through a generic pointer.  Volatile, so they keep their order among themselves
// and against fences and barriers; without a memory clobber, so the values the surrounding loop keeps in
// registers stay there.
__device__ __forceinline__ void stg_u32(void* p, uint32_t v) {
  asm volatile("st.global.u32 [%0], %1;" ::"l"(__cvta_generic_to_global(p)), "r"(v));
}
__device__ __forceinline__ void stg_u16(void* p, uint32_t v) {
  asm volatile("st.global.u16 [%0], %1;" ::"l"(__cvta_generic_to_global(p)), "h"((unsigned short)v));
}
__device__ __forceinline__ void stg_f32(void* p, float v) {
  asm volatile("st.global.f32 [%0], %1;" ::"l"(__cvta_generic_to_global(p)), "f"(v));
}
// a / 7 correctly rounded without the division unit: quotient estimate, exact residual, one correction.
// Equal to the IEEE quotient for every a in [1e-12, FNTHREADS_MAX] (checked exhaustively on the host).
__device__ __forceinline__ float div7_exact(float a) {
  const float r7 = 0.142857149243354797363281250f;  // RN(1/7)
  const float q0 = __fmul_rn(a, r7);
  return __fmaf_rn(__fmaf_rn(-7.0f, q0, a), r7, q0);
}


// a / 127 correctly rounded, as div7_exact (same exhaustive check)
__device__ __forceinline__ float div127_exact(float a) {
  const float r127 = 0.007874015718698501586914062500f;  // RN(1/127)
  const float q0 = __fmul_rn(a, r127);
  return __fmaf_rn(__fmaf_rn(-127.0f, q0, a), r127, q0);
}

}  // namespace kaon
