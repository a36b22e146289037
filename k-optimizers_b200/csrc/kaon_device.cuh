// Device-side arithmetic shared by the kaon_b200 kernels (sm_100a).
//
// The arithmetic contract is that of the reference's torch fp32 ops: FMA only where torch's kernels
// contract (lerp, add(alpha)), true IEEE division, round-half-to-even.  The library is compiled with
// -fmad=false so that no other multiply-add is fused.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace kaon {

// ----------------------------------------------------------------------------- bf16 <-> fp32

__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// round-to-nearest-even fp32 pair -> packed bf16x2 (a in the low half)
__device__ __forceinline__ uint32_t pack_bf16_rn(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// fp32 -> nearest bf16 value, returned as fp32
__device__ __forceinline__ float round_bf16(float a) {
  return __bfloat162float(__float2bfloat16_rn(a));
}

// ----------------------------------------------------------------------------- torch-exact scalar ops

// x.lerp_(end, w): FMA forms, difference rounded first.
__device__ __forceinline__ float lerp_torch(float start, float end, float w, float w_minus_1,
                                            bool small_w) {
  float diff = __fsub_rn(end, start);
  return small_w ? __fmaf_rn(w, diff, start) : __fmaf_rn(w_minus_1, diff, end);
}

// 1/sqrtf(x) with both roundings, the CPU meaning of torch.rsqrt
__device__ __forceinline__ float rsqrt_torch(float x) { return __fdiv_rn(1.0f, __fsqrt_rn(x)); }

// rint(m / scale) computed with one multiply by inv = 1/scale when that is provably the same
// integer, and with the true IEEE division otherwise.  |m/scale| must stay below 2^21.
// The product m*inv is within 2 ulp of the rounded quotient; when it lies further than `margin`
// from a half-integer both round to the same integer.
__device__ __forceinline__ float quant_round(float m, float scale, float inv, float margin) {
  const float magic = 12582912.0f;  // 1.5 * 2^23: adding it rounds to integer, half to even
  float t = __fmul_rn(m, inv);
  float q = __fsub_rn(__fadd_rn(t, magic), magic);
  float frac = fabsf(__fsub_rn(t, q));
  if (frac > 0.5f - margin) {
    float x = __fdiv_rn(m, scale);
    q = __fsub_rn(__fadd_rn(x, magic), magic);
  }
  return q;
}

// ----------------------------------------------------------------------------- Philox4x32-7
// Round function and key schedule of Salmon et al. 2011; the stochastic-rounding stream runs seven
// rounds (the smallest count its authors report as passing BigCrush), as the CPU oracle does.
#define KAON_PHILOX_ROUNDS 7

struct Philox {
  uint32_t k0, k1;
  __device__ __forceinline__ void operator()(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                             uint32_t out[4]) const {
    uint32_t a = k0, b = k1;
#pragma unroll
    for (int r = 0; r < KAON_PHILOX_ROUNDS; ++r) {
      if (r) {
        a += 0x9E3779B9u;
        b += 0xBB67AE85u;
      }
      unsigned long long p0 = (unsigned long long)0xD2511F53u * c0;
      unsigned long long p1 = (unsigned long long)0xCD9E8D57u * c2;
      uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ a;
      uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ b;
      c1 = (uint32_t)p1;
      c3 = (uint32_t)p0;
      c0 = n0;
      c2 = n2;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
  }
};

// Noise for the eight elements 8q..8q+7 of tensor `tid` at `step`, write `tag`:
// counter = (q_lo, tid, step, tag | q_hi << 8); element k takes 16-bit lane k (low half first).
struct SrStream {
  Philox ph;
  uint32_t step, tag;
  __device__ __forceinline__ void draw8(uint32_t tid, uint64_t q, uint32_t out[4]) const {
    ph((uint32_t)q, tid, step, (tag & 0xffu) | ((uint32_t)(q >> 32) << 8), out);
  }
};

// fp32 result -> bf16 bits with 16-bit noise added below the kept mantissa
// (reference src/kaon/_stochastic_rounding.py:88-96)
__device__ __forceinline__ uint32_t sr_bits(float res, uint32_t noise16) {
  return (__float_as_uint(res) + noise16) >> 16;
}

// ----------------------------------------------------------------------------- weight write

// Eight consecutive weights: p += alpha*delta under the configured bf16 method.
//  PT = __nv_bfloat16: pw holds 4 packed words, updated in place.
//  none: rn_bf16(p + alpha * rn_bf16(delta)); SR: fma(delta, alpha, p) + noise, truncate.
template <bool SR>
__device__ __forceinline__ void write8_bf16(uint32_t pw[4], const float d[8], float alpha,
                                            const uint32_t noise[4]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    float p0 = bf16lo(pw[k]), p1 = bf16hi(pw[k]);
    if (SR) {
      float r0 = __fmaf_rn(d[2 * k], alpha, p0);
      float r1 = __fmaf_rn(d[2 * k + 1], alpha, p1);
      uint32_t b0 = sr_bits(r0, noise[k] & 0xffffu);
      uint32_t b1 = sr_bits(r1, noise[k] >> 16);
      pw[k] = (b0 & 0xffffu) | (b1 << 16);
    } else {
      float r0 = __fadd_rn(p0, __fmul_rn(alpha, round_bf16(d[2 * k])));
      float r1 = __fadd_rn(p1, __fmul_rn(alpha, round_bf16(d[2 * k + 1])));
      pw[k] = pack_bf16_rn(r0, r1);
    }
  }
}

// Kahan-compensated bf16 write, p -= d (reference src/kaon/_backend.py:89-94).  Every line of the
// reference is a bf16 tensor op, i.e. an fp32 operation whose result is rounded to bf16:
//   shift -= bf16(d);  p_before = p;  p += shift;  shift += (p_before - p)
// p and shift hold bf16 values in fp32 registers.
__device__ __forceinline__ void kahan_step(float& p, float& shift, float d) {
  const float s1 = round_bf16(__fsub_rn(shift, round_bf16(d)));
  const float pn = round_bf16(__fadd_rn(p, s1));
  shift = round_bf16(__fadd_rn(s1, round_bf16(__fsub_rn(p, pn))));
  p = pn;
}

// ----------------------------------------------------------------------------- warp helpers

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float group_max(float v, int width) {
  for (int o = width >> 1; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// True for a CTA that landed on one of the `reserve` multiprocessors with the highest ids: it should leave
// before claiming work (work is claimed from a counter, so the CTAs that stay do all of it).
__device__ __forceinline__ bool on_reserved_sm(unsigned reserve) {
  if (reserve == 0u) return false;
  unsigned smid, nsm;
  asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
  asm volatile("mov.u32 %0, %%nsmid;" : "=r"(nsm));
  return reserve * 2u <= nsm && smid + reserve >= nsm;
}

// ----------------------------------------------------------------------------- bounded wait

// Spin until *flag >= target or the limit runs out; on timeout records `code` in the status word.
// Returns false on timeout; callers skip their work and fall through to their normal exit.
#define KAON_SPIN_LIMIT (1u << 22)

__device__ __forceinline__ bool wait_counter(const unsigned int* flag, unsigned int target,
                                             unsigned int* status, unsigned int code,
                                             unsigned int limit = KAON_SPIN_LIMIT) {
  unsigned int spins = 0;
  while (true) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (v >= target) return true;
    if (++spins > limit) {
      atomicCAS(status, 0u, code);
      return false;
    }
    __nanosleep(64);
  }
}

__device__ __forceinline__ void signal_counter(unsigned int* flag, unsigned int add) {
  asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(flag), "r"(add) : "memory");
}

}  // namespace kaon
