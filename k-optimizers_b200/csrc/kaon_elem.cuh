// Per-element building blocks of the flat-item kernels (AdaPNM, KProdigy): eight consecutive elements per
// thread and trip, scalar fp32 arithmetic, every codec.
#pragma once

#include <cuda_bf16.h>

#include "kaon_device.cuh"
#include "kaon_ops.cuh"
#include "kaon_packed.cuh"

namespace kaon {

template <typename PT>
__device__ __forceinline__ float pnm_centered(float g, float mu, bool gc) {
  if (!gc) return g;
  const float x = __fsub_rn(g, mu);
  return Elems<PT>::IS_BF16 ? round_bf16(x) : x;
}

template <int MK>
__device__ __forceinline__ float pnm_decode(const void* m, const float* sc, long long i, int row, int bsh) {
  if constexpr (MK == KAON_M_4BIT) {
    const unsigned byte = reinterpret_cast<const unsigned char*>(m)[i >> 1];
    const int nib = (i & 1) ? (byte >> 4) & 0xF : byte & 0xF;
    return __fmul_rn((float)(nib - 8), sc[bsh >= 31 ? 0 : (i >> bsh)]);
  } else if constexpr (MK == KAON_M_INT8) {
    return __fmul_rn((float)reinterpret_cast<const signed char*>(m)[i], sc[row]);
  } else if constexpr (MK == KAON_M_BF16) {
    return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(m)[i]);
  } else {
    return reinterpret_cast<const float*>(m)[i];
  }
}

// x / d for a divisor shared by many elements: rcp = RN(1/d) once, then one Newton step on the residual
// gives the correctly rounded quotient for normal-range operands.
__device__ __forceinline__ float div_by(float x, float d, float rcp) {
  const float q0 = __fmul_rn(x, rcp);
  const float r = __fmaf_rn(-q0, d, x);
  return __fmaf_rn(r, rcp, q0);
}

// Eight consecutive floats at p (a multiple of eight elements into its array): two 16-byte accesses when the
// address allows, element by element otherwise and at a ragged end.
__device__ __forceinline__ void ld8f(const float* p, int cnt, float o[8]) {
  if (cnt >= 8 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = k < cnt ? p[k] : 0.0f;
  }
}
__device__ __forceinline__ void st8f(float* p, int cnt, const float o[8]) {
  if (cnt >= 8 && (reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    reinterpret_cast<float4*>(p)[0] = make_float4(o[0], o[1], o[2], o[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(o[4], o[5], o[6], o[7]);
  } else {
#pragma unroll
    for (int k = 0; k < 8; ++k) if (k < cnt) p[k] = o[k];
  }
}

// The stored momentum of elements e .. e+7 (e a multiple of eight; the buffer 16-byte aligned): one vector
// load for a full trip.  rw[k] is each element's row (the int8 scale index).
template <int MK>
__device__ __forceinline__ void pnm_decode8(const void* m, const float* sc, long long e, int cnt, const int rw[8],
                                            int bsh, float o[8]) {
  if (cnt >= 8) {
    if constexpr (MK == KAON_M_4BIT) {
      const uint32_t w = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const unsigned char*>(m) + (e >> 1));
      const float s = sc[bsh >= 31 ? 0 : (e >> bsh)];   // blocks hold at least 32 elements: one scale per trip
      // nibble n -> the float 2^23 + n by a byte permute into the mantissa of 0x4B000000, less 2^23 + 8: the
      // exact integer n - 8 without a conversion; pairs go through the packed adder and multiplier
      const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
      const f32x2 OFF = pack2(-8388616.0f, -8388616.0f), S2 = pack2(s, s);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const f32x2 v = pack2(__uint_as_float(__byte_perm(lo, 0x4B000000u, 0x7540u + j)),
                              __uint_as_float(__byte_perm(hi, 0x4B000000u, 0x7540u + j)));
        const f32x2 r = mul2(add2(v, OFF), S2);
        o[2 * j] = r.x; o[2 * j + 1] = r.y;
      }
      return;
    } else if constexpr (MK == KAON_M_INT8) {
      const uint2 w = *reinterpret_cast<const uint2*>(reinterpret_cast<const signed char*>(m) + e);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const uint32_t word = k < 4 ? w.x : w.y;
        o[k] = __fmul_rn((float)(signed char)((word >> (8 * (k & 3))) & 0xffu), sc[rw[k]]);
      }
      return;
    } else if constexpr (MK == KAON_M_BF16) {
      const uint4 w = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(m) + e);
      o[0] = bf16lo(w.x); o[1] = bf16hi(w.x); o[2] = bf16lo(w.y); o[3] = bf16hi(w.y);
      o[4] = bf16lo(w.z); o[5] = bf16hi(w.z); o[6] = bf16lo(w.w); o[7] = bf16hi(w.w);
      return;
    } else if constexpr (MK == KAON_M_F32) {
      ld8f(reinterpret_cast<const float*>(m) + e, 8, o);
      return;
    }
  }
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    o[k] = 0.0f;
    if constexpr (MK != KAON_M_NONE) {
      if (k < cnt) o[k] = pnm_decode<MK>(m, sc, e + k, rw[k], bsh);
    }
  }
}

// One weight write on a register value: bf16 weights take stochastic rounding with `noise16` or the
// nearest-even of pv - bf16(d); fp32 weights a plain subtraction.
template <typename PT>
__device__ __forceinline__ float write_step_pnm(float pv, float d, bool sr, uint32_t noise16) {
  if constexpr (Elems<PT>::IS_BF16) {
    if (sr) return __uint_as_float((__float_as_uint(__fmaf_rn(d, -1.0f, pv)) + noise16) & 0xFFFF0000u);
    return round_bf16(__fsub_rn(pv, round_bf16(d)));
  } else {
    return __fmaf_rn(d, -1.0f, pv);
  }
}

__device__ __forceinline__ uint32_t noise_lane_pnm(const uint32_t nz[4], int k) {
  return (k & 1) ? (nz[k >> 1] >> 16) : (nz[k >> 1] & 0xffffu);
}

// Everything a thread needs about the eight consecutive elements it handles in one trip.
struct PnmTrip {
  float y[8];    // (centralised) gradient
  float mp[8];   // new positive momentum, fp32, before requantisation
  float u[8];    // pn * 1/sqrt(v_hat), before the clip
  int rw[8];     // row of each element (0 for 1-D)
  unsigned first;  // bit k: element k is the first of its row
};

// Store the new positive momentum of one trip through its codec.  4-bit: the 16 lanes that share a
// 128-element block take its absmax together, so every lane of the warp must call this (cnt == 0 for a
// lane with nothing).  int8: `amax_bits_of_row` gives the finished absmax of an element's row (factored)
// or of the tensor (1-D).
template <int MK, typename RowMax>
__device__ __forceinline__ void pnm_store_m(void* pos, float* psc, const PnmTrip& tr, long long e, int cnt, int bsh,
                                            int lane, RowMax amax_of_row, float whole_amax = -1.0f) {
  if constexpr (MK == KAON_M_F32) {
    st8f(reinterpret_cast<float*>(pos) + e, cnt, tr.mp);
  } else if constexpr (MK == KAON_M_BF16) {
    uint16_t* dst = reinterpret_cast<uint16_t*>(pos) + e;
    if (cnt >= 8) {
      *reinterpret_cast<uint4*>(dst) = make_uint4(pack_bf16_rn(tr.mp[0], tr.mp[1]), pack_bf16_rn(tr.mp[2], tr.mp[3]),
                                                 pack_bf16_rn(tr.mp[4], tr.mp[5]), pack_bf16_rn(tr.mp[6], tr.mp[7]));
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) if (k < cnt) dst[k] = (uint16_t)(pack_bf16_rn(tr.mp[k], 0.0f) & 0xffffu);
    }
  } else if constexpr (MK == KAON_M_INT8) {
    signed char* dst = reinterpret_cast<signed char*>(pos) + e;
    uint32_t w0 = 0u, w1 = 0u;
    int rp = -1;
    float sc = 1.0f, rsc = 1.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (k >= cnt) continue;
      if (tr.rw[k] != rp) { rp = tr.rw[k]; sc = __fdiv_rn(fmaxf(amax_of_row(rp), 1e-12f), 127.0f); rsc = __frcp_rn(sc); }
      const int q = (int)fminf(fmaxf(rintf(div_by(tr.mp[k], sc, rsc)), -127.0f), 127.0f);
      if (k < 4) w0 |= (uint32_t)(q & 0xff) << (8 * k); else w1 |= (uint32_t)(q & 0xff) << (8 * (k - 4));
      if ((tr.first >> k) & 1u) psc[rp] = sc;
    }
    if (cnt >= 8) *reinterpret_cast<uint2*>(dst) = make_uint2(w0, w1);
    else
#pragma unroll
      for (int k = 0; k < 8; ++k) if (k < cnt) dst[k] = (signed char)((k < 4 ? w0 >> (8 * k) : w1 >> (8 * (k - 4))) & 0xffu);
  } else {  // 4-bit
    float amax = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) if (k < cnt) amax = fmaxf(amax, fabsf(tr.mp[k]));
    const int lanes = bsh >= 31 ? 16 : (1 << (bsh - 3));  // threads that share a block
    for (int o = 1; o < lanes; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    // one block over a whole 1-D tensor: its absmax was taken by the caller's first sweep
    const bool whole = whole_amax >= 0.0f;
    if (whole) amax = whole_amax;
    const float sc = __fdiv_rn(fmaxf(amax, 1e-12f), 7.0f);
    const float rsc = __frcp_rn(sc);
    unsigned q[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      q[k] = k < cnt ? (unsigned)((int)fminf(fmaxf(rintf(div_by(tr.mp[k], sc, rsc)), -7.0f), 7.0f) + 8) : 0u;
    unsigned char* dst = reinterpret_cast<unsigned char*>(pos) + (e >> 1);
    if (cnt >= 8) {
      *reinterpret_cast<uint32_t*>(dst) = q[0] | (q[1] << 4) | (q[2] << 8) | (q[3] << 12) | (q[4] << 16) | (q[5] << 20) |
                                          (q[6] << 24) | (q[7] << 28);
    } else {
      for (int b = 0; 2 * b < cnt; ++b) dst[b] = (unsigned char)(q[2 * b] | (q[2 * b + 1] << 4));
    }
    __syncwarp();  // every lane of the block has decoded with the old scale
    if (!whole && (lane & (lanes - 1)) == 0 && cnt > 0) psc[bsh >= 31 ? 0 : (e >> bsh)] = sc;
  }
}

}  // namespace kaon
