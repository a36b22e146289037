// Per-element building blocks of the flat-item kernels (AdaPNM, KProdigy): eight consecutive elements per
// thread and trip, scalar fp32 arithmetic, every codec.
#pragma once

#include <cuda_bf16.h>

#include "kaon_device.cuh"
#include "kaon_ops.cuh"

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
    float* dst = reinterpret_cast<float*>(pos) + e;
    for (int k = 0; k < cnt; ++k) dst[k] = tr.mp[k];
  } else if constexpr (MK == KAON_M_BF16) {
    uint16_t* dst = reinterpret_cast<uint16_t*>(pos) + e;
    for (int k = 0; k < cnt; ++k) dst[k] = (uint16_t)(pack_bf16_rn(tr.mp[k], 0.0f) & 0xffffu);
  } else if constexpr (MK == KAON_M_INT8) {
    signed char* dst = reinterpret_cast<signed char*>(pos) + e;
    for (int k = 0; k < cnt; ++k) {
      const float sc = __fdiv_rn(fmaxf(amax_of_row(tr.rw[k]), 1e-12f), 127.0f);
      dst[k] = (signed char)(int)fminf(fmaxf(rintf(__fdiv_rn(tr.mp[k], sc)), -127.0f), 127.0f);
      if ((tr.first >> k) & 1u) psc[tr.rw[k]] = sc;
    }
  } else {  // 4-bit
    float amax = 0.0f;
    for (int k = 0; k < cnt; ++k) amax = fmaxf(amax, fabsf(tr.mp[k]));
    const int lanes = bsh >= 31 ? 16 : (1 << (bsh - 3));  // threads that share a block
    for (int o = 1; o < lanes; o <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    // one block over a whole 1-D tensor: its absmax was taken by the caller's first sweep
    const bool whole = whole_amax >= 0.0f;
    if (whole) amax = whole_amax;
    const float sc = __fdiv_rn(fmaxf(amax, 1e-12f), 7.0f);
    unsigned q[8];
#pragma unroll
    for (int k = 0; k < 8; ++k)
      q[k] = k < cnt ? (unsigned)((int)fminf(fmaxf(rintf(__fdiv_rn(tr.mp[k], sc)), -7.0f), 7.0f) + 8) : 0u;
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
