// Per-eight-element building blocks shared by the optimizer kernels: row lookup, weight write,
// momentum decode.
#pragma once

#include "kaon_stage.cuh"

namespace kaon {

__device__ __forceinline__ int row_of(unsigned e, const DevTensor& d) {
  if (d.rows <= 0) return 0;
  return d.cols == 1 ? (int)e : (int)__umulhi(e, d.row_magic);
}

// ---- mirrors of the weight buffer on other GPUs (plain peer stores) ----

// 16 bytes this thread just stored at `local`, repeated at every mirror.
// (pr == nullptr: no mirrors; a null constant compiles the stores out)
__device__ __forceinline__ void mirror16(const Peers* pr, void* local, uint4 v) {
  if (pr == nullptr) return;
  for (int r = 0; r < pr->n; ++r)
    *reinterpret_cast<uint4*>(reinterpret_cast<unsigned char*>(local) + pr->delta[r]) = v;
}

// `bytes` (a multiple of 2) this thread just stored at `local`, copied to every mirror; for the
// ragged ends, where the value is not at hand as a vector.
__device__ __forceinline__ void mirror_copy(const Peers* pr, const void* local, int bytes) {
  if (pr == nullptr || pr->n == 0) return;
  const unsigned short* src = reinterpret_cast<const unsigned short*>(local);
  for (int r = 0; r < pr->n; ++r) {
    unsigned short* dst = reinterpret_cast<unsigned short*>(
        reinterpret_cast<unsigned char*>(const_cast<void*>(local)) + pr->delta[r]);
    for (int k = 0; k < (bytes >> 1); ++k) dst[k] = src[k];
  }
}

// p[0..cnt) += alpha * dlt[0..cnt) with the configured rounding; `q` is the global index of this
// group of eight (element / 8), which keys the noise.
template <typename PT>
__device__ __forceinline__ void update8(void* pe, int cnt, const float dlt[8], float alpha, bool sr,
                                        const SrStream& st, uint32_t tensor_id, uint64_t q,
                                        const Peers* pr, void* she = nullptr) {
  if constexpr (Elems<PT>::IS_BF16) {
    if (she != nullptr) {  // Kahan: p -= dlt with the compensation buffer (alpha is -1 on this path)
      float pv[8], sh[8];
      load8_guard<__nv_bfloat16>(pe, cnt, pv);
      load8_guard<__nv_bfloat16>(she, cnt, sh);
#pragma unroll
      for (int k = 0; k < 8; ++k) kahan_step(pv[k], sh[k], dlt[k]);
      if (cnt >= 8) {
        const uint4 out = make_uint4(pack_bf16_rn(pv[0], pv[1]), pack_bf16_rn(pv[2], pv[3]),
                                     pack_bf16_rn(pv[4], pv[5]), pack_bf16_rn(pv[6], pv[7]));
        *reinterpret_cast<uint4*>(pe) = out;
        mirror16(pr, pe, out);
        *reinterpret_cast<uint4*>(she) = make_uint4(pack_bf16_rn(sh[0], sh[1]), pack_bf16_rn(sh[2], sh[3]),
                                                    pack_bf16_rn(sh[4], sh[5]), pack_bf16_rn(sh[6], sh[7]));
      } else {
        for (int k = 0; k < cnt; ++k) {
          reinterpret_cast<uint16_t*>(pe)[k] = (uint16_t)(__float_as_uint(pv[k]) >> 16);
          reinterpret_cast<uint16_t*>(she)[k] = (uint16_t)(__float_as_uint(sh[k]) >> 16);
        }
        mirror_copy(pr, pe, cnt * 2);
      }
      return;
    }
    uint32_t noise[4] = {0u, 0u, 0u, 0u};
    if (sr) st.draw8(tensor_id, q, noise);
    if (cnt >= 8) {
      uint4 v = *reinterpret_cast<uint4*>(pe);
      uint32_t pw[4] = {v.x, v.y, v.z, v.w};
      if (sr) write8_bf16<true>(pw, dlt, alpha, noise);
      else write8_bf16<false>(pw, dlt, alpha, noise);
      const uint4 out = make_uint4(pw[0], pw[1], pw[2], pw[3]);
      *reinterpret_cast<uint4*>(pe) = out;
      mirror16(pr, pe, out);
    } else {
      uint16_t* ph = reinterpret_cast<uint16_t*>(pe);
      for (int k = 0; k < cnt; ++k) {
        float pv = __uint_as_float((uint32_t)ph[k] << 16);
        uint32_t nz = (k & 1) ? (noise[k >> 1] >> 16) : (noise[k >> 1] & 0xffffu);
        if (sr) {
          ph[k] = (uint16_t)sr_bits(__fmaf_rn(dlt[k], alpha, pv), nz);
        } else {
          float r = __fadd_rn(pv, __fmul_rn(alpha, round_bf16(dlt[k])));
          ph[k] = (uint16_t)(pack_bf16_rn(r, 0.0f) & 0xffffu);
        }
      }
      mirror_copy(pr, pe, cnt * 2);
    }
  } else {
    float* pf = reinterpret_cast<float*>(pe);
    if (cnt >= 8) {
      float4 a = reinterpret_cast<float4*>(pf)[0], b = reinterpret_cast<float4*>(pf)[1];
      a.x = __fmaf_rn(dlt[0], alpha, a.x); a.y = __fmaf_rn(dlt[1], alpha, a.y);
      a.z = __fmaf_rn(dlt[2], alpha, a.z); a.w = __fmaf_rn(dlt[3], alpha, a.w);
      b.x = __fmaf_rn(dlt[4], alpha, b.x); b.y = __fmaf_rn(dlt[5], alpha, b.y);
      b.z = __fmaf_rn(dlt[6], alpha, b.z); b.w = __fmaf_rn(dlt[7], alpha, b.w);
      reinterpret_cast<float4*>(pf)[0] = a;
      reinterpret_cast<float4*>(pf)[1] = b;
      mirror16(pr, pf, make_uint4(__float_as_uint(a.x), __float_as_uint(a.y), __float_as_uint(a.z), __float_as_uint(a.w)));
      mirror16(pr, pf + 4, make_uint4(__float_as_uint(b.x), __float_as_uint(b.y), __float_as_uint(b.z), __float_as_uint(b.w)));
    } else {
      for (int k = 0; k < cnt; ++k) pf[k] = __fmaf_rn(dlt[k], alpha, pf[k]);
      mirror_copy(pr, pf, cnt * 4);
    }
  }
}

// Decode eight momentum values of the staged chunk (vector v of the work item).
template <int MK>
__device__ __forceinline__ void decode8(const unsigned char* m_s, int v, int cnt, float scale,
                                        float m[8]) {
  if constexpr (MK == KAON_M_4BIT) {
    uint32_t w = reinterpret_cast<const uint32_t*>(m_s)[v];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      // (nibble - 8) as fp32 without an int->float conversion: 2^23 + nibble, minus 2^23 + 8
      float f = __uint_as_float(0x4B000000u | ((w >> (4 * k)) & 0xFu)) - 8388616.0f;
      m[k] = (k < cnt) ? __fmul_rn(f, scale) : 0.0f;
    }
  } else if constexpr (MK == KAON_M_INT8) {
    uint2 w = reinterpret_cast<const uint2*>(m_s)[v];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      uint32_t word = k < 4 ? w.x : w.y;
      int c = (int)(signed char)((word >> (8 * (k & 3))) & 0xFFu);
      m[k] = (k < cnt) ? __fmul_rn((float)c, scale) : 0.0f;
    }
  } else if constexpr (MK == KAON_M_BF16) {
    load8_guard<__nv_bfloat16>(m_s + (size_t)v * 16, cnt, m);
  } else {
    load8_guard<float>(m_s + (size_t)v * 32, cnt, m);
  }
}

}  // namespace kaon
