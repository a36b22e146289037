// Lion step for sm_100a: one persistent kernel walks the plan's work list.
//
// MAIN item (a run of whole rows, <= CAP elements): the gradient rows and the momentum bytes arrive in
// shared memory through the bulk-copy engine; row means (gradient centralization) are taken from
// shared memory; then per eight elements: decode momentum, direction sign(b1*m + (1-b1)*g), new
// momentum b2*m + (1-b2)*g, re-encode and store it, and - when cautious masking is on - store a
// 2-bit code per element (0 = masked out, 1/2/3 = update sign -1/0/+1) and add to the tensor's kept
// count.  APPLY item (same run, later in the list): once every MAIN item of the tensor has finished,
// turn the codes into the weight write with the tensor-wide rescale 1/max(kept/numel, 1e-8).
// Quantised momentum is read once and written once; weights are read once and written once.
#include <mutex>

#include "kaon_host.h"
#include "kaon_ops.cuh"

namespace kaon {

struct LionDev {
  float lr, b1, w1, b2, w2, wd;
  int cautious, gc, sr, has_wd;
  uint32_t step, k0, k1;
  uint32_t rk0[10], rk1[10];  // Philox round keys (k + r * Weyl), precomputed on the host
  int kahan;
};

// Philox4x32-10 with the round keys read from the kernel's parameter block.
__device__ __forceinline__ void philox_rk(const LionDev& hp, uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                          uint32_t out[4]) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const unsigned long long p0 = (unsigned long long)0xD2511F53u * c0;
    const unsigned long long p1 = (unsigned long long)0xCD9E8D57u * c2;
    const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ hp.rk0[r];
    const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ hp.rk1[r];
    c1 = (uint32_t)p1;
    c3 = (uint32_t)p0;
    c0 = n0;
    c2 = n2;
  }
  out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// Full-vector fast path of the MAIN item for 4-bit momentum, no weight decay, cautious on, rows that are
// a multiple of 8 elements: no per-element guards, the eight 4-bit codes assembled with one shift-add
// each, one exactness check per vector.  Codes of the update go out as two byte masks per eight
// elements: bit k of the low byte = kept with sign >= 0, bit k of the high byte = kept with sign <= 0.
template <typename PT, bool GC>
__device__ __forceinline__ unsigned lion_fast4(const PlanView& pv, const LionDev& hp, const Task& t,
                                               const DevTensor& d, const unsigned char* g_s,
                                               const unsigned char* m_s, const float* mean_s,
                                               const float* sc_s, int tid) {
  using E = Elems<PT>;
  const int nvec = t.n >> 3;
  const int nvec_pad = (nvec + 31) & ~31;
  const bool blk128 = d.block == 128u;
  uint16_t* cdst = reinterpret_cast<uint16_t*>(pv.codes + d.code_off + (t.e0 >> 2));
  uint32_t* mdst = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(d.m) + (t.e0 >> 1));
  const uint32_t* msrc = reinterpret_cast<const uint32_t*>(m_s);
  unsigned kept_local = 0;
  // sum over k of ((bits(1.5*2^23) - 8) << 4k) mod 2^32: what the shift-add packing must give back
  constexpr uint32_t PACK_BIAS = (uint32_t)(0x4B3FFFF8ull * 0x11111111ull);
  for (int v = tid; v < nvec_pad; v += NTHREADS) {
    const bool act = v < nvec;
    float g[8];
    uint32_t w = 0x88888888u;
    float sc_old = 1.0f;
    const long long blk = blk128 ? ((t.e0 >> 7) + (v >> 4)) : 0;
    if (act) {
      E::load8(g_s + (size_t)v * 8 * E::BYTES, g);
      w = msrc[v];
      sc_old = sc_s[v >> 4];
      if (GC) {
        const float mu = mean_s[row_of((unsigned)v * 8u, d)];
#pragma unroll
        for (int k = 0; k < 8; k += 2) {
          const float x0 = __fsub_rn(g[k], mu), x1 = __fsub_rn(g[k + 1], mu);
          if (E::IS_BF16) {
            const uint32_t pk = pack_bf16_rn(x0, x1);
            g[k] = bf16lo(pk);
            g[k + 1] = bf16hi(pk);
          } else {
            g[k] = x0;
            g[k + 1] = x1;
          }
        }
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) g[k] = 0.0f;
    }
    float mn[8];
    uint32_t pos = 0, neg = 0;
    float amax = 0.0f;
    // nibble k as the low mantissa bits of 2^23: one byte permute per element (even nibbles sit in the
    // bytes of wl, odd ones in the bytes of wh)
    const uint32_t wl = w & 0x0F0F0F0Fu, wh = (w >> 4) & 0x0F0F0F0Fu;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t fb = __byte_perm((k & 1) ? wh : wl, 0x4B000000u, 0x7540u | (uint32_t)(k >> 1));
      const float mo = __fmul_rn(__uint_as_float(fb) - 8388616.0f, sc_old);
      const float c = __fmaf_rn(g[k], hp.w1, __fmul_rn(mo, hp.b1));
      mn[k] = __fmaf_rn(g[k], hp.w2, __fmul_rn(mo, hp.b2));
      amax = fmaxf(amax, fabsf(mn[k]));
      if (fminf(c, g[k]) > 0.0f) pos |= 1u << k;
      if (fmaxf(c, g[k]) < 0.0f) neg |= 1u << k;
    }
    amax = fmaxf(group_max(amax, 16), 1e-12f);
    const float sc = __fdiv_rn(amax, 7.0f);
    const float inv = __fdividef(1.0f, sc);
    const float magic = 12582912.0f;
    uint32_t word = 0;
    float worst = 0.0f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      // r = rint(mn*inv) + magic in one rounding; mn*inv - rint(...) exactly, by a second fma
      const float r = __fmaf_rn(mn[k], inv, magic);
      worst = fmaxf(worst, fabsf(__fmaf_rn(mn[k], inv, -__fsub_rn(r, magic))));
      word += __float_as_uint(r) << (4 * k);
    }
    word -= PACK_BIAS;
    if (worst > 0.5f - 1e-4f) {  // some product sits near a rounding boundary: redo with the true division
      word = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int qi = min(max((int)rintf(__fdiv_rn(mn[k], sc)), -7), 7);
        word |= (uint32_t)(qi + 8) << (4 * k);
      }
    }
    if (act) {
      mdst[v] = word;
      if ((v & 15) == 0) d.m_scale[blk] = sc;
      cdst[v] = (uint16_t)(pos | (neg << 8));
      kept_local += __popc(pos | neg);
    }
  }
  return kept_local;
}

// The Lion arithmetic on eight elements: in g (centralized grads), m (decoded momentum), pvals
// (weights, only read when has_wd).  Out: m <- new momentum, dl <- direction (+ wd*p), kept bits.
__device__ __forceinline__ uint32_t lion_math8(const LionDev& hp, const float g[8], float m[8],
                                               const float pvals[8], float dl[8], int sg[8],
                                               int cnt) {
  uint32_t kept = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    float c = __fmaf_rn(g[k], hp.w1, __fmul_rn(m[k], hp.b1));
    sg[k] = (c > 0.0f) ? 1 : ((c < 0.0f) ? -1 : 0);
    float s = (float)sg[k];
    m[k] = __fmaf_rn(g[k], hp.w2, __fmul_rn(m[k], hp.b2));
    float dv = hp.has_wd ? __fmaf_rn(pvals[k], hp.wd, s) : s;
    dl[k] = dv;
    if (k < cnt && __fmul_rn(dv, g[k]) > 0.0f) kept |= 1u << k;
  }
  return kept;
}

template <typename PT, int MK, bool MIRROR>
__device__ void lion_main(const PlanView& pv, const LionDev& hp, const Task& t, unsigned char* g_s,
                          unsigned char* m_s, float* mean_s, unsigned* rowmax_s, float* scale_s, float* sc_s,
                          uint64_t* bar,
                          unsigned& parity, unsigned* red_s, int tid) {
  using E = Elems<PT>;
  const DevTensor d = pv.tensors[t.tensor];
  const unsigned char* g = reinterpret_cast<const unsigned char*>(pv.grads[t.tensor]);
  const int n = t.n;
  bool ok = g != nullptr;
  if (ok) {
    // ---- stage gradient rows and momentum bytes ----
    const unsigned gbytes = (unsigned)n * E::BYTES;
    unsigned mbytes;
    const unsigned char* msrc;
    if constexpr (MK == KAON_M_4BIT) { mbytes = (unsigned)(n + 1) >> 1; msrc = (const unsigned char*)d.m + (t.e0 >> 1); }
    else if constexpr (MK == KAON_M_INT8) { mbytes = (unsigned)n; msrc = (const unsigned char*)d.m + t.e0; }
    else if constexpr (MK == KAON_M_BF16) { mbytes = (unsigned)n * 2; msrc = (const unsigned char*)d.m + t.e0 * 2; }
    else { mbytes = (unsigned)n * 4; msrc = (const unsigned char*)d.m + t.e0 * 4; }
    const unsigned char* gsrc = g + t.e0 * E::BYTES;
    const unsigned ghead = stage_tail(g_s, gsrc, gbytes, tid);
    const unsigned mhead = stage_tail(m_s, msrc, mbytes, tid);
    const bool use_bar = (ghead + mhead) != 0;
    if (use_bar) {
      if (tid == 0) {
        fence_async_smem();
        mbar_expect_tx(bar, ghead + mhead);
        if (ghead) bulk_g2s(g_s, gsrc, ghead, bar);
        if (mhead) bulk_g2s(m_s, msrc, mhead, bar);
      }
      ok = mbar_wait(bar, parity, pv.status, 1001u);
      parity ^= 1u;
    }
  }
  ok = __syncthreads_and(ok) != 0;
  if (!ok) {  // tensor without a gradient this step, or a copy that never landed: only signal
    __syncthreads();
    if (tid == 0) signal_counter(pv.done + t.tensor, 1u);
    return;
  }

  // ---- gradient centralization: bf16-rounded (bf16 grads) mean of each staged row ----
  const bool do_gc = hp.gc && d.rows > 0;
  const int C = d.cols;
  const int nrows = d.rows > 0 ? n / C : 1;
  if (do_gc) {
    const int warp = tid >> 5, lane = tid & 31;
    for (int r = warp; r < nrows; r += NTHREADS / 32) {
      const unsigned char* rowp = g_s + (size_t)r * C * E::BYTES;
      float s = 0.0f;
      if ((C & 7) == 0) {
        for (int v = lane; v < (C >> 3); v += 32) {
          float x[8];
          E::load8(rowp + (size_t)v * 8 * E::BYTES, x);
          s += ((x[0] + x[1]) + (x[2] + x[3])) + ((x[4] + x[5]) + (x[6] + x[7]));
        }
      } else {
        for (int i = lane; i < C; i += 32) s += E::load1(rowp, i);
      }
      s = warp_sum(s);
      if (lane == 0) {
        float mean = __fdiv_rn(s, (float)C);
        mean_s[r] = E::IS_BF16 ? round_bf16(mean) : mean;
      }
    }
  }
  if constexpr (MK == KAON_M_4BIT) {  // old block scales of the chunk (the fast path reads them from here)
    const int nblk = d.block == 128u ? (n + 127) >> 7 : 1;
    const long long b0 = d.block == 128u ? (t.e0 >> 7) : 0;
    for (int b = tid; b < nblk; b += NTHREADS) sc_s[b] = d.m_scale[b0 + b];
  }
  if constexpr (MK == KAON_M_INT8) {
    for (int r = tid; r < nrows; r += NTHREADS) {
      rowmax_s[r] = 0u;
      scale_s[r] = d.m_scale[t.row0 + r];  // old scales: the row's first vector overwrites them below
    }
  }
  __syncthreads();

  const int nvec = (n + 7) >> 3;
  const int nvec_pad = (nvec + 31) & ~31;  // whole warps stay in the loop together
  const bool row_uniform = (d.rows <= 0) || ((C & 7) == 0);
  auto load_g = [&](int v, int cnt, float gv[8]) {
    load8_guard<PT>(g_s + (size_t)v * 8 * E::BYTES, cnt, gv);
    if (do_gc) {
      if (row_uniform) {
        float mu = mean_s[row_of((unsigned)v * 8u, d)];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float x = __fsub_rn(gv[k], mu);
          gv[k] = (k < cnt) ? (E::IS_BF16 ? round_bf16(x) : x) : 0.0f;
        }
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float x = __fsub_rn(gv[k], mean_s[k < cnt ? row_of((unsigned)(v * 8 + k), d) : 0]);
          gv[k] = (k < cnt) ? (E::IS_BF16 ? round_bf16(x) : x) : 0.0f;
        }
      }
    }
  };
  const bool need_p = hp.has_wd || !hp.cautious;
  unsigned char* pbase = reinterpret_cast<unsigned char*>(d.p) + t.e0 * E::BYTES;
  SrStream st{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_UPDATE};

  // ---- int8: the row scale needs the row's absmax of the NEW momentum first ----
  if constexpr (MK == KAON_M_INT8) {
    for (int v = tid; v < nvec; v += NTHREADS) {
      const int cnt = min(8, n - v * 8);
      float gv[8], mv[8];
      load_g(v, cnt, gv);
      const int r0 = row_of((unsigned)v * 8u, d);
      if (row_uniform) {
        decode8<MK>(m_s, v, cnt, scale_s[r0], mv);
        float a = 0.0f;
#pragma unroll
        for (int k = 0; k < 8; ++k) a = fmaxf(a, fabsf(__fmaf_rn(gv[k], hp.w2, __fmul_rn(mv[k], hp.b2))));
        atomicMax(rowmax_s + r0, __float_as_uint(a));
      } else {
        for (int k = 0; k < cnt; ++k) {
          const int r = row_of((unsigned)(v * 8 + k), d);
          float mo = __fmul_rn((float)(signed char)m_s[v * 8 + k], scale_s[r]);
          float a = fabsf(__fmaf_rn(gv[k], hp.w2, __fmul_rn(mo, hp.b2)));
          atomicMax(rowmax_s + r, __float_as_uint(a));
        }
      }
    }
    __syncthreads();
  }

  // ---- main pass ----
  uint32_t kept_local = 0;
  bool fast = false;
  if constexpr (MK == KAON_M_4BIT) fast = !hp.has_wd && hp.cautious && (n & 7) == 0 && row_uniform;
  if (fast) {
    if constexpr (MK == KAON_M_4BIT)
      kept_local = do_gc ? lion_fast4<PT, true>(pv, hp, t, d, g_s, m_s, mean_s, sc_s, tid)
                         : lion_fast4<PT, false>(pv, hp, t, d, g_s, m_s, mean_s, sc_s, tid);
  } else
  for (int v = tid; v < nvec_pad; v += NTHREADS) {
    const int cnt = max(0, min(8, n - v * 8));
    float gv[8], mv[8], pvals[8], dl[8];
    int sg[8];
    if (cnt > 0) load_g(v, cnt, gv);
    else {
#pragma unroll
      for (int k = 0; k < 8; ++k) gv[k] = 0.0f;
    }
    // old momentum
    float sc_old = 1.0f;
    long long blk = 0;
    if constexpr (MK == KAON_M_4BIT) {
      blk = (d.block == 128u) ? ((t.e0 >> 7) + (v >> 4)) : 0;
      if (cnt > 0) sc_old = d.m_scale[blk];
    }
    if constexpr (MK == KAON_M_INT8) {
      if (cnt > 0 && row_uniform) sc_old = scale_s[row_of((unsigned)v * 8u, d)];
    }
    if (cnt > 0) {
      if (MK == KAON_M_INT8 && !row_uniform) {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          mv[k] = (k < cnt) ? __fmul_rn((float)(signed char)m_s[v * 8 + k],
                                        scale_s[row_of((unsigned)(v * 8 + k), d)])
                            : 0.0f;
      } else {
        decode8<MK>(m_s, v, cnt, sc_old, mv);
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) mv[k] = 0.0f;
    }
    if (need_p && cnt > 0) load8_guard<PT>(pbase + (size_t)v * 8 * E::BYTES, cnt, pvals);
    else {
#pragma unroll
      for (int k = 0; k < 8; ++k) pvals[k] = 0.0f;
    }
    const uint32_t kept = lion_math8(hp, gv, mv, pvals, dl, sg, cnt);

    // ---- store the new momentum ----
    if constexpr (MK == KAON_M_4BIT) {
      float a = 0.0f;
#pragma unroll
      for (int k = 0; k < 8; ++k) a = fmaxf(a, fabsf(mv[k]));
      a = group_max(a, 16);
      a = fmaxf(a, 1e-12f);
      const float sc = __fdiv_rn(a, 7.0f);
      const float inv = __fdividef(1.0f, sc);
      uint32_t word = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        int qi = (int)quant_round(mv[k], sc, inv, 1e-4f);
        qi = min(max(qi, -7), 7) + 8;
        if (k < cnt) word |= (uint32_t)qi << (4 * k);
      }
      if (cnt > 0) {
        unsigned char* mdst = (unsigned char*)d.m + (t.e0 >> 1) + (size_t)v * 4;
        if (cnt == 8) *reinterpret_cast<uint32_t*>(mdst) = word;
        else
          for (int b = 0; b < (cnt + 1) / 2; ++b) mdst[b] = (unsigned char)(word >> (8 * b));
        if ((v & 15) == 0) d.m_scale[blk] = sc;
      }
    } else if constexpr (MK == KAON_M_INT8) {
      if (cnt > 0) {
        unsigned char* mdst = (unsigned char*)d.m + t.e0 + (size_t)v * 8;
        uint32_t w0 = 0, w1 = 0;
        float sc = 0.0f, inv = 0.0f;
        int rprev = -1;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if (k < cnt) {
            const int r = row_uniform ? row_of((unsigned)v * 8u, d) : row_of((unsigned)(v * 8 + k), d);
            if (r != rprev) {
              sc = __fdiv_rn(fmaxf(__uint_as_float(rowmax_s[r]), 1e-12f), 127.0f);
              inv = __fdividef(1.0f, sc);
              rprev = r;
              // first element of a row writes the row's scale
              const unsigned e = (unsigned)(v * 8 + k);
              if ((d.rows <= 0 && e == 0) || (d.rows > 0 && e == (unsigned)r * (unsigned)C)) d.m_scale[t.row0 + r] = sc;
            }
            int qi = (int)quant_round(mv[k], sc, inv, 1e-3f);
            qi = min(max(qi, -127), 127);
            uint32_t byte = (uint32_t)(qi & 0xFF);
            if (k < 4) w0 |= byte << (8 * k); else w1 |= byte << (8 * (k - 4));
          }
        }
        if (cnt == 8) *reinterpret_cast<uint2*>(mdst) = make_uint2(w0, w1);
        else
          for (int k = 0; k < cnt; ++k) mdst[k] = (unsigned char)((k < 4 ? w0 >> (8 * k) : w1 >> (8 * (k - 4))) & 0xFF);
      }
    } else if constexpr (MK == KAON_M_BF16) {
      if (cnt > 0) {
        unsigned char* mdst = (unsigned char*)d.m + t.e0 * 2 + (size_t)v * 16;
        if (cnt == 8) {
          *reinterpret_cast<uint4*>(mdst) = make_uint4(pack_bf16_rn(mv[0], mv[1]), pack_bf16_rn(mv[2], mv[3]),
                                                      pack_bf16_rn(mv[4], mv[5]), pack_bf16_rn(mv[6], mv[7]));
        } else {
          for (int k = 0; k < cnt; ++k) reinterpret_cast<uint16_t*>(mdst)[k] = (uint16_t)(pack_bf16_rn(mv[k], 0.0f) & 0xffffu);
        }
      }
    } else {
      if (cnt > 0) {
        float* mdst = reinterpret_cast<float*>((unsigned char*)d.m + t.e0 * 4) + (size_t)v * 8;
        for (int k = 0; k < cnt; ++k) mdst[k] = mv[k];
      }
    }

    // ---- hand the update on ----
    if (cnt > 0) {
      if (hp.cautious) {
        uint32_t code16 = 0;  // low byte: kept with sign >= 0; high byte: kept with sign <= 0
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if ((kept >> k) & 1u) code16 |= (sg[k] >= 0 ? (1u << k) : 0u) | (sg[k] <= 0 ? (256u << k) : 0u);
        }
        *reinterpret_cast<uint16_t*>(pv.codes + d.code_off + (t.e0 >> 2) + (size_t)v * 2) = (uint16_t)code16;
        kept_local += __popc(kept);
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) dl[k] = __fmul_rn(dl[k], hp.lr);
        update8<PT>(pbase + (size_t)v * 8 * E::BYTES, cnt, dl, -1.0f, hp.sr != 0, st, d.tensor_id,
                    (uint64_t)((t.e0 >> 3) + v), MIRROR ? &pv.peers : nullptr,
                    (MIRROR && hp.kahan) ? reinterpret_cast<unsigned char*>(d.shift) + (size_t)t.e0 * 2 + (size_t)v * 16 : nullptr);
      }
    }
  }

  // ---- publish: kept count, then the item's completion ----
  if (hp.cautious) {
    for (int o = 16; o > 0; o >>= 1) kept_local += __shfl_xor_sync(0xffffffffu, kept_local, o);
    if ((tid & 31) == 0) red_s[tid >> 5] = kept_local;
  }
  __threadfence();
  __syncthreads();
  if (tid == 0) {
    if (hp.cautious) {
      unsigned tot = 0;
      for (int w = 0; w < NTHREADS / 32; ++w) tot += red_s[w];
      atomicAdd(pv.kept + t.tensor, tot);
    }
    signal_counter(pv.done + t.tensor, 1u);
  }
}

// APPLY item: weights of the run [e0, e0+n) once the tensor's kept count is complete.
template <typename PT, bool MIRROR>
__device__ void lion_apply(const PlanView& pv, const LionDev& hp, const Task& t, int tid) {
  using E = Elems<PT>;
  const DevTensor d = pv.tensors[t.tensor];
  if (pv.grads[t.tensor] == nullptr) return;
  bool ok = true;
  if (tid == 0) ok = wait_counter(pv.done + t.tensor, (unsigned)d.n_main, pv.status, 2001u,
                                 pv.spin_limit ? pv.spin_limit : KAON_SPIN_LIMIT);
  ok = __syncthreads_and(ok) != 0;
  if (!ok) return;
  const unsigned kept = __ldcg(pv.kept + t.tensor);
  // cautious rescale (reference src/kaon/_backend.py:127-134): mean(mask) = count / numel in fp32
  const float denom = fmaxf(__fdiv_rn((float)kept, (float)d.numel), 1e-8f);
  const float vpos = __fmul_rn(__fdiv_rn(1.0f, denom), hp.lr);  // |update| of a kept element, wd == 0
  const int n = t.n;
  const int nvec = (n + 7) >> 3;
  unsigned char* pbase = reinterpret_cast<unsigned char*>(d.p) + t.e0 * E::BYTES;
  const unsigned char* cbase = pv.codes + d.code_off + (t.e0 >> 2);
  SrStream st{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_UPDATE};
  const bool fast_sr = E::IS_BF16 && hp.sr && !hp.has_wd;
  int v_begin = tid;
  if (fast_sr) {
    // four full vectors per trip: all loads are issued before the first use
    const int nfull = n >> 3;
    int v = tid;
    for (; v + 3 * NTHREADS < nfull; v += 4 * NTHREADS) {
      uint4 pw4[4];
      uint32_t c16[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        pw4[u] = *reinterpret_cast<const uint4*>(pbase + (size_t)(v + u * NTHREADS) * 16);
        c16[u] = __ldcg(reinterpret_cast<const unsigned short*>(cbase + (size_t)(v + u * NTHREADS) * 2));
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int vv = v + u * NTHREADS;
        const uint32_t pos = c16[u] & 0xFFu, neg = c16[u] >> 8;
        const uint64_t q = (uint64_t)((t.e0 >> 3) + vv);
        uint32_t nz[4];
        philox_rk(hp, (uint32_t)q, d.tensor_id, hp.step, (uint32_t)KAON_TAG_UPDATE | ((uint32_t)(q >> 32) << 8), nz);
        uint32_t pw[4] = {pw4[u].x, pw4[u].y, pw4[u].z, pw4[u].w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int k0 = 2 * j, k1 = 2 * j + 1;
          float d0 = ((pos >> k0) & 1u) ? vpos : 0.0f;
          d0 = ((neg >> k0) & 1u) ? -vpos : d0;
          float d1 = ((pos >> k1) & 1u) ? vpos : 0.0f;
          d1 = ((neg >> k1) & 1u) ? -vpos : d1;
          const uint32_t b0 = __float_as_uint(__fsub_rn(bf16lo(pw[j]), d0)) + (nz[j] & 0xffffu);
          const uint32_t b1 = __float_as_uint(__fsub_rn(bf16hi(pw[j]), d1)) + (nz[j] >> 16);
          pw[j] = __byte_perm(b0, b1, 0x7632);
        }
        const uint4 out = make_uint4(pw[0], pw[1], pw[2], pw[3]);
        *reinterpret_cast<uint4*>(pbase + (size_t)vv * 16) = out;
        mirror16(MIRROR ? &pv.peers : nullptr, pbase + (size_t)vv * 16, out);
      }
    }
    v_begin = v;
  }
  for (int v = v_begin; v < nvec; v += NTHREADS) {
    const int cnt = min(8, n - v * 8);
    const uint32_t c16 = __ldcg(reinterpret_cast<const unsigned short*>(cbase + (size_t)v * 2));
    const uint32_t pos = c16 & 0xFFu, neg = c16 >> 8;
    if (fast_sr && cnt == 8) {
      // eight bf16 weights: p - (+-vpos | 0), noise from the Philox stream, truncate
      const uint64_t q = (uint64_t)((t.e0 >> 3) + v);
      uint32_t nz[4];
      philox_rk(hp, (uint32_t)q, d.tensor_id, hp.step, (uint32_t)KAON_TAG_UPDATE | ((uint32_t)(q >> 32) << 8), nz);
      uint4* pp = reinterpret_cast<uint4*>(pbase + (size_t)v * 16);
      const uint4 pw4 = *pp;
      uint32_t pw[4] = {pw4.x, pw4.y, pw4.z, pw4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int k0 = 2 * j, k1 = 2 * j + 1;
        const float d0 = ((pos >> k0) & 1u) ? (((neg >> k0) & 1u) ? 0.0f : vpos) : (((neg >> k0) & 1u) ? -vpos : 0.0f);
        const float d1 = ((pos >> k1) & 1u) ? (((neg >> k1) & 1u) ? 0.0f : vpos) : (((neg >> k1) & 1u) ? -vpos : 0.0f);
        const uint32_t b0 = __float_as_uint(__fsub_rn(bf16lo(pw[j]), d0)) + (nz[j] & 0xffffu);
        const uint32_t b1 = __float_as_uint(__fsub_rn(bf16hi(pw[j]), d1)) + (nz[j] >> 16);
        pw[j] = __byte_perm(b0, b1, 0x7632);
      }
      const uint4 out = make_uint4(pw[0], pw[1], pw[2], pw[3]);
      *pp = out;
      mirror16(MIRROR ? &pv.peers : nullptr, pp, out);
      continue;
    }
    float dl[8];
    if (hp.has_wd) {
      float pvals[8];
      load8_guard<PT>(pbase + (size_t)v * 8 * E::BYTES, cnt, pvals);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int pb = (pos >> k) & 1, nb = (neg >> k) & 1;
        const float dv = __fmaf_rn(pvals[k], hp.wd, (float)(pb - nb));
        dl[k] = (pb | nb) ? __fmul_rn(__fdiv_rn(dv, denom), hp.lr) : 0.0f;
      }
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int pb = (pos >> k) & 1, nb = (neg >> k) & 1;
        dl[k] = (pb == nb) ? 0.0f : (pb ? vpos : -vpos);
      }
    }
    update8<PT>(pbase + (size_t)v * 8 * E::BYTES, cnt, dl, -1.0f, hp.sr != 0, st, d.tensor_id,
                (uint64_t)((t.e0 >> 3) + v), MIRROR ? &pv.peers : nullptr,
                (MIRROR && hp.kahan) ? reinterpret_cast<unsigned char*>(d.shift) + (size_t)t.e0 * 2 + (size_t)v * 16 : nullptr);
  }
}

// MIRROR = true is the general build: weight mirrors on other GPUs and the Kahan write.  MIRROR = false
// compiles both out (the common single-GPU stochastic-rounding / nearest step pays nothing for them).
template <typename PT, int MK, bool MIRROR>
__global__ void __launch_bounds__(NTHREADS, 4) lion_kernel(PlanView pv, LionDev hp) {
  extern __shared__ __align__(128) unsigned char dyn[];
  __shared__ float mean_s[MAX_TASK_ROWS];
  __shared__ unsigned rowmax_s[MK == KAON_M_INT8 ? MAX_TASK_ROWS : 1];
  __shared__ float scale_s[MK == KAON_M_INT8 ? MAX_TASK_ROWS : 1];
  __shared__ float sc_s[MK == KAON_M_4BIT ? CAP / 128 : 1];
  __shared__ __align__(8) uint64_t bar;
  __shared__ int next_s[2];
  __shared__ unsigned red_s[NTHREADS / 32];
  unsigned char* g_s = dyn;
  unsigned char* m_s = dyn + (size_t)CAP * Elems<PT>::BYTES;
  const int tid = threadIdx.x;
  auto claim_next = [&](int slot) {
    if (tid == 0) {
      const unsigned st = *reinterpret_cast<volatile unsigned*>(pv.status);
      next_s[slot] = st ? 0x7fffffff : (int)atomicAdd(pv.task_counter, 1u);
    }
  };
  if (tid == 0) mbar_init(&bar, 1);
  claim_next(0);
  __syncthreads();
  unsigned parity = 0;
  int slot = 0;
  int cur = next_s[0];
  while (cur < pv.n_tasks) {
    claim_next(slot ^ 1);
    const Task t = pv.tasks[cur];
    if (t.phase == PH_LION_MAIN)
      lion_main<PT, MK, MIRROR>(pv, hp, t, g_s, m_s, mean_s, rowmax_s, scale_s, sc_s, &bar, parity, red_s, tid);
    else
      lion_apply<PT, MIRROR>(pv, hp, t, tid);
    __syncthreads();
    slot ^= 1;
    cur = next_s[slot];
  }
}

typedef void (*LionKernel)(PlanView, LionDev);

static LionKernel pick_lion(int pdt, int mk, bool mirror) {
#define KAON_PICK(PT, MIR)                                         \
  switch (mk) {                                                    \
    case KAON_M_F32: return lion_kernel<PT, KAON_M_F32, MIR>;      \
    case KAON_M_BF16: return lion_kernel<PT, KAON_M_BF16, MIR>;    \
    case KAON_M_INT8: return lion_kernel<PT, KAON_M_INT8, MIR>;    \
    case KAON_M_4BIT: return lion_kernel<PT, KAON_M_4BIT, MIR>;    \
    default: return nullptr;                                       \
  }
  if (mirror) {
    if (pdt == KAON_DT_BF16) { KAON_PICK(__nv_bfloat16, true) }
    KAON_PICK(float, true)
  }
  if (pdt == KAON_DT_BF16) { KAON_PICK(__nv_bfloat16, false) }
  KAON_PICK(float, false)
#undef KAON_PICK
}

int configure_launch(kaon_plan* pl, const cudaDeviceProp& prop) {
  const size_t esz = pl->param_dtype == KAON_DT_BF16 ? 2 : 4;
  pl->smem_bytes = (size_t)CAP * esz + momentum_bytes_per_cap(pl->momentum_kind);
  int per_sm = 2;
  if (pl->optimizer == KAON_OPT_LION) {
    LionKernel k = pick_lion(pl->param_dtype, pl->momentum_kind, false);
    if (!k) return fail(KAON_E_INVALID, "no Lion kernel for this dtype combination");
    KAON_CUDA(cudaFuncSetAttribute((const void*)k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl->smem_bytes));
    KAON_CUDA(cudaFuncSetAttribute((const void*)pick_lion(pl->param_dtype, pl->momentum_kind, true),
                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl->smem_bytes));
    KAON_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void*)k, NTHREADS, pl->smem_bytes));
    if (per_sm < 1) return fail(KAON_E_UNSUPPORTED, "Lion kernel does not fit on an SM (shared memory %zu)", pl->smem_bytes);
  }
  pl->grid = prop.multiProcessorCount * per_sm;
  return KAON_OK;
}

}  // namespace kaon

using namespace kaon;

extern "C" int kaon_lion_step(kaon_plan* pl, const kaon_lion_hparams* h, uint64_t seed, uint32_t step,
                              void* stream) {
  if (!pl || !h) return fail(KAON_E_INVALID, "kaon_lion_step: null argument");
  if (pl->optimizer != KAON_OPT_LION) return fail(KAON_E_INVALID, "plan was not built for Lion");
  if (int rc = check_device(pl)) return rc;
  if (h->bf16_method < KAON_W_NONE || h->bf16_method > KAON_W_KAHAN) return fail(KAON_E_UNSUPPORTED, "bf16_method %d", h->bf16_method);
  if (int rc = check_kahan(pl, h->bf16_method)) return rc;
  LionDev hp;
  hp.lr = (float)h->lr;
  hp.b1 = (float)h->beta1; hp.w1 = (float)(1.0 - h->beta1);
  hp.b2 = (float)h->beta2; hp.w2 = (float)(1.0 - h->beta2);
  hp.wd = (float)h->weight_decay;
  hp.has_wd = h->weight_decay != 0.0;
  hp.cautious = h->cautious != 0;
  hp.gc = h->gradient_centralization != 0;
  hp.sr = h->bf16_method == KAON_W_SR && pl->param_dtype == KAON_DT_BF16;
  hp.kahan = h->bf16_method == KAON_W_KAHAN && pl->param_dtype == KAON_DT_BF16;
  hp.step = step; hp.k0 = (uint32_t)seed; hp.k1 = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; ++r) { hp.rk0[r] = hp.k0 + 0x9E3779B9u * (uint32_t)r; hp.rk1[r] = hp.k1 + 0xBB67AE85u * (uint32_t)r; }
  cudaStream_t s = (cudaStream_t)stream;
  PlanView v = pl->view;
  if (hp.cautious) { v.tasks = pl->d_tasks_full; v.n_tasks = pl->n_tasks_full; }
  else { v.tasks = pl->d_tasks_main; v.n_tasks = pl->n_tasks_main; }
  KAON_CUDA(cudaMemsetAsync(v.task_counter, 0, pl->counters_bytes - sizeof(unsigned), s));
  LionKernel k = pick_lion(pl->param_dtype, pl->momentum_kind, v.peers.n > 0 || hp.kahan);
  k<<<pl->grid, NTHREADS, pl->smem_bytes, s>>>(v, hp);
  KAON_CUDA(cudaGetLastError());
  pl->launches += 1;
  return KAON_OK;
}

// ---------------------------------------------------------------------------------------------------
// Lion step for ONE tensor that allocates nothing.
//
// Some callers cannot call cudaMalloc at the point where they step the optimizer: code that runs
// under a memory pool it must not disturb, a real-time or fault-handling path that may only launch
// work, a host framework that hands this library raw pointers but keeps every allocation for itself.
// kaon_plan_create allocates the descriptor table, the work list, the counters and the 2-bit code
// scratch with cudaMalloc; the entry point below needs none of that.  Its table, work list, counters and
// code scratch live in the file-scope device array g_noalloc, which every GPU that loads this library
// holds (about 1.3 MiB) until the process exits; a small set-up kernel fills it from the call's
// arguments, then the same persistent kernel as kaon_lion_step runs over it.
//
// Limits and rules: one tensor per call, at most KAON_NOALLOC_MAX_NUMEL elements, 4-bit momentum
// (block 128, or one block for a tensor of <= 128 elements), bf16 or fp32 weights.  All calls on a
// device share the array, and it keeps what the last call left there: the set-up kernel rewrites every
// field the step reads and zeroes the counters, so calls that follow each other on one stream are
// independent, but two calls whose kernels overlap on the GPU (different streams) race on it.  The
// first call on a device looks the array's address up and configures the kernel (no allocation, but
// synchronous driver work, serialised by a host mutex); make that first call outside any stream capture.
// Device status: if a bounded wait inside a call's kernel runs out, that call stops early (its CTAs
// drain) and the code stays in the array; the NEXT call's set-up kernel moves it to a "last failure"
// word and clears the live word, so later calls run normally.  kaon_lion_noalloc_status reads and
// clears both words: a caller that must know whether every step completed calls it after the steps.
// ---------------------------------------------------------------------------------------------------
namespace kaon {

constexpr long long NOALLOC_MAX_NUMEL = KAON_NOALLOC_MAX_NUMEL;
constexpr int NOALLOC_MAX_ITEMS = 4096;  // work items per phase
constexpr size_t NA_OFF_COUNTERS = 0;    // status @0, last failure @4, task counter @64, done @68, kept @72
constexpr size_t NA_OFF_TENSOR = 256;
constexpr size_t NA_OFF_GRAD = 512;
constexpr size_t NA_OFF_TASKS = 1024;
constexpr size_t NA_OFF_CODES = NA_OFF_TASKS + 2 * (size_t)NOALLOC_MAX_ITEMS * sizeof(Task);
constexpr size_t NA_BYTES = NA_OFF_CODES + (size_t)NOALLOC_MAX_NUMEL / 4 + 256;

static __device__ __align__(256) unsigned char g_noalloc[NA_BYTES];

// Fills the table, the gradient pointer, the work list (all MAIN items, then all APPLY items) and
// clears the counters.  Device code names the array directly.
__global__ void noalloc_setup_kernel(DevTensor d, const void* grad, long long item_elems, int item_rows,
                                     int n_items) {
  unsigned* counters = reinterpret_cast<unsigned*>(g_noalloc + NA_OFF_COUNTERS);
  Task* tasks = reinterpret_cast<Task*>(g_noalloc + NA_OFF_TASKS);
  if (threadIdx.x == 0) {
    *reinterpret_cast<DevTensor*>(g_noalloc + NA_OFF_TENSOR) = d;
    *reinterpret_cast<const void**>(g_noalloc + NA_OFF_GRAD) = grad;
    if (counters[0] != 0u) {  // an earlier call's bounded wait ran out: keep its code, run this call normally
      if (counters[1] == 0u) counters[1] = counters[0];
      counters[0] = 0u;
    }
    counters[16] = 0u;  // task counter
    counters[17] = 0u;  // done
    counters[18] = 0u;  // kept
  }
  for (int i = threadIdx.x; i < n_items; i += blockDim.x) {
    const long long e0 = (long long)i * item_elems;
    Task t;
    t.tensor = 0;
    t.phase = PH_LION_MAIN;
    t.e0 = e0;
    t.n = (int)min(item_elems, d.numel - e0);
    t.row0 = i * item_rows;
    t.slot = 0;
    t.pad = 0;
    tasks[i] = t;
    t.phase = PH_LION_APPLY;
    tasks[n_items + i] = t;
  }
}

struct NoAllocDevice {
  bool ready = false;
  unsigned char* base = nullptr;  // device address of g_noalloc on this device
  int grid[2] = {0, 0};           // per param dtype
  size_t smem[2] = {0, 0};
};
static NoAllocDevice g_na_dev[64];
static std::mutex g_na_mutex;  // guards the once-per-device set-up against concurrent first calls

// Once per device, with that device current: the array's name is a host-side stand-in, so the address
// the kernels get must come from cudaGetSymbolAddress.
static int noalloc_setup_device(int dev) {
  NoAllocDevice& nd = g_na_dev[dev];
  void* ptr = nullptr;
  cudaError_t ce = cudaGetSymbolAddress(&ptr, g_noalloc);
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaGetSymbolAddress(g_noalloc)");
  if (!ptr) return fail(KAON_E_CUDA, "cudaGetSymbolAddress(g_noalloc) returned a null address");
  cudaDeviceProp prop;
  KAON_CUDA(cudaGetDeviceProperties(&prop, dev));
  for (int pdt = 0; pdt < 2; ++pdt) {
    LionKernel k = pick_lion(pdt, KAON_M_4BIT, false);
    nd.smem[pdt] = (size_t)CAP * (pdt == KAON_DT_BF16 ? 2 : 4) + momentum_bytes_per_cap(KAON_M_4BIT);
    KAON_CUDA(cudaFuncSetAttribute((const void*)k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)nd.smem[pdt]));
    int per_sm = 0;
    KAON_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void*)k, NTHREADS, nd.smem[pdt]));
    if (per_sm < 1) return fail(KAON_E_UNSUPPORTED, "Lion kernel does not fit on an SM");
    nd.grid[pdt] = prop.multiProcessorCount * per_sm;
  }
  nd.base = reinterpret_cast<unsigned char*>(ptr);
  nd.ready = true;
  return KAON_OK;
}

}  // namespace kaon

extern "C" int kaon_lion_step_noalloc(const kaon_tensor_desc* t, int param_dtype, const kaon_lion_hparams* h,
                                      uint64_t seed, uint32_t step, void* stream) {
  if (!t || !h) return fail(KAON_E_INVALID, "kaon_lion_step_noalloc: null argument");
  if (param_dtype != KAON_DT_F32 && param_dtype != KAON_DT_BF16) return fail(KAON_E_INVALID, "param_dtype %d", param_dtype);
  if (h->bf16_method != KAON_W_NONE && h->bf16_method != KAON_W_SR) return fail(KAON_E_UNSUPPORTED, "bf16_method %d", h->bf16_method);
  if (!t->p || !t->g || !t->m || !t->m_scale) return fail(KAON_E_INVALID, "kaon_lion_step_noalloc: weights, gradient, momentum and m_scale must all be set");
  if (((uintptr_t)t->p | (uintptr_t)t->g | (uintptr_t)t->m) & 15) return fail(KAON_E_INVALID, "kaon_lion_step_noalloc: pointers must be 16-byte aligned");
  const long long n = t->numel;
  if (n <= 0) return n == 0 ? KAON_OK : fail(KAON_E_INVALID, "negative numel");
  if (n > NOALLOC_MAX_NUMEL)
    return fail(KAON_E_UNSUPPORTED, "kaon_lion_step_noalloc: %lld elements exceed the built-in scratch (KAON_NOALLOC_MAX_NUMEL = %lld); use a plan (kaon_plan_create + kaon_lion_step) for larger tensors", n, NOALLOC_MAX_NUMEL);
  if (!(t->block == 128 || ((long long)t->block == n && n <= 128)))
    return fail(KAON_E_UNSUPPORTED, "kaon_lion_step_noalloc: 4-bit block size %u (numel %lld) is not handled", t->block, n);
  // work items: the same cut as a plan makes (whole rows, each item starting on a 4-bit block boundary)
  long long item_elems;
  int item_rows = 0;
  long long C = n;
  if (t->rows > 0) {
    C = n / t->rows;
    if (C * t->rows != n || t->rows > 0x7fffffffll) return fail(KAON_E_INVALID, "numel %lld not divisible by rows %lld", n, (long long)t->rows);
    if (n <= CAP && t->rows <= MAX_TASK_ROWS) {
      item_elems = n; item_rows = (int)t->rows;
    } else {
      long long g = C, b = 128;
      while (b) { long long r = g % b; g = b; b = r; }
      const long long unit = 128 / g;
      long long rpt = (CAP / C) / unit * unit;
      rpt = std::min<long long>(rpt, MAX_TASK_ROWS / unit * unit);
      if (rpt <= 0) return fail(KAON_E_UNSUPPORTED, "kaon_lion_step_noalloc: rows of %lld elements cannot be cut into block-aligned work items", C);
      item_rows = (int)rpt; item_elems = rpt * C;
    }
  } else {
    item_elems = CAP;
  }
  const long long n_items = (n + item_elems - 1) / item_elems;
  if (n_items > NOALLOC_MAX_ITEMS) return fail(KAON_E_UNSUPPORTED, "kaon_lion_step_noalloc: %lld work items exceed the built-in work list (%d)", n_items, NOALLOC_MAX_ITEMS);

  int dev = 0;
  KAON_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(KAON_E_UNSUPPORTED, "device index %d", dev);
  {
    std::lock_guard<std::mutex> lock(g_na_mutex);
    if (!g_na_dev[dev].ready) {
      int rc = noalloc_setup_device(dev);
      if (rc) return rc;
    }
  }
  const NoAllocDevice& nd = g_na_dev[dev];

  DevTensor d{};
  d.p = t->p; d.m = t->m; d.m_scale = t->m_scale;
  d.numel = n; d.code_off = 0;
  d.rows = (int)t->rows;
  d.cols = (int)std::min<long long>(C, 0x7fffffff);
  d.row_magic = d.cols > 1 ? (unsigned)((0x100000000ull + (unsigned)d.cols - 1) / (unsigned)d.cols) : 0u;
  d.tensor_id = t->tensor_id; d.block = t->block;
  d.n_main = (int)n_items;

  LionDev hp;
  hp.lr = (float)h->lr;
  hp.b1 = (float)h->beta1; hp.w1 = (float)(1.0 - h->beta1);
  hp.b2 = (float)h->beta2; hp.w2 = (float)(1.0 - h->beta2);
  hp.wd = (float)h->weight_decay;
  hp.has_wd = h->weight_decay != 0.0;
  hp.cautious = h->cautious != 0;
  hp.gc = h->gradient_centralization != 0;
  hp.sr = h->bf16_method == KAON_W_SR && param_dtype == KAON_DT_BF16;
  hp.kahan = 0;
  hp.step = step; hp.k0 = (uint32_t)seed; hp.k1 = (uint32_t)(seed >> 32);
  for (int r = 0; r < 10; ++r) { hp.rk0[r] = hp.k0 + 0x9E3779B9u * (uint32_t)r; hp.rk1[r] = hp.k1 + 0xBB67AE85u * (uint32_t)r; }

  unsigned* counters = reinterpret_cast<unsigned*>(nd.base + NA_OFF_COUNTERS);
  PlanView v{};
  v.tensors = reinterpret_cast<const DevTensor*>(nd.base + NA_OFF_TENSOR);
  v.grads = reinterpret_cast<const void* const*>(nd.base + NA_OFF_GRAD);
  v.tasks = reinterpret_cast<const Task*>(nd.base + NA_OFF_TASKS);
  v.n_tasks = (int)(hp.cautious ? 2 * n_items : n_items);
  v.n_tensors = 1;
  v.status = counters;
  v.task_counter = counters + 16;
  v.done = counters + 17;
  v.kept = counters + 18;
  v.aux = nullptr;
  v.codes = nd.base + NA_OFF_CODES;
  cudaStream_t s = (cudaStream_t)stream;
  noalloc_setup_kernel<<<1, 256, 0, s>>>(d, t->g, item_elems, item_rows, (int)n_items);
  KAON_CUDA(cudaGetLastError());
  LionKernel k = pick_lion(param_dtype, KAON_M_4BIT, false);
  k<<<nd.grid[param_dtype], NTHREADS, nd.smem[param_dtype], s>>>(v, hp);
  KAON_CUDA(cudaGetLastError());
  return KAON_OK;
}

extern "C" int kaon_lion_noalloc_status(void* stream) {
  int dev = 0;
  KAON_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(KAON_E_UNSUPPORTED, "device index %d", dev);
  unsigned char* base = nullptr;
  {
    std::lock_guard<std::mutex> lock(g_na_mutex);
    if (!g_na_dev[dev].ready) return KAON_OK;  // no call has run on this device yet
    base = g_na_dev[dev].base;
  }
  cudaStream_t s = (cudaStream_t)stream;
  unsigned st[2] = {0u, 0u};
  KAON_CUDA(cudaMemcpyAsync(st, base + NA_OFF_COUNTERS, sizeof st, cudaMemcpyDeviceToHost, s));
  KAON_CUDA(cudaStreamSynchronize(s));
  if (st[0] == 0u && st[1] == 0u) return KAON_OK;
  KAON_CUDA(cudaMemsetAsync(base + NA_OFF_COUNTERS, 0, sizeof st, s));
  return fail(KAON_E_DEVICE, "kaon_lion_step_noalloc: device status %u: a bounded wait ran out in an earlier call "
                             "(code = 1000*phase + kind); that call's tensor was not fully stepped",
              st[0] ? st[0] : st[1]);
}
