// AdaPNM (positive-negative momentum over Adakaon's factored second moment) on the plan machinery of
// the Adakaon step.  Replaces reference src/kaon/adapnm.py:1039-1273 (the foreach buckets and the
// per-parameter step).
//
// One step of a plan:
//   1. STATS + FINAL of the Adakaon kernels (row / column statistics of the centralised gradient, the
//      factors r_i = rsqrt(row_i / mean(row)), c_j = rsqrt(col_j), the centralisation means) - the second
//      moment is the same recurrence as Adakaon's (reference src/kaon/_factored.py:26-83).
//   2. SUM: flat items of 8192 elements over every factored tensor: both momenta are decoded, the positive
//      one takes the gradient, u = pn * ((r*c) * bc2); each item leaves its sum of u^2 (double), its count
//      of u*g > 0 and, for int8 momentum, the row maxima of the new positive momentum.
//   3. REDUCE: one CTA per factored tensor adds the item partials in item order: clip divisor, cautious
//      denominator.
//   4. APPLY: the same flat items again: recompute, weight decay, clip, mask, weight write, store the
//      positive momentum through its codec.
//   5. FLAT: one CTA per 1-D tensor (full second moment v, optional running maximum) doing 2-4 in place.
// The two stored momenta swap roles every step (reference src/kaon/adapnm.py:588-596); `swap` selects.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <vector>

#include <type_traits>

#include "adakaon_dev.h"
#include "kaon_device.cuh"
#include "kaon_host.h"
#include "kaon_elem.cuh"
#include "kaon_ops.cuh"

namespace kaon {

constexpr int PNM_ITEM = 16384;
constexpr int PT_THREADS = 256;

struct PnmDev {
  float fb, fw;          // beta1^2, 1 - beta1^2
  float c1, c2, c3;      // 1 + beta0, -beta0, 1 / noise_norm
  float bc2, fstep;      // sqrt(1 - beta2^t), lr / (1 - beta1^t)
  float wdsc;            // 1 - lr * weight_decay
  float fb2, fw2, eps;   // 1-D second moment: beta2, 1 - beta2, eps on the denominator
  float clip;
  int has_wd, clip_on, cautious, gc, ams, sr, kahan, swap;
  uint32_t step, k0, k1;
};

struct PnmBufs {
  void* m[2];       // stored "m_pos", "m_neg"
  float* sc[2];
  float* max_v;     // 1-D tensors with ams_bound, else null
};

struct PnmView {
  const Task* items;      // flat items of the factored tensors, tensor by tensor
  int n_items;
  const int* item_begin;  // [n_tensors + 1] ranges into items
  const PnmBufs* bufs;    // [n_tensors]
  double* part;           // [n_items] sum of u^2
  unsigned* kpart;        // [n_items] count of u*g > 0
  float* scal;            // [n_tensors][2] clip divisor, cautious denominator
  const int* fact;        // indices of the factored tensors
  int n_fact;
  const int* flat;        // indices of the 1-D tensors
  int n_flat;
};

// Weight write of one trip (reference src/kaon/adapnm.py:1090-1092, 1117-1124; _backend.py:82-142).
template <typename PT>
__device__ __forceinline__ void pnm_write(const PnmDev& hp, const DevTensor& d, const PnmTrip& tr, long long e, int cnt,
                                          float div, float denom, const SrStream& s_upd, const Peers* peers) {
  using E = Elems<PT>;
  unsigned char* pe = reinterpret_cast<unsigned char*>(d.p) + e * E::BYTES;
  float pw[8], sh[8];
  load8_guard<PT>(pe, cnt, pw);
  uint32_t nz[4] = {0u, 0u, 0u, 0u};
  if (hp.sr) s_upd.draw8(d.tensor_id, (uint64_t)(e >> 3), nz);
  const bool kahan = E::IS_BF16 && hp.kahan;
  const float rdiv = __frcp_rn(div), rdenom = __frcp_rn(denom);
  unsigned char* she = kahan ? reinterpret_cast<unsigned char*>(d.shift) + e * 2 : nullptr;
  if (kahan) load8_guard<__nv_bfloat16>(she, cnt, sh);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    if (k >= cnt) continue;
    float p0 = pw[k];
    if (hp.has_wd) p0 = E::IS_BF16 ? round_bf16(__fmul_rn(p0, hp.wdsc)) : __fmul_rn(p0, hp.wdsc);
    float dl = hp.clip_on ? div_by(tr.u[k], div, rdiv) : tr.u[k];
    dl = __fmul_rn(dl, hp.fstep);
    if (hp.cautious) dl = (__fmul_rn(dl, tr.y[k]) > 0.0f) ? div_by(dl, denom, rdenom) : 0.0f;
    if (kahan) kahan_step(p0, sh[k], dl);
    else p0 = write_step_pnm<PT>(p0, dl, hp.sr != 0, noise_lane_pnm(nz, k));
    pw[k] = p0;
  }
  if constexpr (E::IS_BF16) {
    // every value is a bf16 already: the high halves are the bits
    if (cnt >= 8) {
      const uint4 out = make_uint4((__float_as_uint(pw[0]) >> 16) | (__float_as_uint(pw[1]) & 0xFFFF0000u),
                                   (__float_as_uint(pw[2]) >> 16) | (__float_as_uint(pw[3]) & 0xFFFF0000u),
                                   (__float_as_uint(pw[4]) >> 16) | (__float_as_uint(pw[5]) & 0xFFFF0000u),
                                   (__float_as_uint(pw[6]) >> 16) | (__float_as_uint(pw[7]) & 0xFFFF0000u));
      *reinterpret_cast<uint4*>(pe) = out;
      mirror16(peers, pe, out);
      if (kahan)
        *reinterpret_cast<uint4*>(she) =
            make_uint4((__float_as_uint(sh[0]) >> 16) | (__float_as_uint(sh[1]) & 0xFFFF0000u),
                       (__float_as_uint(sh[2]) >> 16) | (__float_as_uint(sh[3]) & 0xFFFF0000u),
                       (__float_as_uint(sh[4]) >> 16) | (__float_as_uint(sh[5]) & 0xFFFF0000u),
                       (__float_as_uint(sh[6]) >> 16) | (__float_as_uint(sh[7]) & 0xFFFF0000u));
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) if (k < cnt) {
        reinterpret_cast<uint16_t*>(pe)[k] = (uint16_t)(__float_as_uint(pw[k]) >> 16);
        if (kahan) reinterpret_cast<uint16_t*>(she)[k] = (uint16_t)(__float_as_uint(sh[k]) >> 16);
      }
      mirror_copy(peers, pe, cnt * 2);
    }
  } else {
    float* pf = reinterpret_cast<float*>(pe);
    if (cnt >= 8) {
      reinterpret_cast<float4*>(pf)[0] = make_float4(pw[0], pw[1], pw[2], pw[3]);
      reinterpret_cast<float4*>(pf)[1] = make_float4(pw[4], pw[5], pw[6], pw[7]);
      mirror16(peers, pf, make_uint4(__float_as_uint(pw[0]), __float_as_uint(pw[1]), __float_as_uint(pw[2]), __float_as_uint(pw[3])));
      mirror16(peers, pf + 4, make_uint4(__float_as_uint(pw[4]), __float_as_uint(pw[5]), __float_as_uint(pw[6]), __float_as_uint(pw[7])));
    } else {
#pragma unroll
      for (int k = 0; k < 8; ++k) if (k < cnt) pf[k] = pw[k];
      mirror_copy(peers, pf, cnt * 4);
    }
  }
}

// ----------------------------------------------------------------------------- factored tensors

template <typename PT, int MK, bool APPLY>
__global__ void __launch_bounds__(PT_THREADS, 4) pnm_pass_kernel(PlanView pv, PnmDev hp, PnmView x) {
  using E = Elems<PT>;
  __shared__ double red_d[PT_THREADS / 32];
  __shared__ unsigned red_u[PT_THREADS / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const SrStream s_upd{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_UPDATE};
  for (int it = blockIdx.x; it < x.n_items; it += gridDim.x) {
    const Task t = x.items[it];
    const DevTensor d = pv.tensors[t.tensor];
    const unsigned char* g = reinterpret_cast<const unsigned char*>(pv.grads[t.tensor]);
    double ss = 0.0;
    unsigned kept = 0;
    if (g != nullptr) {
      const PnmBufs b = x.bufs[t.tensor];
      void* pos = b.m[hp.swap];
      float* psc = b.sc[hp.swap];
      const void* neg = b.m[hp.swap ^ 1];
      const float* nsc = b.sc[hp.swap ^ 1];
      const int C = d.cols;
      const float* rfac = pv.aux + aux_rfac(d);
      const float* cfac = pv.aux + aux_cfac(d);
      const float* mean = pv.aux + aux_mean(d);
      unsigned* rowmax = reinterpret_cast<unsigned*>(pv.aux + aux_rowmax(d));
      // int8: the positive buffer's row scales as they were before this step (its rows get new ones in APPLY)
      const float* psc_rd = MK == KAON_M_INT8 ? pv.aux + aux_oldsc(d) : psc;
      const int bsh = d.bshift;  // 4-bit: element -> block shift (31: one block)
      float div = 1.0f, denom = 1.0f;
      if (APPLY) { div = x.scal[2 * t.tensor]; denom = x.scal[2 * t.tensor + 1]; }
      const int nvec = (t.n + 7) >> 3;
      for (int v0 = 0; v0 < nvec; v0 += PT_THREADS) {
        const int v = v0 + tid;
        const long long e = t.e0 + (long long)v * 8;
        const int cnt_rt = v < nvec ? min(8, (int)(t.e0 + t.n - e)) : 0;
        int r0 = 0, c0 = 0;
        if (cnt_rt > 0) {
          r0 = e < 0x100000000ll ? (int)((unsigned)e / (unsigned)C) : (int)(e / C);
          c0 = (int)(e - (long long)r0 * C);
        }
        // FULL: every lane of the warp has eight elements inside one row, so the element guards and the
        // row bookkeeping fold away at compile time; anything else (a row end, a tensor's tail) takes
        // the guarded form.  The choice is per warp: the 4-bit store shuffles block maxima across lanes.
        auto trip = [&](auto full_tag) {
          constexpr bool FULL = decltype(full_tag)::value;
          const int cnt = FULL ? 8 : cnt_rt;
          PnmTrip tr;
          tr.first = 0u;
          if (cnt > 0) {
            float gx[8], mpo[8], mno[8];
            int cl[8];
            load8_guard<PT>(g + e * E::BYTES, cnt, gx);
            int r = r0, c = c0;
            // the common trip: eight elements of one row (no row bookkeeping, one row factor, one mean)
            const bool one_row = FULL || (cnt == 8 && c + 8 <= C);
            if (one_row) {
  #pragma unroll
              for (int k = 0; k < 8; ++k) { tr.rw[k] = r; cl[k] = c + k; }
              if (c == 0) tr.first = 1u;
            } else {
  #pragma unroll
              for (int k = 0; k < 8; ++k) {
                tr.rw[k] = 0; cl[k] = 0;
                if (k < cnt) {
                  while (c >= C) { c -= C; ++r; }
                  tr.rw[k] = r;
                  cl[k] = c;
                  if (c == 0) tr.first |= 1u << k;
                  ++c;
                }
              }
            }
            pnm_decode8<MK>(pos, psc_rd, e, cnt, tr.rw, bsh, mpo);
            pnm_decode8<MK>(neg, nsc, e, cnt, tr.rw, bsh, mno);
            auto chain = [&](int k, float rf, float mu, float cf) {
              const float yk = pnm_centered<PT>(gx[k], mu, hp.gc != 0);
              const float mpn = __fmaf_rn(yk, hp.fw, __fmul_rn(mpo[k], hp.fb));
              const float pn = __fmul_rn(__fmaf_rn(mno[k], hp.c2, __fmul_rn(mpn, hp.c1)), hp.c3);
              const float inv = __fmul_rn(__fmul_rn(rf, cf), hp.bc2);
              tr.y[k] = yk; tr.mp[k] = mpn; tr.u[k] = __fmul_rn(pn, inv);
            };
            if (one_row) {
              const float rf = rfac[tr.rw[0]], mu = hp.gc ? mean[tr.rw[0]] : 0.0f;
              float cf[8];
              ld8f(cfac + cl[0], 8, cf);  // the eight column factors: two vector loads where the address allows
              // the same chain on pairs (each lane of a packed instruction is the scalar IEEE operation)
              const f32x2 FW = pack2(hp.fw, hp.fw), FB = pack2(hp.fb, hp.fb), C1 = pack2(hp.c1, hp.c1);
              const f32x2 C2 = pack2(hp.c2, hp.c2), C3 = pack2(hp.c3, hp.c3), BC2 = pack2(hp.bc2, hp.bc2);
              const f32x2 RF = pack2(rf, rf), MUN = pack2(-mu, -mu);
  #pragma unroll
              for (int j = 0; j < 4; ++j) {
                f32x2 y2 = pack2(gx[2 * j], gx[2 * j + 1]);
                if (hp.gc) {
                  y2 = add2(y2, MUN);
                  if constexpr (E::IS_BF16) {
                    const uint32_t w = pack_bf16_rn(y2.x, y2.y);
                    y2 = pack2(bf16lo(w), bf16hi(w));
                  }
                }
                const f32x2 mp2 = fma2(y2, FW, mul2(pack2(mpo[2 * j], mpo[2 * j + 1]), FB));
                const f32x2 pn2 = mul2(fma2(pack2(mno[2 * j], mno[2 * j + 1]), C2, mul2(mp2, C1)), C3);
                const f32x2 inv2 = mul2(mul2(RF, pack2(cf[2 * j], cf[2 * j + 1])), BC2);
                const f32x2 u2 = mul2(pn2, inv2);
                tr.y[2 * j] = y2.x; tr.y[2 * j + 1] = y2.y;
                tr.mp[2 * j] = mp2.x; tr.mp[2 * j + 1] = mp2.y;
                tr.u[2 * j] = u2.x; tr.u[2 * j + 1] = u2.y;
              }
            } else {
  #pragma unroll
              for (int k = 0; k < 8; ++k) {
                tr.y[k] = 0.0f; tr.mp[k] = 0.0f; tr.u[k] = 0.0f;
                if (k < cnt) chain(k, rfac[tr.rw[k]], hp.gc ? mean[tr.rw[k]] : 0.0f, cfac[cl[k]]);
              }
            }
          } else {
  #pragma unroll
            for (int k = 0; k < 8; ++k) { tr.y[k] = 0.0f; tr.mp[k] = 0.0f; tr.u[k] = 0.0f; tr.rw[k] = 0; }
          }
          if constexpr (!APPLY) {
            float s8 = 0.0f;  // the trip's eight squares in fp32, then one wide addition
  #pragma unroll
            for (int k = 0; k < 8; ++k) if (k < cnt) {
              s8 = __fmaf_rn(tr.u[k], tr.u[k], s8);
              kept += (__fmul_rn(tr.u[k], tr.y[k]) > 0.0f) ? 1u : 0u;
            }
            ss += (double)s8;
            if constexpr (MK == KAON_M_INT8) {
              int cr = -1;
              float mx = 0.0f;
  #pragma unroll
              for (int k = 0; k < 8; ++k) if (k < cnt) {
                if (tr.rw[k] != cr) {
                  if (cr >= 0) atomicMax(rowmax + cr, __float_as_uint(mx));
                  cr = tr.rw[k];
                  mx = 0.0f;
                }
                mx = fmaxf(mx, fabsf(tr.mp[k]));
              }
              if (cr >= 0) atomicMax(rowmax + cr, __float_as_uint(mx));
            }
          } else {
            if (cnt > 0) pnm_write<PT>(hp, d, tr, e, cnt, div, denom, s_upd, &pv.peers);
            pnm_store_m<MK>(pos, psc, tr, e, cnt, bsh, lane,
                            [&](int r) { return __uint_as_float(__ldcg(rowmax + r)); });
          }
        };
        if (__all_sync(0xffffffffu, cnt_rt == 8 && c0 + 8 <= C)) trip(std::true_type{});
        else trip(std::false_type{});
      }
    }
    if constexpr (!APPLY) {
      // the item's partial sums, lanes then warps in order
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
        kept += __shfl_xor_sync(0xffffffffu, kept, o);
      }
      __syncthreads();
      if (lane == 0) { red_d[warp] = ss; red_u[warp] = kept; }
      __syncthreads();
      if (tid == 0) {
        double s = 0.0;
        unsigned kk = 0;
        for (int w = 0; w < PT_THREADS / 32; ++w) { s += red_d[w]; kk += red_u[w]; }
        x.part[it] = s;
        x.kpart[it] = kk;
      }
    }
  }
}

// int8 momentum: before SUM, zero the row maxima and set the positive buffer's row scales aside.
__global__ void __launch_bounds__(PT_THREADS) pnm_prep_kernel(PlanView pv, PnmDev hp, PnmView x) {
  const int ti = x.fact[blockIdx.x];
  if (pv.grads[ti] == nullptr) return;
  const DevTensor d = pv.tensors[ti];
  unsigned* rowmax = reinterpret_cast<unsigned*>(pv.aux + aux_rowmax(d));
  float* oldsc = pv.aux + aux_oldsc(d);
  const float* psc = x.bufs[ti].sc[hp.swap];
  for (int r = threadIdx.x; r < d.rows; r += PT_THREADS) { rowmax[r] = 0u; oldsc[r] = psc[r]; }
}

// One CTA per factored tensor: item partials in item order -> clip divisor, cautious denominator.
__global__ void __launch_bounds__(PT_THREADS) pnm_reduce_kernel(PlanView pv, PnmDev hp, PnmView x) {
  __shared__ double red_d[PT_THREADS];
  __shared__ unsigned red_u[PT_THREADS];
  const int ti = x.fact[blockIdx.x];
  if (pv.grads[ti] == nullptr) return;
  const DevTensor d = pv.tensors[ti];
  const int b0 = x.item_begin[ti], b1 = x.item_begin[ti + 1];
  // thread j takes the contiguous run of items [b0 + j*per, ...): the order of the additions is fixed
  const int per = (b1 - b0 + PT_THREADS - 1) / PT_THREADS;
  double s = 0.0;
  unsigned kk = 0;
  for (int i = b0 + threadIdx.x * per; i < min(b1, b0 + (threadIdx.x + 1) * per); ++i) { s += x.part[i]; kk += x.kpart[i]; }
  red_d[threadIdx.x] = s;
  red_u[threadIdx.x] = kk;
  __syncthreads();
  if (threadIdx.x == 0) {
    double tot = 0.0;
    unsigned kept = 0;
    for (int j = 0; j < PT_THREADS; ++j) { tot += red_d[j]; kept += red_u[j]; }
    const float rms = __fdiv_rn((float)sqrt(tot), (float)sqrt((double)d.numel));
    x.scal[2 * ti] = hp.clip_on ? fmaxf(__fdiv_rn(rms, hp.clip), 1.0f) : 1.0f;
    x.scal[2 * ti + 1] = fmaxf(__fdiv_rn((float)kept, (float)d.numel), 1e-8f);
    pv.kept[ti] = kept;
  }
}

// ----------------------------------------------------------------------------- 1-D tensors

// reference src/kaon/adapnm.py:1126-1172 / 1238-1249: full second moment v (optionally its running
// maximum), eps on the denominator.  One CTA per tensor, any length: a first sweep updates v and takes
// the tensor-wide sums, a second one recomputes the chain and writes.
template <typename PT, int MK>
__global__ void __launch_bounds__(PT_THREADS) pnm_flat_kernel(PlanView pv, PnmDev hp, PnmView x) {
  using E = Elems<PT>;
  __shared__ double red_d[PT_THREADS / 32];
  __shared__ unsigned red_u[PT_THREADS / 32];
  __shared__ float red_f[PT_THREADS / 32];
  __shared__ float bc_s[3];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int ti = x.flat[blockIdx.x];
  const unsigned char* g = reinterpret_cast<const unsigned char*>(pv.grads[ti]);
  if (g == nullptr) return;
  const DevTensor d = pv.tensors[ti];
  const PnmBufs b = x.bufs[ti];
  void* pos = b.m[hp.swap];
  float* psc = b.sc[hp.swap];
  const void* neg = b.m[hp.swap ^ 1];
  const float* nsc = b.sc[hp.swap ^ 1];
  const int bsh = d.bshift;  // 4-bit: element -> block shift (31: one block)
  const long long n = d.numel;
  const long long nvec = (n + 7) >> 3;
  float* v = d.stat_a;
  float* max_v = hp.ams ? b.max_v : nullptr;
  const SrStream s_upd{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_UPDATE};
  // int8: one scalar scale; every thread keeps the old one before anything is written
  __shared__ float old_sc_s;
  const bool one_scale = MK == KAON_M_INT8 || (MK == KAON_M_4BIT && bsh >= 31);
  if (tid == 0) old_sc_s = one_scale ? psc[0] : 0.0f;
  __syncthreads();
  const float old_sc = old_sc_s;
  const float* psc_rd = one_scale ? &old_sc : psc;

  auto chain = [&](long long e, int cnt, bool first_sweep, PnmTrip& tr) {
    float gx[8], vv[8], mx[8], mpo[8], mno[8];
    load8_guard<PT>(g + e * E::BYTES, cnt, gx);
    ld8f(v + e, cnt, vv);
    if (max_v != nullptr) ld8f(max_v + e, cnt, mx);
#pragma unroll
    for (int k = 0; k < 8; ++k) tr.rw[k] = 0;
    pnm_decode8<MK>(pos, psc_rd, e, cnt, tr.rw, bsh, mpo);
    pnm_decode8<MK>(neg, nsc, e, cnt, tr.rw, bsh, mno);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      tr.y[k] = 0.0f; tr.mp[k] = 0.0f; tr.u[k] = 0.0f;
      if (k < cnt) {
        const float yk = gx[k];
        if (first_sweep) {
          vv[k] = __fmaf_rn(__fmul_rn(hp.fw2, yk), yk, __fmul_rn(vv[k], hp.fb2));
          if (max_v != nullptr) mx[k] = fmaxf(mx[k], vv[k]);
        }
        const float vd = max_v != nullptr ? mx[k] : vv[k];
        const float den = __fdiv_rn(__fadd_rn(__fsqrt_rn(__fadd_rn(vd, 1e-15f)), hp.eps), hp.bc2);
        const float mpn = __fmaf_rn(yk, hp.fw, __fmul_rn(mpo[k], hp.fb));
        const float pn = __fmul_rn(__fmaf_rn(mno[k], hp.c2, __fmul_rn(mpn, hp.c1)), hp.c3);
        tr.y[k] = yk; tr.mp[k] = mpn; tr.u[k] = __fdiv_rn(pn, den);
      }
    }
    if (first_sweep) {
      st8f(v + e, cnt, vv);
      if (max_v != nullptr) st8f(max_v + e, cnt, mx);
    }
  };

  double ss = 0.0;
  unsigned kept = 0;
  float amax = 0.0f;
  for (long long v0 = 0; v0 < nvec; v0 += PT_THREADS) {
    const long long vi = v0 + tid;
    const long long e = vi * 8;
    const int cnt = vi < nvec ? (int)min(8ll, n - e) : 0;
    if (cnt > 0) {
      PnmTrip tr;
      chain(e, cnt, true, tr);
#pragma unroll
      for (int k = 0; k < 8; ++k) if (k < cnt) {
        ss += (double)tr.u[k] * (double)tr.u[k];
        kept += (__fmul_rn(tr.u[k], tr.y[k]) > 0.0f) ? 1u : 0u;
        amax = fmaxf(amax, fabsf(tr.mp[k]));
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ss += __shfl_xor_sync(0xffffffffu, ss, o);
    kept += __shfl_xor_sync(0xffffffffu, kept, o);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  }
  if (lane == 0) { red_d[warp] = ss; red_u[warp] = kept; red_f[warp] = amax; }
  __syncthreads();  // also: every write of v / max_v by this CTA is visible to it from here on
  if (tid == 0) {
    double tot = 0.0;
    unsigned kk = 0;
    float am = 0.0f;
    for (int w = 0; w < PT_THREADS / 32; ++w) { tot += red_d[w]; kk += red_u[w]; am = fmaxf(am, red_f[w]); }
    const float rms = __fdiv_rn((float)sqrt(tot), (float)sqrt((double)n));
    bc_s[0] = hp.clip_on ? fmaxf(__fdiv_rn(rms, hp.clip), 1.0f) : 1.0f;
    bc_s[1] = fmaxf(__fdiv_rn((float)kk, (float)n), 1e-8f);
    bc_s[2] = am;
    pv.kept[ti] = kk;
  }
  __syncthreads();
  const float div = bc_s[0], denom = bc_s[1], tmax = bc_s[2];
  for (long long v0 = 0; v0 < nvec; v0 += PT_THREADS) {
    const long long vi = v0 + tid;
    const long long e = vi * 8;
    const int cnt = vi < nvec ? (int)min(8ll, n - e) : 0;
    PnmTrip tr;
    tr.first = 0u;
    if (cnt > 0) {
      chain(e, cnt, false, tr);
      pnm_write<PT>(hp, d, tr, e, cnt, div, denom, s_upd, &pv.peers);
    }
    pnm_store_m<MK>(pos, psc, tr, e, cnt, bsh, lane, [&](int) { return tmax; },
                    (MK == KAON_M_4BIT && bsh >= 31) ? tmax : -1.0f);
  }
  if constexpr (MK == KAON_M_INT8 || MK == KAON_M_4BIT) {
    // the one scale of the tensor (int8, or a 4-bit block that covers it), once every thread has decoded with the old one
    __syncthreads();
    if (tid == 0 && (MK == KAON_M_INT8 || bsh >= 31)) psc[0] = __fdiv_rn(fmaxf(tmax, 1e-12f), MK == KAON_M_INT8 ? 127.0f : 7.0f);
  }
}

// ----------------------------------------------------------------------------- host

struct PnmHost {
  PnmView view{};
  void* block = nullptr;
  Task* d_stats = nullptr;   // STATS items the small-CTA launch takes, or null
  Task* d_final = nullptr;   // the other STATS items and the FINAL items, for the persistent kernel
  int n_stats = 0, n_final = 0;
  bool attached = false;
  int64_t bytes = 0;
};

typedef void (*PnmPass)(PlanView, PnmDev, PnmView);

template <typename PT, bool APPLY>
static PnmPass pick_pass_pt(int mk) {
  switch (mk) {
    case KAON_M_F32: return pnm_pass_kernel<PT, KAON_M_F32, APPLY>;
    case KAON_M_BF16: return pnm_pass_kernel<PT, KAON_M_BF16, APPLY>;
    case KAON_M_INT8: return pnm_pass_kernel<PT, KAON_M_INT8, APPLY>;
    case KAON_M_4BIT: return pnm_pass_kernel<PT, KAON_M_4BIT, APPLY>;
    default: return nullptr;
  }
}
template <typename PT>
static PnmPass pick_flat_pt(int mk) {
  switch (mk) {
    case KAON_M_F32: return pnm_flat_kernel<PT, KAON_M_F32>;
    case KAON_M_BF16: return pnm_flat_kernel<PT, KAON_M_BF16>;
    case KAON_M_INT8: return pnm_flat_kernel<PT, KAON_M_INT8>;
    case KAON_M_4BIT: return pnm_flat_kernel<PT, KAON_M_4BIT>;
    default: return nullptr;
  }
}

void pnm_free(kaon_plan* pl) {
  PnmHost* h = reinterpret_cast<PnmHost*>(pl->pnm);
  if (!h) return;
  cudaFree(h->block);
  delete h;
  pl->pnm = nullptr;
}

// Lists, partial-sum buffers and the table of the second momentum, built by kaon_adapnm_attach.
static int pnm_build(kaon_plan* pl, const void* const* m_neg, float* const* m_neg_scale, float* const* max_v) {
  pnm_free(pl);
  PnmHost* h = new PnmHost();
  pl->pnm = h;
  const int n = pl->n_tensors;
  std::vector<Task> items, stats, fin;
  std::vector<int> begin(n + 1, 0), fact, flat;
  std::vector<PnmBufs> bufs(n);
  for (int i = 0; i < n; ++i) {
    const DevTensor& t = pl->h_tensors[i];
    begin[i] = (int)items.size();
    bufs[i].m[0] = t.m; bufs[i].sc[0] = t.m_scale;
    bufs[i].m[1] = const_cast<void*>(m_neg[i]);
    bufs[i].sc[1] = m_neg_scale ? m_neg_scale[i] : nullptr;
    bufs[i].max_v = max_v ? max_v[i] : nullptr;
    if (t.numel == 0) continue;
    if (!m_neg[i]) return fail(KAON_E_INVALID, "kaon_adapnm_attach: tensor %d has no second momentum", i);
    if ((uintptr_t)m_neg[i] & 15) return fail(KAON_E_INVALID, "kaon_adapnm_attach: tensor %d: second momentum not 16-byte aligned", i);
    if ((pl->momentum_kind == KAON_M_INT8 || pl->momentum_kind == KAON_M_4BIT) && !bufs[i].sc[1])
      return fail(KAON_E_INVALID, "kaon_adapnm_attach: tensor %d: scales of the second momentum missing", i);
    if (t.rows <= 0) { flat.push_back(i); continue; }
    fact.push_back(i);
    for (long long e = 0; e < t.numel; e += PNM_ITEM)
      items.push_back(Task{i, PH_ADA_APPLY, e, (int)std::min<long long>(PNM_ITEM, t.numel - e), 0, 0, 0});
  }
  begin[n] = (int)items.size();
  {
    std::vector<Task> hm((size_t)pl->n_tasks_main);
    KAON_CUDA(cudaMemcpy(hm.data(), pl->d_tasks_main, sizeof(Task) * hm.size(), cudaMemcpyDeviceToHost));
    // STATS items the small-CTA launch can take go there, the others stay with FINAL in the persistent
    // kernel (which stages whole rows, so it cannot take rows longer than a work item)
    const bool bf16 = pl->param_dtype == KAON_DT_BF16;
    for (const Task& t : hm) {
      if (t.phase == PH_ADA_STATS) {
        if (bf16 && stats_item_ok(pl, t)) stats.push_back(t);
        else if (pl->h_tensors[t.tensor].cols > CAP)
          return fail(KAON_E_UNSUPPORTED, "AdaPNM: tensor %d: rows longer than %d elements need bf16 weights and a row length that is a multiple of 8", t.tensor, CAP);
        else fin.push_back(t);
      } else if (t.phase == PH_ADA_FINAL) {
        fin.push_back(t);
      }
    }
  }
  auto up = [](size_t b) { return (b + 255) / 256 * 256; };
  size_t o = 0;
  auto take = [&](size_t b) { size_t r = o; o += up(b); return r; };
  const size_t o_items = take(sizeof(Task) * items.size()), o_begin = take(sizeof(int) * (n + 1));
  const size_t o_bufs = take(sizeof(PnmBufs) * n), o_part = take(sizeof(double) * items.size());
  const size_t o_kpart = take(sizeof(unsigned) * items.size()), o_scal = take(sizeof(float) * 2 * n);
  const size_t o_fact = take(sizeof(int) * fact.size()), o_flat = take(sizeof(int) * flat.size());
  const size_t o_stats = take(sizeof(Task) * stats.size());
  const size_t o_fin = take(sizeof(Task) * fin.size());
  KAON_CUDA(cudaMalloc(&h->block, std::max<size_t>(o, 256)));
  unsigned char* base = reinterpret_cast<unsigned char*>(h->block);
  h->bytes = (int64_t)o;
  auto put = [&](size_t off, const void* src, size_t b) -> cudaError_t {
    return b ? cudaMemcpy(base + off, src, b, cudaMemcpyHostToDevice) : cudaSuccess;
  };
  KAON_CUDA(put(o_items, items.data(), sizeof(Task) * items.size()));
  KAON_CUDA(put(o_begin, begin.data(), sizeof(int) * (n + 1)));
  KAON_CUDA(put(o_bufs, bufs.data(), sizeof(PnmBufs) * n));
  KAON_CUDA(put(o_fact, fact.data(), sizeof(int) * fact.size()));
  KAON_CUDA(put(o_flat, flat.data(), sizeof(int) * flat.size()));
  KAON_CUDA(put(o_stats, stats.data(), sizeof(Task) * stats.size()));
  KAON_CUDA(put(o_fin, fin.data(), sizeof(Task) * fin.size()));
  KAON_CUDA(cudaMemset(base + o_scal, 0, sizeof(float) * 2 * n));
  PnmView& x = h->view;
  x.items = reinterpret_cast<const Task*>(base + o_items); x.n_items = (int)items.size();
  x.item_begin = reinterpret_cast<const int*>(base + o_begin);
  x.bufs = reinterpret_cast<const PnmBufs*>(base + o_bufs);
  x.part = reinterpret_cast<double*>(base + o_part);
  x.kpart = reinterpret_cast<unsigned*>(base + o_kpart);
  x.scal = reinterpret_cast<float*>(base + o_scal);
  x.fact = reinterpret_cast<const int*>(base + o_fact); x.n_fact = (int)fact.size();
  x.flat = reinterpret_cast<const int*>(base + o_flat); x.n_flat = (int)flat.size();
  h->d_stats = stats.empty() ? nullptr : reinterpret_cast<Task*>(base + o_stats); h->n_stats = (int)stats.size();
  h->d_final = reinterpret_cast<Task*>(base + o_fin); h->n_final = (int)fin.size();
  h->attached = true;
  pl->device_bytes += h->bytes;
  return KAON_OK;
}

}  // namespace kaon

using namespace kaon;

extern "C" int kaon_adapnm_attach(kaon_plan* pl, const void* const* m_neg, float* const* m_neg_scale,
                                  float* const* max_v, int n) {
  if (!pl || !m_neg) return fail(KAON_E_INVALID, "kaon_adapnm_attach: null argument");
  if (pl->optimizer != KAON_OPT_ADAPNM) return fail(KAON_E_INVALID, "plan was not built for AdaPNM");
  if (n != pl->n_tensors) return fail(KAON_E_INVALID, "kaon_adapnm_attach: %d pointers for a plan of %d tensors", n, pl->n_tensors);
  if (int rc = check_device(pl)) return rc;
  pl->pnm_has_max_v = max_v != nullptr;
  if (max_v)
    for (int i = 0; i < n; ++i)
      if (pl->h_tensors[i].rows <= 0 && pl->h_tensors[i].numel > 0 && !max_v[i]) pl->pnm_has_max_v = false;
  return pnm_build(pl, m_neg, m_neg_scale, max_v);
}

extern "C" int kaon_adapnm_step(kaon_plan* pl, const kaon_adapnm_hparams* h, uint64_t seed, uint32_t step,
                                void* stream) {
  if (!pl || !h) return fail(KAON_E_INVALID, "kaon_adapnm_step: null argument");
  if (pl->optimizer != KAON_OPT_ADAPNM) return fail(KAON_E_INVALID, "plan was not built for AdaPNM");
  if (int rc = check_device(pl)) return rc;
  PnmHost* ph = reinterpret_cast<PnmHost*>(pl->pnm);
  if (!ph || !ph->attached) return fail(KAON_E_INVALID, "kaon_adapnm_step: call kaon_adapnm_attach first (the second momentum)");
  if (pl->momentum_kind == KAON_M_NONE) return fail(KAON_E_INVALID, "AdaPNM needs its two momenta");
  if (h->bf16_method < KAON_W_NONE || h->bf16_method > KAON_W_KAHAN) return fail(KAON_E_UNSUPPORTED, "bf16_method %d", h->bf16_method);
  if (int rc = check_kahan(pl, h->bf16_method)) return rc;
  if (h->group_step < 1) return fail(KAON_E_INVALID, "group_step is the 1-based step count of the parameter group");
  if (h->ams_bound && ph->view.n_flat > 0 && !pl->pnm_has_max_v)
    return fail(KAON_E_INVALID, "ams_bound: the 1-D tensors need their max_v buffers (kaon_adapnm_attach)");
  const double b1 = h->beta1, b2 = h->beta2, b0 = h->beta0, t = (double)h->group_step;
  const double b1sq = b1 * b1, nn = std::sqrt((1.0 + b0) * (1.0 + b0) + b0 * b0);
  const double bc1 = 1.0 - std::pow(b1, t), bc2 = std::sqrt(1.0 - std::pow(b2, t));
  PnmDev hp{};
  hp.fb = (float)b1sq; hp.fw = (float)(1.0 - b1sq);
  hp.c1 = (float)(1.0 + b0); hp.c2 = (float)(-b0); hp.c3 = (float)(1.0 / nn);
  hp.bc2 = (float)bc2; hp.fstep = (float)(h->lr / bc1);
  hp.wdsc = (float)(1.0 - h->lr * h->weight_decay); hp.has_wd = h->weight_decay != 0.0;
  hp.fb2 = (float)b2; hp.fw2 = (float)(1.0 - b2); hp.eps = (float)h->eps;
  hp.clip = (float)h->clip_threshold; hp.clip_on = h->clip_threshold > 0.0;
  hp.cautious = h->cautious != 0; hp.gc = h->gradient_centralization != 0; hp.ams = h->ams_bound != 0;
  hp.sr = h->bf16_method == KAON_W_SR && pl->param_dtype == KAON_DT_BF16;
  hp.kahan = h->bf16_method == KAON_W_KAHAN && pl->param_dtype == KAON_DT_BF16;
  hp.swap = (h->group_step & 1u) ? 0 : 1;  // odd steps: "m_pos" is positive
  hp.step = step; hp.k0 = (uint32_t)seed; hp.k1 = (uint32_t)(seed >> 32);
  cudaStream_t s = (cudaStream_t)stream;
  const bool bf = pl->param_dtype == KAON_DT_BF16;
  const int mk = pl->momentum_kind;
  const PnmView& x = ph->view;
  // 1. second moment of the factored tensors: Adakaon's STATS and FINAL items
  if (x.n_fact > 0) {
    AdaDev ad{};
    ad.w2 = (float)(1.0 - b2); ad.w2m1 = ad.w2 - 1.0f; ad.small_w2 = ad.w2 < 0.5f;
    ad.w1 = 1.0f; ad.eps1 = (float)h->eps; ad.has_eps = h->eps > 0.0; ad.clip = 1.0f;
    ad.gc = hp.gc; ad.step = step; ad.k0 = hp.k0; ad.k1 = hp.k1;
    PlanView v = pl->view;
    KAON_CUDA(cudaMemsetAsync(v.task_counter, 0, pl->counters_bytes - sizeof(unsigned), s));
    if (ph->d_stats != nullptr)
      if (int rc = launch_stats_tasks(pl, pl->view, ad, ph->d_stats, ph->n_stats, s)) return rc;
    v.tasks = ph->d_final; v.n_tasks = ph->n_final;
    // the variant the plan's launch configuration was made for (STATS and FINAL do not depend on the momentum kind)
    AdaKernel k = pick_ada(pl->param_dtype, pl->momentum_kind, false);
    k<<<pl->grid, ADA_THREADS, pl->smem_bytes, s>>>(v, ad, (int)x_offset_rows(pl) | (pl->double_buffer ? 1 : 0));
    KAON_CUDA(cudaGetLastError());
    pl->launches += 1;
    // 2-4. the two sweeps over the flat items
    const int grid = std::min(x.n_items, pl->sm_count * 8);
    if (mk == KAON_M_INT8) {
      pnm_prep_kernel<<<x.n_fact, PT_THREADS, 0, s>>>(pl->view, hp, x);
      pl->launches += 1;
    }
    PnmPass sum = bf ? pick_pass_pt<__nv_bfloat16, false>(mk) : pick_pass_pt<float, false>(mk);
    PnmPass app = bf ? pick_pass_pt<__nv_bfloat16, true>(mk) : pick_pass_pt<float, true>(mk);
    if (!sum || !app) return fail(KAON_E_INVALID, "no AdaPNM kernel for this dtype combination");
    sum<<<grid, PT_THREADS, 0, s>>>(pl->view, hp, x);
    pnm_reduce_kernel<<<x.n_fact, PT_THREADS, 0, s>>>(pl->view, hp, x);
    app<<<grid, PT_THREADS, 0, s>>>(pl->view, hp, x);
    KAON_CUDA(cudaGetLastError());
    pl->launches += 3;
  }
  if (x.n_flat > 0) {
    PnmPass fl = bf ? pick_flat_pt<__nv_bfloat16>(mk) : pick_flat_pt<float>(mk);
    if (!fl) return fail(KAON_E_INVALID, "no AdaPNM kernel for this dtype combination");
    fl<<<x.n_flat, PT_THREADS, 0, s>>>(pl->view, hp, x);
    KAON_CUDA(cudaGetLastError());
    pl->launches += 1;
  }
  return KAON_OK;
}
