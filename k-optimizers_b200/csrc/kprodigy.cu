// KProdigy (Prodigy's distance estimate over kaon's memory backend) on the plan machinery.  Replaces
// reference src/kaon/kprodigy.py:417-703 (pass 1: the D statistics, the d-scaled momentum EMA, the second
// moment) and :706-949 (pass 2: the weight update).  The estimate itself - one scalar over every tensor of
// a scope, kprodigy.py:299-404 - stays on the host between the two calls, as in the reference.
//
// Pass 1 of a plan:
//   factored second moment: Adakaon's STATS and FINAL items (row / column EMA of g^2 + eps_factored, the
//     factors r_i, c_j and the centralisation means into the scratch); full second moment with gradient
//     centralisation: a row-mean launch (one warp per row) into the same scratch slot
//   SWEEP over flat items of 8192 elements of EVERY tensor: the centralised gradient (plus coupled weight
//     decay), on every slice_p-th element the numerator term g*(p0 - p) and the s buffer with its |s| sum
//     (per item, double, added per tensor in item order), the momentum through its codec (int8: only the
//     row maxima here, the codes in a second sweep), the full second moment v
//   the per-tensor partial sums are copied to the host, which folds them in fp32 in tensor order.
// Pass 2: [COUNT sweep + per-tensor reduce for the cautious mask] and the weight sweep.
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <vector>

#include "adakaon_dev.h"
#include "kaon_device.cuh"
#include "kaon_elem.cuh"
#include "kaon_host.h"
#include "kaon_ops.cuh"

namespace kaon {

constexpr int KP_ITEM = 16384;
constexpr int KP_THREADS = 256;

struct KpDev {
  // pass 1
  float fb1, ft, ftb, fd, w1, w1m1;   // beta1, d*(1-beta1) (and rounded to bf16), d, 1-beta1 (4-bit lerp)
  float fb2, fv;                      // beta2, d*d*(1-beta2)
  float fb3, fa;                      // beta3, alpha_s
  float fwd;                          // coupled weight decay
  int small_w1, d_is_one, do_d, has_wdc, gc, factored, has_m;
  long long slice_p;
  // pass 2
  float floor_, cap, fdlr, fdecay;    // d*eps, 1/(d*eps), dlr, decay*dlr
  int has_decay, cautious, sr, kahan, store;  // store: the int8 second sweep of pass 1
  uint32_t step, k0, k1;
};

struct KpBufs {
  float* s;
  const float* p0;   // null: the zero reference point
};

struct KpView {
  const Task* items;      // flat items of every tensor, tensor by tensor
  int n_items;
  const int* item_begin;  // [n_tensors + 1]
  const KpBufs* bufs;     // [n_tensors]
  double* part;           // [n_items][2]: numerator term, |s| sum; pass 2: [n_items] kept counts as doubles
  float* sums;            // [n_tensors][2] per-tensor sums (pass 1), [n_tensors] cautious denominators (pass 2)
  unsigned* tmax;         // [n_tensors] 1-D int8: bits of the tensor's absmax of the new momentum
  float* told;            // [n_tensors] 1-D int8: the scalar scale before this step
  const int* fact;        // indices of the >=2-D tensors
  int n_fact;
  const long long* row_begin;  // [n_fact + 1] rows before each >=2-D tensor
  long long n_rows;
};

// ----------------------------------------------------------------------------- row means (full second moment)

template <typename PT>
__global__ void __launch_bounds__(KP_THREADS) kp_rowmean_kernel(PlanView pv, KpView x) {
  using E = Elems<PT>;
  const int lane = threadIdx.x & 31;
  const long long warp0 = ((long long)blockIdx.x * KP_THREADS + threadIdx.x) >> 5;
  const long long nwarps = ((long long)gridDim.x * KP_THREADS) >> 5;
  for (long long gr = warp0; gr < x.n_rows; gr += nwarps) {
    int lo = 0, hi = x.n_fact - 1;   // the tensor this row belongs to
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (x.row_begin[mid] <= gr) lo = mid; else hi = mid - 1;
    }
    const int ti = x.fact[lo];
    const unsigned char* g = reinterpret_cast<const unsigned char*>(pv.grads[ti]);
    if (g == nullptr) continue;
    const DevTensor d = pv.tensors[ti];
    const long long r = gr - x.row_begin[lo];
    const unsigned char* rowp = g + (size_t)r * d.cols * E::BYTES;
    float s = 0.0f;
    for (int i = lane; i < d.cols; i += 32) s += E::load1(rowp, i);
    s = warp_sum(s);
    if (lane == 0) {
      const float mean = __fdiv_rn(s, (float)d.cols);
      pv.aux[aux_mean(d) + r] = E::IS_BF16 ? round_bf16(mean) : mean;
    }
  }
}

// int8 momentum: zero the maxima and set the scales of before this step aside (>=2-D: per row in the
// tensor's scratch; 1-D: one word each in the plan's own arrays).
__global__ void __launch_bounds__(KP_THREADS) kp_prep_kernel(PlanView pv, KpView x) {
  const int ti = blockIdx.x;
  if (pv.grads[ti] == nullptr) return;
  const DevTensor d = pv.tensors[ti];
  if (d.numel == 0) return;
  if (d.rows <= 0) {
    if (threadIdx.x == 0) { x.tmax[ti] = 0u; x.told[ti] = d.m_scale[0]; }
    return;
  }
  unsigned* rowmax = reinterpret_cast<unsigned*>(pv.aux + aux_rowmax(d));
  float* oldsc = pv.aux + aux_oldsc(d);
  for (int r = threadIdx.x; r < d.rows; r += KP_THREADS) { rowmax[r] = 0u; oldsc[r] = d.m_scale[r]; }
}

// ----------------------------------------------------------------------------- the sweeps

// MODE 0: pass 1 (statistics, moments).  MODE 1: pass 1's second sweep for int8 (codes and scales).
// MODE 2: pass 2 COUNT (cautious kept count).  MODE 3: pass 2 weight write.
template <typename PT, int MK, int MODE>
__global__ void __launch_bounds__(KP_THREADS, 4) kp_sweep_kernel(PlanView pv, KpDev hp, KpView x) {
  using E = Elems<PT>;
  __shared__ double red_a[KP_THREADS / 32], red_b[KP_THREADS / 32];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const SrStream s_upd{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_UPDATE};
  for (int it = blockIdx.x; it < x.n_items; it += gridDim.x) {
    const Task t = x.items[it];
    const DevTensor d = pv.tensors[t.tensor];
    const unsigned char* g = reinterpret_cast<const unsigned char*>(pv.grads[t.tensor]);
    double acc_a = 0.0, acc_b = 0.0;
    if (g != nullptr) {
      const KpBufs b = x.bufs[t.tensor];
      const bool two_d = d.rows > 0;
      const int C = two_d ? d.cols : 1;
      const bool gc = hp.gc && two_d;
      const bool fac = hp.factored && two_d;
      const float* mean = pv.aux + (two_d ? aux_mean(d) : 0);
      const float* rfac = pv.aux + (two_d ? aux_rfac(d) : 0);
      const float* cfac = pv.aux + (two_d ? aux_cfac(d) : 0);
      unsigned* rowmax = two_d ? reinterpret_cast<unsigned*>(pv.aux + aux_rowmax(d)) : x.tmax + t.tensor;
      // int8: the scales as they were before this step
      const float* msc_rd = MK == KAON_M_INT8 ? (two_d ? pv.aux + aux_oldsc(d) : x.told + t.tensor) : d.m_scale;
      const int bsh = d.bshift;
      float denom = 1.0f;
      if (MODE == 3 && hp.cautious) denom = x.sums[t.tensor];
      const float rdenom = __frcp_rn(denom), rfd = __frcp_rn(hp.fd);
      const int nvec = (t.n + 7) >> 3;
      for (int v0 = 0; v0 < nvec; v0 += KP_THREADS) {
        const int v = v0 + tid;
        const long long e = t.e0 + (long long)v * 8;
        const int cnt = v < nvec ? min(8, (int)(t.e0 + t.n - e)) : 0;
        PnmTrip tr;   // y: gradient, mp: new momentum / numerator, u: delta, rw: row
        tr.first = 0u;
#pragma unroll
        for (int k = 0; k < 8; ++k) { tr.y[k] = 0.0f; tr.mp[k] = 0.0f; tr.u[k] = 0.0f; tr.rw[k] = 0; }
        float pw[8];
        if (cnt > 0) {
          float gx[8], mo[8], vv[8], sv[8], p0v[8];
          int cl[8];
          load8_guard<PT>(g + e * E::BYTES, cnt, gx);
          const bool need_p = MODE == 0 ? (hp.do_d || hp.has_wdc) : (MODE >= 2);
          if (need_p) load8_guard<PT>(reinterpret_cast<const unsigned char*>(d.p) + e * E::BYTES, cnt, pw);
          int r = 0, c = 0;
          if (two_d) {
            r = e < 0x100000000ll ? (int)((unsigned)e / (unsigned)C) : (int)(e / C);
            c = (int)(e - (long long)r * C);
          }
          // the common trip: eight elements of one row (or of a 1-D tensor)
          const bool one_row = cnt == 8 && (!two_d || c + 8 <= C);
          const int r0 = r;
          if (one_row) {
#pragma unroll
            for (int k = 0; k < 8; ++k) { tr.rw[k] = r; cl[k] = c + k; }
            if (two_d ? c == 0 : e == 0) tr.first = 1u;
          } else {
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              cl[k] = 0;
              if (k < cnt) {
                if (two_d) {
                  while (c >= C) { c -= C; ++r; }
                  if (c == 0) tr.first |= 1u << k;
                } else if (e + k == 0) {
                  tr.first |= 1u << k;
                }
                tr.rw[k] = r;
                cl[k] = c;
                ++c;
              }
            }
          }
          // the momentum: before the EMA in pass 1, as stored in pass 2
          const bool read_m = hp.has_m && MK != KAON_M_NONE;
          if (read_m) pnm_decode8<MK>(d.m, (MODE <= 1 && MK == KAON_M_INT8) ? msc_rd : d.m_scale, e, cnt, tr.rw, bsh, mo);
          const bool full_v = !fac;
          if (full_v && (MODE == 0 || MODE >= 2)) ld8f(d.stat_a + e, cnt, vv);
          const bool dstat = MODE == 0 && hp.do_d;
          const bool dense = hp.slice_p == 1;
          if (dstat && dense) {
            ld8f(b.s + e, cnt, sv);
            if (b.p0) ld8f(b.p0 + e, cnt, p0v);
          }
          int rp = -1;
          float rf = 0.0f, mu = 0.0f;
          if (one_row) {
            rp = r0;
            mu = gc ? mean[rp] : 0.0f;
            if (MODE >= 2 && fac) rf = rfac[rp];
          }
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            if (k >= cnt) continue;
            if (!one_row && tr.rw[k] != rp) {
              rp = tr.rw[k];
              mu = gc ? mean[rp] : 0.0f;
              if (MODE >= 2 && fac) rf = rfac[rp];
            }
            const float yraw = pnm_centered<PT>(gx[k], mu, gc);
            if constexpr (MODE <= 1) {
              const float y = hp.has_wdc ? __fmaf_rn(pw[k], hp.fwd, yraw) : yraw;
              tr.y[k] = y;
              if (dstat) {
                if (dense) {
                  const float pr = b.p0 ? p0v[k] : 0.0f;
                  acc_a += (double)__fmul_rn(y, __fsub_rn(pr, pw[k]));
                  sv[k] = __fmaf_rn(y, hp.fa, __fmul_rn(sv[k], hp.fb3));
                  acc_b += (double)fabsf(sv[k]);
                } else if (((e + k) % hp.slice_p) == 0) {
                  const long long j = (e + k) / hp.slice_p;
                  const float pr = b.p0 ? b.p0[j] : 0.0f;
                  acc_a += (double)__fmul_rn(y, __fsub_rn(pr, pw[k]));
                  const float sn = __fmaf_rn(y, hp.fa, __fmul_rn(b.s[j], hp.fb3));
                  b.s[j] = sn;
                  acc_b += (double)fabsf(sn);
                }
              }
              if (hp.has_m) {
                if constexpr (MK == KAON_M_BF16) {
                  tr.mp[k] = round_bf16(__fmaf_rn(round_bf16(y), hp.ftb, round_bf16(__fmul_rn(mo[k], hp.fb1))));
                } else if constexpr (MK == KAON_M_4BIT) {
                  tr.mp[k] = lerp_torch(mo[k], hp.d_is_one ? y : __fmul_rn(y, hp.fd), hp.w1, hp.w1m1, hp.small_w1 != 0);
                } else if constexpr (MK == KAON_M_INT8 || MK == KAON_M_F32) {
                  tr.mp[k] = __fmaf_rn(y, hp.ft, __fmul_rn(mo[k], hp.fb1));
                }
              }
              if (MODE == 0 && full_v)   // the full second moment (also every 1-D tensor)
                vv[k] = __fmaf_rn(__fmul_rn(hp.fv, y), y, __fmul_rn(vv[k], hp.fb2));
            } else {
              tr.y[k] = yraw;
              const float numer = read_m ? mo[k] : yraw;
              float dl;
              if (fac) {
                const float inv = fminf(div_by(__fmul_rn(rf, cfac[cl[k]]), hp.fd, rfd), hp.cap);
                dl = __fmul_rn(numer, inv);
              } else {
                dl = __fdiv_rn(numer, fmaxf(__fsqrt_rn(vv[k]), hp.floor_));
              }
              dl = __fmul_rn(dl, hp.fdlr);
              if (hp.has_decay) dl = __fmaf_rn(pw[k], hp.fdecay, dl);
              const bool keep = __fmul_rn(dl, yraw) > 0.0f;
              if (MODE == 2) { if (keep) acc_a += 1.0; }
              else if (hp.cautious) dl = keep ? div_by(dl, denom, rdenom) : 0.0f;
              tr.u[k] = dl;
            }
          }
          if (MODE == 0) {
            if (full_v) st8f(d.stat_a + e, cnt, vv);
            if (dstat && dense) st8f(b.s + e, cnt, sv);
          }
        }
        if constexpr (MODE == 0) {
          if (hp.has_m) {
            if constexpr (MK == KAON_M_INT8) {  // the row maxima first; the codes in the second sweep
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
            } else if constexpr (MK != KAON_M_NONE) {
              pnm_store_m<MK>(d.m, d.m_scale, tr, e, cnt, bsh, lane, [](int) { return 0.0f; });
            }
          }
        } else if constexpr (MODE == 1) {
          if constexpr (MK == KAON_M_INT8)
            pnm_store_m<MK>(d.m, d.m_scale, tr, e, cnt, bsh, lane, [&](int r) { return __uint_as_float(__ldcg(rowmax + r)); });
        } else if constexpr (MODE == 3) {
          if (cnt > 0) {
            uint32_t nz[4] = {0u, 0u, 0u, 0u};
            if (hp.sr) s_upd.draw8(d.tensor_id, (uint64_t)(e >> 3), nz);
            const bool kahan = E::IS_BF16 && hp.kahan;
            unsigned char* pe = reinterpret_cast<unsigned char*>(d.p) + e * E::BYTES;
            uint16_t* she = kahan ? reinterpret_cast<uint16_t*>(d.shift) + e : nullptr;
#pragma unroll
            for (int k = 0; k < 8; ++k) if (k < cnt) {
              float p0 = pw[k];
              if (kahan) {
                float sh = __uint_as_float((uint32_t)she[k] << 16);
                kahan_step(p0, sh, tr.u[k]);
                she[k] = (uint16_t)(__float_as_uint(sh) >> 16);
              } else {
                p0 = write_step_pnm<PT>(p0, tr.u[k], hp.sr != 0, noise_lane_pnm(nz, k));
              }
              pw[k] = p0;
            }
            if constexpr (E::IS_BF16) {
              if (cnt >= 8) {
                const uint4 out = make_uint4((__float_as_uint(pw[0]) >> 16) | (__float_as_uint(pw[1]) & 0xFFFF0000u),
                                             (__float_as_uint(pw[2]) >> 16) | (__float_as_uint(pw[3]) & 0xFFFF0000u),
                                             (__float_as_uint(pw[4]) >> 16) | (__float_as_uint(pw[5]) & 0xFFFF0000u),
                                             (__float_as_uint(pw[6]) >> 16) | (__float_as_uint(pw[7]) & 0xFFFF0000u));
                *reinterpret_cast<uint4*>(pe) = out;
                mirror16(&pv.peers, pe, out);
              } else {
#pragma unroll
                for (int k = 0; k < 8; ++k) if (k < cnt) reinterpret_cast<uint16_t*>(pe)[k] = (uint16_t)(__float_as_uint(pw[k]) >> 16);
                mirror_copy(&pv.peers, pe, cnt * 2);
              }
            } else {
              float* pf = reinterpret_cast<float*>(pe);
#pragma unroll
              for (int k = 0; k < 8; ++k) if (k < cnt) pf[k] = pw[k];
              mirror_copy(&pv.peers, pf, cnt * 4);
            }
          }
        }
      }
    }
    if constexpr (MODE == 0 || MODE == 2) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        acc_a += __shfl_xor_sync(0xffffffffu, acc_a, o);
        acc_b += __shfl_xor_sync(0xffffffffu, acc_b, o);
      }
      __syncthreads();
      if (lane == 0) { red_a[warp] = acc_a; red_b[warp] = acc_b; }
      __syncthreads();
      if (tid == 0) {
        double a = 0.0, bb = 0.0;
        for (int w = 0; w < KP_THREADS / 32; ++w) { a += red_a[w]; bb += red_b[w]; }
        x.part[2 * it] = a;
        x.part[2 * it + 1] = bb;
      }
    }
  }
}

// One CTA per tensor: item partials in item order.  COUNT = false: the two pass-1 sums as floats;
// COUNT = true: the kept count -> cautious denominator.
template <bool COUNT>
__global__ void __launch_bounds__(KP_THREADS) kp_reduce_kernel(PlanView pv, KpView x) {
  __shared__ double ra[KP_THREADS], rb[KP_THREADS];
  const int ti = blockIdx.x;
  const int b0 = x.item_begin[ti], b1 = x.item_begin[ti + 1];
  const int per = (b1 - b0 + KP_THREADS - 1) / KP_THREADS;
  double a = 0.0, b = 0.0;
  for (int i = b0 + threadIdx.x * per; i < min(b1, b0 + (threadIdx.x + 1) * per); ++i) { a += x.part[2 * i]; b += x.part[2 * i + 1]; }
  ra[threadIdx.x] = a;
  rb[threadIdx.x] = b;
  __syncthreads();
  if (threadIdx.x == 0) {
    double ta = 0.0, tb = 0.0;
    for (int j = 0; j < KP_THREADS; ++j) { ta += ra[j]; tb += rb[j]; }
    if (COUNT) {
      const DevTensor d = pv.tensors[ti];
      const unsigned kept = (unsigned)(ta + 0.5);
      x.sums[ti] = fmaxf(__fdiv_rn((float)kept, (float)max(d.numel, 1ll)), 1e-8f);
      pv.kept[ti] = kept;
    } else {
      x.sums[2 * ti] = (float)ta;
      x.sums[2 * ti + 1] = (float)tb;
    }
  }
}

// ----------------------------------------------------------------------------- host

struct KpHost {
  KpView view{};
  void* block = nullptr;
  Task* d_stats = nullptr;
  Task* d_final = nullptr;
  int n_stats = 0, n_final = 0;
  long long slice_p = 1;
  std::vector<float> h_sums;
  int64_t bytes = 0;
};

typedef void (*KpSweep)(PlanView, KpDev, KpView);

template <typename PT, int MODE>
static KpSweep pick_sweep_pt(int mk) {
  switch (mk) {
    case KAON_M_F32: return kp_sweep_kernel<PT, KAON_M_F32, MODE>;
    case KAON_M_BF16: return kp_sweep_kernel<PT, KAON_M_BF16, MODE>;
    case KAON_M_INT8: return kp_sweep_kernel<PT, KAON_M_INT8, MODE>;
    case KAON_M_4BIT: return kp_sweep_kernel<PT, KAON_M_4BIT, MODE>;
    case KAON_M_NONE: return kp_sweep_kernel<PT, KAON_M_NONE, MODE>;
    default: return nullptr;
  }
}
template <int MODE>
static KpSweep pick_sweep(int pdt, int mk) {
  return pdt == KAON_DT_BF16 ? pick_sweep_pt<__nv_bfloat16, MODE>(mk) : pick_sweep_pt<float, MODE>(mk);
}

void kp_free(kaon_plan* pl) {
  KpHost* h = reinterpret_cast<KpHost*>(pl->kp);
  if (!h) return;
  cudaFree(h->block);
  delete h;
  pl->kp = nullptr;
}

static int kp_build(kaon_plan* pl, float* const* s, const float* const* p0, long long slice_p) {
  kp_free(pl);
  KpHost* h = new KpHost();
  pl->kp = h;
  h->slice_p = slice_p;
  const int n = pl->n_tensors;
  std::vector<Task> items, stats, fin;
  std::vector<int> begin(n + 1, 0), fact;
  std::vector<long long> row_begin(1, 0);
  std::vector<KpBufs> bufs(n);
  for (int i = 0; i < n; ++i) {
    const DevTensor& t = pl->h_tensors[i];
    begin[i] = (int)items.size();
    bufs[i].s = s[i];
    bufs[i].p0 = p0 ? p0[i] : nullptr;
    if (t.numel == 0) continue;
    if (!s[i]) return fail(KAON_E_INVALID, "kaon_kprodigy_attach: tensor %d has no s buffer", i);
    if (pl->momentum_kind == KAON_M_4BIT && t.bshift >= 31 && t.numel > 128)
      return fail(KAON_E_UNSUPPORTED, "KProdigy: tensor %d: one 4-bit block over %lld elements", i, (long long)t.numel);
    if (t.rows > 0) {
      if (t.cols > CAP) return fail(KAON_E_UNSUPPORTED, "KProdigy: tensor %d: rows of %d elements exceed a work item of %d", i, t.cols, CAP);
      fact.push_back(i);
      row_begin.push_back(row_begin.back() + t.rows);
    }
    for (long long e = 0; e < t.numel; e += KP_ITEM)
      items.push_back(Task{i, PH_ADA_APPLY, e, (int)std::min<long long>(KP_ITEM, t.numel - e), 0, 0, 0});
  }
  begin[n] = (int)items.size();
  {
    std::vector<Task> hm((size_t)pl->n_tasks_main);
    KAON_CUDA(cudaMemcpy(hm.data(), pl->d_tasks_main, sizeof(Task) * hm.size(), cudaMemcpyDeviceToHost));
    const bool bf16 = pl->param_dtype == KAON_DT_BF16;
    for (const Task& t : hm) {
      if (t.phase == PH_ADA_STATS) {
        if (bf16 && stats_item_ok(pl, t)) stats.push_back(t);
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
  const size_t o_bufs = take(sizeof(KpBufs) * n), o_part = take(sizeof(double) * 2 * items.size());
  const size_t o_sums = take(sizeof(float) * 2 * n), o_tmax = take(sizeof(unsigned) * n), o_told = take(sizeof(float) * n);
  const size_t o_fact = take(sizeof(int) * fact.size()), o_rows = take(sizeof(long long) * row_begin.size());
  const size_t o_stats = take(sizeof(Task) * stats.size()), o_fin = take(sizeof(Task) * fin.size());
  KAON_CUDA(cudaMalloc(&h->block, std::max<size_t>(o, 256)));
  unsigned char* base = reinterpret_cast<unsigned char*>(h->block);
  KAON_CUDA(cudaMemset(base, 0, std::max<size_t>(o, 256)));
  h->bytes = (int64_t)o;
  auto put = [&](size_t off, const void* src, size_t b) -> cudaError_t {
    return b ? cudaMemcpy(base + off, src, b, cudaMemcpyHostToDevice) : cudaSuccess;
  };
  KAON_CUDA(put(o_items, items.data(), sizeof(Task) * items.size()));
  KAON_CUDA(put(o_begin, begin.data(), sizeof(int) * (n + 1)));
  KAON_CUDA(put(o_bufs, bufs.data(), sizeof(KpBufs) * n));
  KAON_CUDA(put(o_fact, fact.data(), sizeof(int) * fact.size()));
  KAON_CUDA(put(o_rows, row_begin.data(), sizeof(long long) * row_begin.size()));
  KAON_CUDA(put(o_stats, stats.data(), sizeof(Task) * stats.size()));
  KAON_CUDA(put(o_fin, fin.data(), sizeof(Task) * fin.size()));
  KpView& x = h->view;
  x.items = reinterpret_cast<const Task*>(base + o_items); x.n_items = (int)items.size();
  x.item_begin = reinterpret_cast<const int*>(base + o_begin);
  x.bufs = reinterpret_cast<const KpBufs*>(base + o_bufs);
  x.part = reinterpret_cast<double*>(base + o_part);
  x.sums = reinterpret_cast<float*>(base + o_sums);
  x.tmax = reinterpret_cast<unsigned*>(base + o_tmax);
  x.told = reinterpret_cast<float*>(base + o_told);
  x.fact = reinterpret_cast<const int*>(base + o_fact); x.n_fact = (int)fact.size();
  x.row_begin = reinterpret_cast<const long long*>(base + o_rows); x.n_rows = row_begin.back();
  h->d_stats = stats.empty() ? nullptr : reinterpret_cast<Task*>(base + o_stats); h->n_stats = (int)stats.size();
  h->d_final = reinterpret_cast<Task*>(base + o_fin); h->n_final = (int)fin.size();
  h->h_sums.assign((size_t)2 * n, 0.0f);
  pl->device_bytes += h->bytes;
  return KAON_OK;
}

}  // namespace kaon

using namespace kaon;

extern "C" int kaon_kprodigy_attach(kaon_plan* pl, float* const* s, const float* const* p0, int n, int64_t slice_p) {
  if (!pl || !s) return fail(KAON_E_INVALID, "kaon_kprodigy_attach: null argument");
  if (pl->optimizer != KAON_OPT_KPRODIGY) return fail(KAON_E_INVALID, "plan was not built for KProdigy");
  if (n != pl->n_tensors) return fail(KAON_E_INVALID, "kaon_kprodigy_attach: %d pointers for a plan of %d tensors", n, pl->n_tensors);
  if (slice_p < 1) return fail(KAON_E_INVALID, "slice_p must be >= 1");
  if (int rc = check_device(pl)) return rc;
  return kp_build(pl, s, p0, slice_p);
}

extern "C" int kaon_kprodigy_pass1(kaon_plan* pl, const kaon_kprodigy_pass1_hparams* h, float* sums_host, void* stream) {
  if (!pl || !h) return fail(KAON_E_INVALID, "kaon_kprodigy_pass1: null argument");
  if (pl->optimizer != KAON_OPT_KPRODIGY) return fail(KAON_E_INVALID, "plan was not built for KProdigy");
  if (int rc = check_device(pl)) return rc;
  KpHost* kh = reinterpret_cast<KpHost*>(pl->kp);
  if (!kh) return fail(KAON_E_INVALID, "kaon_kprodigy_pass1: call kaon_kprodigy_attach first");
  const bool has_m = pl->momentum_kind != KAON_M_NONE;
  if (has_m != (h->beta1 > 0.0)) return fail(KAON_E_INVALID, "beta1 %g does not match the plan's momentum kind", h->beta1);
  if (h->do_d && !sums_host) return fail(KAON_E_INVALID, "kaon_kprodigy_pass1: do_d needs the host array for the sums");
  KpDev hp{};
  hp.fb1 = (float)h->beta1; hp.ft = (float)(h->d * (1.0 - h->beta1));
  { __nv_bfloat16 tb = __float2bfloat16_rn(hp.ft); hp.ftb = __bfloat162float(tb); }
  hp.fd = (float)h->d; hp.d_is_one = h->d == 1.0;
  hp.w1 = (float)(1.0 - h->beta1); hp.w1m1 = hp.w1 - 1.0f; hp.small_w1 = hp.w1 < 0.5f;
  hp.fb2 = (float)h->beta2; hp.fv = (float)(h->d * h->d * (1.0 - h->beta2));
  hp.fb3 = (float)h->beta3; hp.fa = (float)h->alpha_s;
  hp.fwd = (float)h->weight_decay_coupled; hp.has_wdc = h->weight_decay_coupled != 0.0;
  hp.do_d = h->do_d != 0; hp.gc = h->gradient_centralization != 0; hp.factored = h->factored != 0;
  hp.has_m = has_m; hp.slice_p = kh->slice_p;
  cudaStream_t s = (cudaStream_t)stream;
  const KpView& x = kh->view;
  const int mk = pl->momentum_kind;
  const int grid = std::max(1, std::min(x.n_items, pl->sm_count * 8));
  if (hp.factored && x.n_fact > 0) {
    AdaDev ad{};
    ad.w2 = (float)(1.0 - h->beta2); ad.w2m1 = ad.w2 - 1.0f; ad.small_w2 = ad.w2 < 0.5f;
    ad.w1 = 1.0f; ad.eps1 = (float)h->eps_factored; ad.has_eps = h->eps_factored > 0.0; ad.clip = 1.0f;
    ad.gc = hp.gc;
    PlanView v = pl->view;
    KAON_CUDA(cudaMemsetAsync(v.task_counter, 0, pl->counters_bytes - sizeof(unsigned), s));
    if (kh->d_stats != nullptr)
      if (int rc = launch_stats_tasks(pl, pl->view, ad, kh->d_stats, kh->n_stats, s)) return rc;
    v.tasks = kh->d_final; v.n_tasks = kh->n_final;
    AdaKernel k = pick_ada(pl->param_dtype, pl->momentum_kind, false);
    k<<<pl->grid, ADA_THREADS, pl->smem_bytes, s>>>(v, ad, (int)x_offset_rows(pl) | (pl->double_buffer ? 1 : 0));
    KAON_CUDA(cudaGetLastError());
    pl->launches += 1;
  } else if (hp.gc && x.n_fact > 0) {
    if (pl->param_dtype == KAON_DT_BF16) kp_rowmean_kernel<__nv_bfloat16><<<pl->sm_count * 8, KP_THREADS, 0, s>>>(pl->view, x);
    else kp_rowmean_kernel<float><<<pl->sm_count * 8, KP_THREADS, 0, s>>>(pl->view, x);
    pl->launches += 1;
  }
  if (x.n_items > 0) {
    if (mk == KAON_M_INT8) {
      kp_prep_kernel<<<pl->n_tensors, KP_THREADS, 0, s>>>(pl->view, x);
      pl->launches += 1;
    }
    KpSweep k0 = pick_sweep<0>(pl->param_dtype, mk);
    if (!k0) return fail(KAON_E_INVALID, "no KProdigy kernel for this dtype combination");
    k0<<<grid, KP_THREADS, 0, s>>>(pl->view, hp, x);
    pl->launches += 1;
    if (mk == KAON_M_INT8) {
      pick_sweep<1>(pl->param_dtype, mk)<<<grid, KP_THREADS, 0, s>>>(pl->view, hp, x);
      pl->launches += 1;
    }
    if (hp.do_d) {
      kp_reduce_kernel<false><<<pl->n_tensors, KP_THREADS, 0, s>>>(pl->view, x);
      pl->launches += 1;
    }
    KAON_CUDA(cudaGetLastError());
  }
  if (hp.do_d) {  // the per-tensor sums go to the host, which owns the estimate (one synchronisation, as the reference's .item())
    KAON_CUDA(cudaMemcpyAsync(sums_host, x.sums, sizeof(float) * 2 * pl->n_tensors, cudaMemcpyDeviceToHost, s));
    KAON_CUDA(cudaStreamSynchronize(s));
  }
  return KAON_OK;
}

extern "C" int kaon_kprodigy_pass2(kaon_plan* pl, const kaon_kprodigy_pass2_hparams* h, uint64_t seed, uint32_t step,
                                   void* stream) {
  if (!pl || !h) return fail(KAON_E_INVALID, "kaon_kprodigy_pass2: null argument");
  if (pl->optimizer != KAON_OPT_KPRODIGY) return fail(KAON_E_INVALID, "plan was not built for KProdigy");
  if (int rc = check_device(pl)) return rc;
  KpHost* kh = reinterpret_cast<KpHost*>(pl->kp);
  if (!kh) return fail(KAON_E_INVALID, "kaon_kprodigy_pass2: call kaon_kprodigy_attach first");
  if (h->bf16_method < KAON_W_NONE || h->bf16_method > KAON_W_KAHAN) return fail(KAON_E_UNSUPPORTED, "bf16_method %d", h->bf16_method);
  if (int rc = check_kahan(pl, h->bf16_method)) return rc;
  if (!(h->d > 0.0) || !(h->eps > 0.0)) return fail(KAON_E_INVALID, "d and eps must be > 0");
  KpDev hp{};
  hp.fd = (float)h->d; hp.floor_ = (float)(h->d * h->eps); hp.cap = (float)(1.0 / (h->d * h->eps));
  hp.fdlr = (float)h->dlr; hp.fdecay = (float)h->decay_dlr; hp.has_decay = h->decay_dlr != 0.0;
  hp.cautious = h->cautious != 0; hp.gc = h->gradient_centralization != 0; hp.factored = h->factored != 0;
  hp.has_m = pl->momentum_kind != KAON_M_NONE;
  hp.sr = h->bf16_method == KAON_W_SR && pl->param_dtype == KAON_DT_BF16;
  hp.kahan = h->bf16_method == KAON_W_KAHAN && pl->param_dtype == KAON_DT_BF16;
  hp.slice_p = kh->slice_p;
  hp.step = step; hp.k0 = (uint32_t)seed; hp.k1 = (uint32_t)(seed >> 32);
  cudaStream_t s = (cudaStream_t)stream;
  const KpView& x = kh->view;
  if (x.n_items == 0) return KAON_OK;
  const int mk = pl->momentum_kind;
  const int grid = std::max(1, std::min(x.n_items, pl->sm_count * 8));
  if (hp.cautious) {
    pick_sweep<2>(pl->param_dtype, mk)<<<grid, KP_THREADS, 0, s>>>(pl->view, hp, x);
    kp_reduce_kernel<true><<<pl->n_tensors, KP_THREADS, 0, s>>>(pl->view, x);
    pl->launches += 2;
  }
  pick_sweep<3>(pl->param_dtype, mk)<<<grid, KP_THREADS, 0, s>>>(pl->view, hp, x);
  KAON_CUDA(cudaGetLastError());
  pl->launches += 1;
  return KAON_OK;
}
