// Adakaon step (and, fused into it, the Nekaon climb/removal) for sm_100a: one persistent kernel walks
// the plan's work list.
//
// Factored (>=2-D) tensor, viewed as [R, C]:
//   STATS (a run of rows): gradient rows arrive in shared memory through the bulk-copy engine; per
//     row: centralization mean, row mean of g^2+eps1, row EMA (stored); per column, partial sums over
//     the run of g^2+eps1 and of g^2/row_i (thread-owned columns, fixed row order) -> scratch slot.
//   FINAL (a strip of columns): sum the slots in order -> column EMA (stored), c_j = rsqrt(col_j);
//     the last strip to arrive combines the partials into mean(row) and the clip divisor
//     max(rms(u)/clip, 1) with  sum u^2 = mean(row) * sum_j (1/col_j) * sum_i g_ij^2/row_i.
//   COUNT (same runs): recompute u and the momentum EMA, count delta*g > 0 (cautious).
//   APPLY (same runs): recompute, encode + store the momentum, write the weights; the Nekaon removal
//     of the previous climb and the new climb ride on the same read and write of each weight.
// 1-D tensor: FLAT, the whole tensor in one work item.
// Every cross-item sum is taken in a fixed order: results do not depend on scheduling.
//
// Each of STATS / COUNT / APPLY exists twice.  The staged form above (ada_stats, ada_rows) handles any
// shape.  The streaming form (ada_stats_stream, ada_stream) needs rows that are a multiple of 8
// elements and reads gradient, momentum and weights straight from global memory, with what is per row
// or per column fetched from the scratch in L2; it has no barrier in its loops.  When every factored
// tensor of a plan streams, COUNT and APPLY leave this kernel altogether and run as launches of
// adakaon_apply_kernel (256-thread CTAs, four per SM, one bulk-copied flat item each), ordered by the
// stream instead of by completion counters.
#include <map>
#include <vector>
#include <mutex>
#include <utility>
#include <type_traits>

#include "adakaon_dev.h"
#include "kaon_host.h"
#include "kaon_ops.cuh"
#include "kaon_packed.cuh"

namespace kaon {


constexpr int AT = ADA_THREADS;

// ----------------------------------------------------------------------------- block reductions

__device__ __forceinline__ double block_sum_d(double v, double* red, int tid) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  __syncthreads();
  if ((tid & 31) == 0) red[tid >> 5] = v;
  __syncthreads();
  double t = 0.0;
  for (int w = 0; w < AT / 32; ++w) t += red[w];
  return t;
}

__device__ __forceinline__ unsigned block_sum_u(unsigned v, double* red, int tid) {
  return (unsigned)(block_sum_d((double)v, red, tid) + 0.5);
}

__device__ __forceinline__ float block_max_f(float v, double* red, int tid) {
  v = group_max(v, 32);
  __syncthreads();
  if ((tid & 31) == 0) red[tid >> 5] = (double)v;
  __syncthreads();
  float t = 0.0f;
  for (int w = 0; w < AT / 32; ++w) t = fmaxf(t, (float)red[w]);
  return t;
}

// ----------------------------------------------------------------------------- scalar helpers

// x / d for a divisor shared by many elements: rcp = RN(1/d) computed once; one Newton step on the
// residual gives the correctly rounded quotient for normal-range operands.
__device__ __forceinline__ float div_shared(float x, float d, float rcp) {
  float q0 = __fmul_rn(x, rcp);
  float r = __fmaf_rn(-q0, d, x);
  return __fmaf_rn(r, rcp, q0);
}

// Nekaon perturbation of one element (reference src/kaon/msam.py:222-230)
__device__ __forceinline__ float climb_e(float m_dec, float alpha, float bound) {
  float e = __fmul_rn(m_dec, alpha);
  if (e != e) e = 0.0f;
  return fminf(fmaxf(e, -bound), bound);
}

// One weight write on a register value: pv <- round(pv + alpha*d).  bf16 params: stochastic rounding
// with `noise16`, or (sr == false, alpha == -1) nearest-even of pv - bf16(d); fp32 params: one fma.
template <typename PT>
__device__ __forceinline__ float write_step(float pv, float d, float alpha, bool sr, uint32_t noise16) {
  if constexpr (Elems<PT>::IS_BF16) {
    if (sr) return __uint_as_float((__float_as_uint(__fmaf_rn(d, alpha, pv)) + noise16) & 0xFFFF0000u);
    return round_bf16(__fadd_rn(pv, __fmul_rn(alpha, round_bf16(d))));
  } else {
    return __fmaf_rn(d, alpha, pv);
  }
}

__device__ __forceinline__ uint32_t noise_lane(const uint32_t nz[4], int k) {
  return (k & 1) ? (nz[k >> 1] >> 16) : (nz[k >> 1] & 0xffffu);
}

// Eight values out (weights: `pr` names the mirrors on other GPUs; state: none).
template <typename PT>
__device__ __forceinline__ void store8(void* pe, int cnt, const float v[8], const Peers* pr) {
  if constexpr (Elems<PT>::IS_BF16) {
    if (cnt >= 8) {
      const uint4 out = make_uint4(pack_bf16_rn(v[0], v[1]), pack_bf16_rn(v[2], v[3]),
                                   pack_bf16_rn(v[4], v[5]), pack_bf16_rn(v[6], v[7]));
      *reinterpret_cast<uint4*>(pe) = out;
      mirror16(pr, pe, out);
    } else {
      for (int k = 0; k < cnt; ++k)
        reinterpret_cast<uint16_t*>(pe)[k] = (uint16_t)(__float_as_uint(v[k]) >> 16);
      mirror_copy(pr, pe, cnt * 2);
    }
  } else {
    for (int k = 0; k < cnt; ++k) reinterpret_cast<float*>(pe)[k] = v[k];
    mirror_copy(pr, pe, cnt * 4);
  }
}

// ----------------------------------------------------------------------------- staging

// Two staging buffers: while the CTA works on one chunk, the bulk-copy engine fills the other.
struct Stage {
  unsigned char* g_s;   // buffers of the chunk being processed (set by stage_wait)
  unsigned char* m_s;
  unsigned char* gbuf[2];
  unsigned char* mbuf[2];
  uint64_t* bar[2];
  unsigned parity[2];
  int nbuf;             // 2, or 1 when shared memory has no room for a second buffer
};

__device__ __forceinline__ unsigned bulk_head(const unsigned char* src, unsigned bytes) {
  return (reinterpret_cast<uintptr_t>(src) & 15) ? 0u : (bytes & ~15u);
}

// Start bringing a chunk into buffer b.  All threads call (the ragged ends are plain loads).
__device__ __forceinline__ void stage_issue(Stage& st, int b, const unsigned char* gsrc, unsigned gbytes,
                                            const unsigned char* msrc, unsigned mbytes, int tid) {
  const unsigned ghead = stage_tail(st.gbuf[b], gsrc, gbytes, tid);
  const unsigned mhead = mbytes ? stage_tail(st.mbuf[b], msrc, mbytes, tid) : 0u;
  if ((ghead + mhead) && tid == 0) {
    fence_async_smem();
    mbar_expect_tx(st.bar[b], ghead + mhead);
    if (ghead) bulk_g2s(st.gbuf[b], gsrc, ghead, st.bar[b]);
    if (mhead) bulk_g2s(st.mbuf[b], msrc, mhead, st.bar[b]);
  }
}

// Wait for the chunk issued into buffer b (same arguments) and make it the current one.
__device__ __forceinline__ bool stage_wait(Stage& st, int b, const unsigned char* gsrc, unsigned gbytes,
                                           const unsigned char* msrc, unsigned mbytes, unsigned* status) {
  bool ok = true;
  if (bulk_head(gsrc, gbytes) + (mbytes ? bulk_head(msrc, mbytes) : 0u)) {
    ok = mbar_wait(st.bar[b], st.parity[b], status, 1002u);
    st.parity[b] ^= 1u;
  }
  st.g_s = st.gbuf[b];
  st.m_s = st.mbuf[b];
  return __syncthreads_and(ok) != 0;
}

template <int MK>
__device__ __forceinline__ unsigned m_bytes(long long n) {
  if constexpr (MK == KAON_M_4BIT) return (unsigned)((n + 1) >> 1);
  else if constexpr (MK == KAON_M_INT8) return (unsigned)n;
  else if constexpr (MK == KAON_M_BF16) return (unsigned)(n * 2);
  else if constexpr (MK == KAON_M_F32) return (unsigned)(n * 4);
  else return 0u;
}

template <int MK>
__device__ __forceinline__ const unsigned char* m_ptr(const DevTensor& d, long long e0) {
  const unsigned char* b = reinterpret_cast<const unsigned char*>(d.m);
  if constexpr (MK == KAON_M_4BIT) return b + (e0 >> 1);
  else if constexpr (MK == KAON_M_INT8) return b + e0;
  else if constexpr (MK == KAON_M_BF16) return b + e0 * 2;
  else if constexpr (MK == KAON_M_F32) return b + e0 * 4;
  else return nullptr;
}

// Row means of the staged chunk for gradient centralization (0 when it is off).
template <typename PT>
__device__ __forceinline__ float row_mean(const unsigned char* rowp, int C, int lane) {
  using E = Elems<PT>;
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
  float mean = __fdiv_rn(s, (float)C);
  return E::IS_BF16 ? round_bf16(mean) : mean;
}

// One warp's share of a row reduction when a row is split over G warps (part = 0..G-1): the plain sum
// (SQ = false, for the centralization mean) or the sum of (x - mu)^2 + eps1 (SQ = true).
template <typename PT, bool SQ>
__device__ __forceinline__ float row_part(const unsigned char* rowp, int C, int part, int G, int lane,
                                          float mu, bool gc, bool has_eps, float eps1) {
  using E = Elems<PT>;
  float s = 0.0f;
  auto term = [&](float x) -> float {
    if (!SQ) return x;
    float y = x;
    if (gc) { y = __fsub_rn(x, mu); if (E::IS_BF16) y = round_bf16(y); }
    float sq = __fmul_rn(y, y);
    return has_eps ? __fadd_rn(sq, eps1) : sq;
  };
  if ((C & 7) == 0) {
    for (int v = part * 32 + lane; v < (C >> 3); v += G * 32) {
      float x[8];
      E::load8(rowp + (size_t)v * 8 * E::BYTES, x);
      s += ((term(x[0]) + term(x[1])) + (term(x[2]) + term(x[3]))) + ((term(x[4]) + term(x[5])) + (term(x[6]) + term(x[7])));
    }
  } else {
    for (int i = part * 32 + lane; i < C; i += G * 32) s += term(E::load1(rowp, i));
  }
  return warp_sum(s);
}

template <typename PT>
__device__ __forceinline__ float centered(float g, float mu, bool gc) {
  if (!gc) return g;
  float x = __fsub_rn(g, mu);
  return Elems<PT>::IS_BF16 ? round_bf16(x) : x;
}

// ----------------------------------------------------------------------------- STATS

struct AdaSmem {
  float* mean_s;     // [MAX_TASK_ROWS] centralization mean of each staged row
  float* rfac_s;     // [MAX_TASK_ROWS] STATS: 1/row_i; COUNT/APPLY: r_i = rsqrt(row_i / mean(row))
  unsigned* rowmax_s;  // [MAX_TASK_ROWS] int8: bits of the row's absmax of the new momentum
  float* scale_s;    // [MAX_TASK_ROWS] int8: old row scales
  float* x_s;        // region X as floats (column accumulators / cfac / flat buffer)
  double* red;       // [AT/32]
  float* part_s;     // [AT/32] per-warp partial sums of split rows
};

// ST = element type of the signal whose second moment is tracked: the gradient (Adakaon) or the
// orthogonalised momentum in bf16 (AdaMuon, `pv.signal`).
template <typename ST>
__device__ void ada_stats(const PlanView& pv, const AdaDev& hp, const Task& t, Stage& st,
                          const AdaSmem& sm, int tid) {
  using E = Elems<ST>;
  using PT = ST;
  const DevTensor d = pv.tensors[t.tensor];
  const unsigned char* g = reinterpret_cast<const unsigned char*>(pv.grads[t.tensor]);
  if (g != nullptr && pv.signal != nullptr) g = reinterpret_cast<const unsigned char*>(pv.signal[t.tensor]);
  const int C = d.cols;
  const int nrows = t.n / C;
  const bool gc = hp.gc != 0 && pv.signal == nullptr;
  bool ok = g != nullptr;
  float* acc1 = sm.x_s;       // sum_i (g^2 + eps1)
  float* acc2 = sm.x_s + C;   // sum_i g^2 / row_i
  for (int j = tid; j < 2 * C; j += AT) sm.x_s[j] = 0.0f;
  double rowsum = 0.0;  // lane 0 of each warp: sum of the new row statistics it produced
  const int warp = tid >> 5, lane = tid & 31;
  auto issue = [&](int c0, int b) {
    const int nrc = min(d.chunk_rows, nrows - c0);
    stage_issue(st, b, g + (t.e0 + (long long)c0 * C) * E::BYTES, (unsigned)(nrc * C) * E::BYTES, nullptr, 0u, tid);
  };
  if (ok && st.nbuf == 2) issue(0, 0);
  for (int c0 = 0, ci = 0; ok && c0 < nrows; c0 += d.chunk_rows, ++ci) {
    const int nrc = min(d.chunk_rows, nrows - c0);
    const long long e0 = t.e0 + (long long)c0 * C;
    const int b = st.nbuf == 2 ? (ci & 1) : 0;
    if (st.nbuf == 1) issue(c0, 0);
    else if (c0 + d.chunk_rows < nrows) issue(c0 + d.chunk_rows, b ^ 1);
    const bool pre_rows = nrc <= AT;  // old row statistics: load before the wait, hand over through rfac_s
    float pre_old = 0.0f;
    if (pre_rows && tid < nrc) pre_old = d.stat_a[t.row0 + c0 + tid];
    ok = stage_wait(st, b, g + e0 * E::BYTES, (unsigned)(nrc * C) * E::BYTES, nullptr, 0u, pv.status);
    if (!ok) break;
    if (pre_rows) {
      if (tid < nrc) sm.rfac_s[tid] = pre_old;
      __syncthreads();
    }
    // rows: centralization mean, mean of g^2+eps1, row EMA
    constexpr int NW = AT / 32;
    if (nrc < NW) {
      // fewer rows than warps (wide rows): split every row over G warps, combine in warp order
      const int G = NW / nrc, r = warp / G, part = warp % G;
      const bool act = r < nrc;
      const unsigned char* rowp = st.g_s + (size_t)(act ? r : 0) * C * E::BYTES;
      if (gc) {
        const float ps = act ? row_part<PT, false>(rowp, C, part, G, lane, 0.0f, false, false, 0.0f) : 0.0f;
        if (lane == 0) sm.part_s[warp] = ps;
        __syncthreads();
        if (tid < nrc) {
          float tot = 0.0f;
          for (int q = 0; q < G; ++q) tot += sm.part_s[tid * G + q];
          const float mean = __fdiv_rn(tot, (float)C);
          const float mr = E::IS_BF16 ? round_bf16(mean) : mean;
          sm.mean_s[tid] = mr;
          pv.aux[aux_mean(d) + t.row0 + c0 + tid] = mr;
        }
        __syncthreads();
      } else if (tid < nrc) {
        sm.mean_s[tid] = 0.0f;
      }
      const float mu = (gc && act) ? sm.mean_s[r] : 0.0f;
      const float ps2 = act ? row_part<PT, true>(rowp, C, part, G, lane, mu, gc, hp.has_eps != 0, hp.eps1) : 0.0f;
      if (lane == 0) sm.part_s[warp] = ps2;
      __syncthreads();
      if (tid < nrc) {
        float tot = 0.0f;
        for (int q = 0; q < G; ++q) tot += sm.part_s[tid * G + q];
        const int row = t.row0 + c0 + tid;
        const float mean = __fdiv_rn(tot, (float)C);
        const float rn = lerp_torch(pre_old, mean, hp.w2, hp.w2m1, hp.small_w2 != 0);
        d.stat_a[row] = rn;
        sm.rfac_s[tid] = __fdiv_rn(1.0f, rn);
        rowsum += (double)rn;
      }
    } else
    for (int r = warp; r < nrc; r += AT / 32) {
      const unsigned char* rowp = st.g_s + (size_t)r * C * E::BYTES;
      const float mu = gc ? row_mean<PT>(rowp, C, lane) : 0.0f;
      float s = 0.0f;
      if ((C & 7) == 0) {
        for (int v = lane; v < (C >> 3); v += 32) {
          float x[8];
          E::load8(rowp + (size_t)v * 8 * E::BYTES, x);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float y = centered<PT>(x[k], mu, gc);
            float sq = __fmul_rn(y, y);
            if (hp.has_eps) sq = __fadd_rn(sq, hp.eps1);
            s += sq;
          }
        }
      } else {
        for (int i = lane; i < C; i += 32) {
          const float x = centered<PT>(E::load1(rowp, i), mu, gc);
          float sq = __fmul_rn(x, x);
          if (hp.has_eps) sq = __fadd_rn(sq, hp.eps1);
          s += sq;
        }
      }
      s = warp_sum(s);
      if (lane == 0) {
        const int row = t.row0 + c0 + r;
        const float mean = __fdiv_rn(s, (float)C);
        const float rn = lerp_torch(pre_rows ? sm.rfac_s[r] : d.stat_a[row], mean, hp.w2, hp.w2m1, hp.small_w2 != 0);
        d.stat_a[row] = rn;
        sm.mean_s[r] = mu;
        if (gc) pv.aux[aux_mean(d) + row] = mu;
        sm.rfac_s[r] = __fdiv_rn(1.0f, rn);
        rowsum += (double)rn;
      }
    }
    __syncthreads();
    // columns: each thread owns columns tid, tid+AT, ... and walks the staged rows in order
    if ((C & 7) == 0) {
      // eight columns per thread, rows in order
      for (int v = tid; v < (C >> 3); v += AT) {
        float a1[8], a2[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) { a1[k] = 0.0f; a2[k] = 0.0f; }
        for (int r = 0; r < nrc; ++r) {
          float x[8];
          E::load8(st.g_s + ((size_t)r * C + (size_t)v * 8) * E::BYTES, x);
          const float mu = sm.mean_s[r], ri = sm.rfac_s[r];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float y = centered<PT>(x[k], mu, gc);
            const float sq = __fmul_rn(y, y);
            a1[k] += hp.has_eps ? __fadd_rn(sq, hp.eps1) : sq;
            a2[k] += __fmul_rn(sq, ri);
          }
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) { acc1[v * 8 + k] += a1[k]; acc2[v * 8 + k] += a2[k]; }
      }
    } else
    for (int j = tid; j < C; j += AT) {
      float a1 = 0.0f, a2 = 0.0f;
      for (int r = 0; r < nrc; ++r) {
        const float x = centered<PT>(E::load1(st.g_s + (size_t)r * C * E::BYTES, j), sm.mean_s[r], gc);
        const float sq = __fmul_rn(x, x);
        a1 += hp.has_eps ? __fadd_rn(sq, hp.eps1) : sq;
        a2 += __fmul_rn(sq, sm.rfac_s[r]);
      }
      acc1[j] += a1;
      acc2[j] += a2;
    }
    __syncthreads();
  }
  // publish the slot
  float* slot = pv.aux + d.aux_off + 2ll * t.slot * C;
  if (ok)
    for (int j = tid; j < 2 * C; j += AT) slot[j] = sm.x_s[j];
  const double rs = block_sum_d(rowsum, sm.red, tid);
  if (tid == 0 && ok) reinterpret_cast<double*>(pv.aux + aux_rowpart(d))[t.slot] = rs;
  __threadfence();
  __syncthreads();
  if (tid == 0) signal_counter(pv.done + 0 * pv.n_tensors + t.tensor, 1u);
}

// ----------------------------------------------------------------------------- STATS, streaming

// The same work item without shared-memory staging, for rows of at least 256 elements that are a
// multiple of 8: rows are taken in groups that stay in L2 (a few hundred KB per CTA); each warp owns
// whole rows of the group and streams them from global memory twice (mean, then the sum of squares:
// no barrier inside), then every thread walks the group's rows for the columns it owns, with the
// column partial sums in registers for the whole item.  Two barriers per group instead of six per
// 16 K elements.  Sums are taken in a fixed order: results are reproducible run to run (they differ
// from ada_stats in the last bits: another summation order).
template <typename ST>
__device__ void ada_stats_stream(const PlanView& pv, const AdaDev& hp, const Task& t, const AdaSmem& sm,
                                 unsigned char* dyn, int tid) {
  using E = Elems<ST>;
  using PT = ST;
  const DevTensor d = pv.tensors[t.tensor];
  const unsigned char* g = reinterpret_cast<const unsigned char*>(pv.grads[t.tensor]);
  if (g != nullptr && pv.signal != nullptr) g = reinterpret_cast<const unsigned char*>(pv.signal[t.tensor]);
  const int C = d.cols;
  const int nv = C >> 3;                 // vectors per row
  const int nrows = t.n / C;
  const bool gc = hp.gc != 0 && pv.signal == nullptr;
  const bool ok = g != nullptr;
  const int warp = tid >> 5, lane = tid & 31;
  constexpr int NW = AT / 32;
  // column ownership: nv >= AT: vectors tid, tid+AT, ... of every row; nv < AT: Q row groups, one vector
  const int Q = nv >= AT ? 1 : AT / nv;
  const int q = nv >= AT ? 0 : tid / nv;
  const int v0 = nv >= AT ? tid : tid - q * nv;
  const bool col_act = q < Q;
  constexpr int VPT = CAP / 8 / AT;      // vectors per thread at most (rows are <= CAP elements)
  float a1[VPT][8], a2[VPT][8];
#pragma unroll
  for (int j = 0; j < VPT; ++j)
#pragma unroll
    for (int k = 0; k < 8; ++k) { a1[j][k] = 0.0f; a2[j][k] = 0.0f; }
  double rowsum = 0.0;
  // rows per group: about 384 KB of gradient, a multiple of the warp count, within the row arrays
  int grp = (int)((384 * 1024) / ((long long)C * E::BYTES));
  grp = max(NW, min(grp / NW * NW, MAX_TASK_ROWS));
  const unsigned char* gitem = g + t.e0 * E::BYTES;
  for (int r0 = 0; ok && r0 < nrows; r0 += grp) {
    const int nr = min(grp, nrows - r0);
    // ---- rows: one warp per row ----
    for (int r = warp; r < nr; r += NW) {
      const unsigned char* rowp = gitem + (size_t)(r0 + r) * C * E::BYTES;
      const int row = t.row0 + r0 + r;
      const float old = d.stat_a[row];
      float mu = 0.0f;
      float s2 = 0.0f;
      if constexpr (E::IS_BF16) {
        // packed pairs, four 16-byte loads in flight per lane
        const uint4* rowq = reinterpret_cast<const uint4*>(rowp);
        auto pairs = [](uint32_t w) { return pack2(bf16lo(w), bf16hi(w)); };
        if (gc) {
          f32x2 a0 = pack2(0.0f, 0.0f), a1v = pack2(0.0f, 0.0f);
          int v = lane;
          for (; v + 96 < nv; v += 128) {
            const uint4 q0 = rowq[v], q1 = rowq[v + 32], q2 = rowq[v + 64], q3 = rowq[v + 96];
            a0 = add2(a0, add2(add2(pairs(q0.x), pairs(q0.y)), add2(pairs(q1.x), pairs(q1.y))));
            a1v = add2(a1v, add2(add2(pairs(q0.z), pairs(q0.w)), add2(pairs(q1.z), pairs(q1.w))));
            a0 = add2(a0, add2(add2(pairs(q2.x), pairs(q2.y)), add2(pairs(q3.x), pairs(q3.y))));
            a1v = add2(a1v, add2(add2(pairs(q2.z), pairs(q2.w)), add2(pairs(q3.z), pairs(q3.w))));
          }
          for (; v < nv; v += 32) {
            const uint4 q0 = rowq[v];
            a0 = add2(a0, add2(pairs(q0.x), pairs(q0.y)));
            a1v = add2(a1v, add2(pairs(q0.z), pairs(q0.w)));
          }
          const float s = warp_sum((a0.x + a0.y) + (a1v.x + a1v.y));
          mu = round_bf16(__fdiv_rn(s, (float)C));
        }
        const uint32_t mu2 = pack_bf16_rn(mu, mu);
        const f32x2 EPS = pack2(hp.eps1, hp.eps1);
        auto sq2 = [&](uint32_t w) {
          const f32x2 y = pairs(gc ? sub_bf16x2(w, mu2) : w);
          const f32x2 q = mul2(y, y);
          return hp.has_eps ? add2(q, EPS) : q;
        };
        f32x2 b0 = pack2(0.0f, 0.0f), b1 = pack2(0.0f, 0.0f);
        int v = lane;
        for (; v + 96 < nv; v += 128) {
          const uint4 q0 = rowq[v], q1 = rowq[v + 32], q2 = rowq[v + 64], q3 = rowq[v + 96];
          b0 = add2(b0, add2(add2(sq2(q0.x), sq2(q0.y)), add2(sq2(q1.x), sq2(q1.y))));
          b1 = add2(b1, add2(add2(sq2(q0.z), sq2(q0.w)), add2(sq2(q1.z), sq2(q1.w))));
          b0 = add2(b0, add2(add2(sq2(q2.x), sq2(q2.y)), add2(sq2(q3.x), sq2(q3.y))));
          b1 = add2(b1, add2(add2(sq2(q2.z), sq2(q2.w)), add2(sq2(q3.z), sq2(q3.w))));
        }
        for (; v < nv; v += 32) {
          const uint4 q0 = rowq[v];
          b0 = add2(b0, add2(sq2(q0.x), sq2(q0.y)));
          b1 = add2(b1, add2(sq2(q0.z), sq2(q0.w)));
        }
        s2 = warp_sum((b0.x + b0.y) + (b1.x + b1.y));
      } else {
        if (gc) {
          float s = 0.0f;
          for (int v = lane; v < nv; v += 32) {
            float x[8];
            E::load8(rowp + (size_t)v * 8 * E::BYTES, x);
            s += ((x[0] + x[1]) + (x[2] + x[3])) + ((x[4] + x[5]) + (x[6] + x[7]));
          }
          s = warp_sum(s);
          mu = __fdiv_rn(s, (float)C);
        }
        for (int v = lane; v < nv; v += 32) {
          float x[8];
          E::load8(rowp + (size_t)v * 8 * E::BYTES, x);
          float sq[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float y = centered<PT>(x[k], mu, gc);
            sq[k] = __fmul_rn(y, y);
            if (hp.has_eps) sq[k] = __fadd_rn(sq[k], hp.eps1);
          }
          s2 += ((sq[0] + sq[1]) + (sq[2] + sq[3])) + ((sq[4] + sq[5]) + (sq[6] + sq[7]));
        }
        s2 = warp_sum(s2);
      }
      if (lane == 0) {
        const float mean = __fdiv_rn(s2, (float)C);
        const float rn = lerp_torch(old, mean, hp.w2, hp.w2m1, hp.small_w2 != 0);
        d.stat_a[row] = rn;
        sm.mean_s[r] = mu;
        if (gc) pv.aux[aux_mean(d) + row] = mu;
        sm.rfac_s[r] = __fdiv_rn(1.0f, rn);
        rowsum += (double)rn;
      }
    }
    __syncthreads();
    // ---- columns: this thread's vectors, the group's rows in order (L2 hits) ----
    if (col_act) {
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int v = v0 + j * AT;
        if (v < nv && (j == 0 || Q == 1)) {
          if constexpr (E::IS_BF16) {
            // the same per-element operations on packed pairs (a1[j][2w], a1[j][2w+1] = one pair)
            const f32x2 EPS = pack2(hp.eps1, hp.eps1);
            f32x2 A1[4], A2[4];
#pragma unroll
            for (int w = 0; w < 4; ++w) { A1[w] = pack2(a1[j][2 * w], a1[j][2 * w + 1]); A2[w] = pack2(a2[j][2 * w], a2[j][2 * w + 1]); }
#pragma unroll 4
            for (int r = q; r < nr; r += Q) {
              const uint4 qv = *reinterpret_cast<const uint4*>(gitem + ((size_t)(r0 + r) * C + (size_t)v * 8) * 2);
              const float mu = sm.mean_s[r], ri = sm.rfac_s[r];
              const uint32_t mu2 = pack_bf16_rn(mu, mu);
              const f32x2 RI = pack2(ri, ri);
              const uint32_t ww[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                const uint32_t yw = gc ? sub_bf16x2(ww[w], mu2) : ww[w];
                const f32x2 y = pack2(bf16lo(yw), bf16hi(yw));
                const f32x2 sq = mul2(y, y);
                A1[w] = add2(A1[w], hp.has_eps ? add2(sq, EPS) : sq);
                A2[w] = add2(A2[w], mul2(sq, RI));
              }
            }
#pragma unroll
            for (int w = 0; w < 4; ++w) { a1[j][2 * w] = A1[w].x; a1[j][2 * w + 1] = A1[w].y; a2[j][2 * w] = A2[w].x; a2[j][2 * w + 1] = A2[w].y; }
          } else
          for (int r = q; r < nr; r += Q) {
            float x[8];
            E::load8(gitem + ((size_t)(r0 + r) * C + (size_t)v * 8) * E::BYTES, x);
            const float mu = sm.mean_s[r], ri = sm.rfac_s[r];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const float y = centered<PT>(x[k], mu, gc);
              const float sq = __fmul_rn(y, y);
              a1[j][k] += hp.has_eps ? __fadd_rn(sq, hp.eps1) : sq;
              a2[j][k] += __fmul_rn(sq, ri);
            }
          }
        }
      }
    }
    __syncthreads();
  }
  // ---- publish the slot: column partial sums (row groups combined in order), row-statistic sum ----
  float* slot = pv.aux + d.aux_off + 2ll * t.slot * C;
  if (ok) {
    if (Q == 1) {
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int v = v0 + j * AT;
        if (col_act && v < nv) {
#pragma unroll
          for (int k = 0; k < 8; ++k) { slot[v * 8 + k] = a1[j][k]; slot[C + v * 8 + k] = a2[j][k]; }
        }
      }
    } else {
      // partials of the Q row groups through shared memory: [q][2][C] floats (at most AT * 16 floats)
      float* xs = reinterpret_cast<float*>(dyn);
      if (col_act) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          xs[(size_t)q * 2 * C + v0 * 8 + k] = a1[0][k];
          xs[(size_t)q * 2 * C + C + v0 * 8 + k] = a2[0][k];
        }
      }
      __syncthreads();
      for (int j = tid; j < 2 * C; j += AT) {
        float tot = 0.0f;
        for (int qq = 0; qq < Q; ++qq) tot += xs[(size_t)qq * 2 * C + j];
        slot[j] = tot;
      }
    }
  }
  const double rs = block_sum_d(rowsum, sm.red, tid);
  if (tid == 0 && ok) reinterpret_cast<double*>(pv.aux + aux_rowpart(d))[t.slot] = rs;
  __threadfence();
  __syncthreads();
  if (tid == 0) signal_counter(pv.done + 0 * pv.n_tensors + t.tensor, 1u);
}

__device__ __forceinline__ bool stats_stream_ok(const DevTensor& d, const void* g, int ebytes) {
  return (d.cols & 7) == 0 && d.cols >= 256 && (reinterpret_cast<uintptr_t>(g) & 15) == 0 &&
         (((long long)d.cols * ebytes) & 15) == 0;
}

// ----------------------------------------------------------------------------- STATS as a launch of its own

// The streaming STATS work item in small CTAs (256 threads, four per SM) for plans whose factored tensors
// all stream bf16 rows of at least 256 elements: the same outputs as ada_stats_stream (row statistics,
// centralization means, the item's column partial sums and row-statistic sum), taken with packed-pair
// arithmetic.  Phase 1: one warp per row, the row streamed twice (mean, then sum of squares).  Phase 2:
// thread-owned columns over the item's rows, which are in L2 by then; rows narrower than the CTA are
// shared out over row groups whose partial sums are combined in a fixed order.  FINAL runs in the
// following launch, so the order of the stream stands in for waiting on the completion counter (which
// is still raised: the FINAL items look at it).
constexpr int STT = 256;
constexpr int ST_MAXROWS = 1024;   // rows of one STATS item at most
constexpr int ST_VPT = 2;          // column vectors a thread accumulates at a time

__global__ void __launch_bounds__(STT, 4) ada_stats_kernel(PlanView pv, AdaDev hp) {
  __shared__ uint32_t mean2_s[ST_MAXROWS];  // centralization mean of each row, two bf16 copies
  __shared__ float rinv_s[ST_MAXROWS];      // 1 / row statistic
  __shared__ float xs[STT * 16];            // partial sums of the row groups (narrow rows)
  __shared__ double red[STT / 32];
  __shared__ int next_s[2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (on_reserved_sm(pv.sm_reserve)) return;
  auto claim_next = [&](int slot) {
    if (tid == 0) {
      const unsigned st = *reinterpret_cast<volatile unsigned*>(pv.status);
      next_s[slot] = st ? 0x7fffffff : (int)atomicAdd(pv.task_counter, 1u);
    }
  };
  claim_next(0);
  __syncthreads();
  int slot_i = 0;
  int cur = next_s[0];
  const bool gc = hp.gc != 0 && pv.signal == nullptr;
  const f32x2 EPS = pack2(hp.eps1, hp.eps1);
  auto pairs = [](uint32_t w) { return pack2(bf16lo(w), bf16hi(w)); };
  while (cur < pv.n_tasks) {
    claim_next(slot_i ^ 1);
    const Task t = pv.tasks[cur];
    const DevTensor d = pv.tensors[t.tensor];
    const unsigned char* g = reinterpret_cast<const unsigned char*>(pv.grads[t.tensor]);
    if (g != nullptr && pv.signal != nullptr) g = reinterpret_cast<const unsigned char*>(pv.signal[t.tensor]);
    const bool ok = g != nullptr;
    const int C = d.cols, nv = C >> 3, nrows = t.n / C;
    double rowsum = 0.0;
    const uint4* gitem = reinterpret_cast<const uint4*>(g + (ok ? t.e0 * 2 : 0));
    float* slot = pv.aux + d.aux_off + 2ll * t.slot * C;
    // row statistics of rows [ra, rb) of the item, one warp per row
    auto rows_phase = [&](const int ra, const int rb) {
      for (int r = ra + warp; r < rb; r += STT / 32) {
        const uint4* rowq = gitem + (size_t)r * nv;
        const int row = t.row0 + r;
        const float old = d.stat_a[row];
        float mu = 0.0f;
        if (gc) {
          f32x2 a0 = pack2(0.0f, 0.0f), a1 = pack2(0.0f, 0.0f);
          int v = lane;
          for (; v + 96 < nv; v += 128) {
            const uint4 q0 = rowq[v], q1 = rowq[v + 32], q2 = rowq[v + 64], q3 = rowq[v + 96];
            a0 = add2(a0, add2(add2(pairs(q0.x), pairs(q0.y)), add2(pairs(q1.x), pairs(q1.y))));
            a1 = add2(a1, add2(add2(pairs(q0.z), pairs(q0.w)), add2(pairs(q1.z), pairs(q1.w))));
            a0 = add2(a0, add2(add2(pairs(q2.x), pairs(q2.y)), add2(pairs(q3.x), pairs(q3.y))));
            a1 = add2(a1, add2(add2(pairs(q2.z), pairs(q2.w)), add2(pairs(q3.z), pairs(q3.w))));
          }
          for (; v < nv; v += 32) {
            const uint4 q0 = rowq[v];
            a0 = add2(a0, add2(pairs(q0.x), pairs(q0.y)));
            a1 = add2(a1, add2(pairs(q0.z), pairs(q0.w)));
          }
          mu = round_bf16(__fdiv_rn(warp_sum((a0.x + a0.y) + (a1.x + a1.y)), (float)C));
        }
        const uint32_t mu2 = pack_bf16_rn(mu, mu);
        auto sq2 = [&](uint32_t w) {
          const f32x2 y = pairs(gc ? sub_bf16x2(w, mu2) : w);
          const f32x2 q = mul2(y, y);
          return hp.has_eps ? add2(q, EPS) : q;
        };
        f32x2 b0 = pack2(0.0f, 0.0f), b1 = pack2(0.0f, 0.0f);
        int v = lane;
        for (; v + 96 < nv; v += 128) {
          const uint4 q0 = rowq[v], q1 = rowq[v + 32], q2 = rowq[v + 64], q3 = rowq[v + 96];
          b0 = add2(b0, add2(add2(sq2(q0.x), sq2(q0.y)), add2(sq2(q1.x), sq2(q1.y))));
          b1 = add2(b1, add2(add2(sq2(q0.z), sq2(q0.w)), add2(sq2(q1.z), sq2(q1.w))));
          b0 = add2(b0, add2(add2(sq2(q2.x), sq2(q2.y)), add2(sq2(q3.x), sq2(q3.y))));
          b1 = add2(b1, add2(add2(sq2(q2.z), sq2(q2.w)), add2(sq2(q3.z), sq2(q3.w))));
        }
        for (; v < nv; v += 32) {
          const uint4 q0 = rowq[v];
          b0 = add2(b0, add2(sq2(q0.x), sq2(q0.y)));
          b1 = add2(b1, add2(sq2(q0.z), sq2(q0.w)));
        }
        const float s2 = warp_sum((b0.x + b0.y) + (b1.x + b1.y));
        if (lane == 0) {
          const float rn = lerp_torch(old, __fdiv_rn(s2, (float)C), hp.w2, hp.w2m1, hp.small_w2 != 0);
          d.stat_a[row] = rn;
          mean2_s[r] = mu2;
          if (gc) pv.aux[aux_mean(d) + row] = mu;
          rinv_s[r] = __fdiv_rn(1.0f, rn);
          rowsum += (double)rn;
        }
      }
    };
    // one vector of four pairs from row r into the two column accumulators
    auto accum = [&](f32x2 A1[4], f32x2 A2[4], const uint4 qv, const int r) {
      const uint32_t mu2 = mean2_s[r];
      const f32x2 RI = pack2(rinv_s[r], rinv_s[r]);
      const uint32_t ww[4] = {qv.x, qv.y, qv.z, qv.w};
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const f32x2 y = pairs(gc ? sub_bf16x2(ww[w], mu2) : ww[w]);
        const f32x2 sq = mul2(y, y);
        A1[w] = add2(A1[w], hp.has_eps ? add2(sq, EPS) : sq);
        A2[w] = add2(A2[w], mul2(sq, RI));
      }
    };
    if (ok && nv <= STT) {
      // Rows of at most 2048 elements: one column vector per thread, its accumulators in registers for the
      // whole item, so rows and columns alternate over sub-groups of rows small enough (about 48 KB) for the
      // column phase to find the rows in L2.  Rows narrower than half the CTA: Q groups of nv threads take
      // every Q-th row and their partial sums are combined in group order.
      const int Q = STT / nv, q = tid / nv, v = tid - q * nv;
      int sg = (48 * 1024) / (C * 2);
      sg = max(STT / 32, sg / (STT / 32) * (STT / 32));
      f32x2 A1[4], A2[4];
#pragma unroll
      for (int w = 0; w < 4; ++w) { A1[w] = pack2(0.0f, 0.0f); A2[w] = pack2(0.0f, 0.0f); }
      for (int ra = 0; ra < nrows; ra += sg) {
        const int rb = min(nrows, ra + sg);
        rows_phase(ra, rb);
        __syncthreads();
        if (q < Q) {
#pragma unroll 4
          for (int r = ra + q; r < rb; r += Q) accum(A1, A2, gitem[(size_t)r * nv + v], r);
        }
      }
      if (Q == 1) {
        if (q < Q) {
          float4* s1 = reinterpret_cast<float4*>(slot + (size_t)v * 8);
          float4* s2 = reinterpret_cast<float4*>(slot + C + (size_t)v * 8);
          s1[0] = make_float4(A1[0].x, A1[0].y, A1[1].x, A1[1].y);
          s1[1] = make_float4(A1[2].x, A1[2].y, A1[3].x, A1[3].y);
          s2[0] = make_float4(A2[0].x, A2[0].y, A2[1].x, A2[1].y);
          s2[1] = make_float4(A2[2].x, A2[2].y, A2[3].x, A2[3].y);
        }
      } else {
        if (q < Q) {
#pragma unroll
          for (int w = 0; w < 4; ++w) {
            xs[(size_t)q * 2 * C + v * 8 + 2 * w] = A1[w].x; xs[(size_t)q * 2 * C + v * 8 + 2 * w + 1] = A1[w].y;
            xs[(size_t)q * 2 * C + C + v * 8 + 2 * w] = A2[w].x; xs[(size_t)q * 2 * C + C + v * 8 + 2 * w + 1] = A2[w].y;
          }
        }
        __syncthreads();
        for (int j = tid; j < 2 * C; j += STT) {
          float tot = 0.0f;
          for (int qq = 0; qq < Q; ++qq) tot += xs[(size_t)qq * 2 * C + j];
          slot[j] = tot;
        }
      }
    } else if (ok) {
      // wider rows: all rows first, then the columns in chunks of ST_VPT vectors per thread
      rows_phase(0, nrows);
      __syncthreads();
      for (int c0 = 0; c0 < nv; c0 += STT * ST_VPT) {
        f32x2 A1[ST_VPT][4], A2[ST_VPT][4];
#pragma unroll
        for (int j = 0; j < ST_VPT; ++j)
#pragma unroll
          for (int w = 0; w < 4; ++w) { A1[j][w] = pack2(0.0f, 0.0f); A2[j][w] = pack2(0.0f, 0.0f); }
        const int v0 = c0 + tid, v1 = v0 + STT;
        if (v1 < nv) {
#pragma unroll 2
          for (int r = 0; r < nrows; ++r) {
            const uint4 qa = gitem[(size_t)r * nv + v0], qb = gitem[(size_t)r * nv + v1];
            accum(A1[0], A2[0], qa, r);
            accum(A1[1], A2[1], qb, r);
          }
        } else if (v0 < nv) {
#pragma unroll 4
          for (int r = 0; r < nrows; ++r) accum(A1[0], A2[0], gitem[(size_t)r * nv + v0], r);
        }
#pragma unroll
        for (int j = 0; j < ST_VPT; ++j) {
          const int v = v0 + j * STT;
          if (v < nv) {
            float4* s1 = reinterpret_cast<float4*>(slot + (size_t)v * 8);
            float4* s2 = reinterpret_cast<float4*>(slot + C + (size_t)v * 8);
            s1[0] = make_float4(A1[j][0].x, A1[j][0].y, A1[j][1].x, A1[j][1].y);
            s1[1] = make_float4(A1[j][2].x, A1[j][2].y, A1[j][3].x, A1[j][3].y);
            s2[0] = make_float4(A2[j][0].x, A2[j][0].y, A2[j][1].x, A2[j][1].y);
            s2[1] = make_float4(A2[j][2].x, A2[j][2].y, A2[j][3].x, A2[j][3].y);
          }
        }
      }
    }
    // ---- the item's row-statistic sum, in warp order ----
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) rowsum += __shfl_xor_sync(0xffffffffu, rowsum, o);
    if (lane == 0) red[warp] = rowsum;
    __syncthreads();
    if (tid == 0) {
      if (ok) {
        double rs = 0.0;
        for (int w = 0; w < STT / 32; ++w) rs += red[w];
        reinterpret_cast<double*>(pv.aux + aux_rowpart(d))[t.slot] = rs;
      }
      __threadfence();  // this item's stores (ordered before the barrier) go out before the signal
      signal_counter(pv.done + 0 * pv.n_tensors + t.tensor, 1u);
    }
    slot_i ^= 1;
    cur = next_s[slot_i];
  }
}

// ----------------------------------------------------------------------------- FINAL

__device__ void ada_final(const PlanView& pv, const AdaDev& hp, const Task& t, const AdaSmem& sm,
                          int tid) {
  const DevTensor d = pv.tensors[t.tensor];
  if (pv.grads[t.tensor] == nullptr) return;
  bool ok = true;
  if (tid == 0) ok = wait_counter(pv.done + 0 * pv.n_tensors + t.tensor, (unsigned)d.n_stats, pv.status, 11001u);
  ok = __syncthreads_and(ok) != 0;
  if (!ok) return;
  const int C = d.cols, j0 = t.row0, nc = t.n;
  const float* part = pv.aux + d.aux_off;
  float* cfac = pv.aux + aux_cfac(d);
  double tl = 0.0;
  for (int j = tid; j < nc; j += AT) {
    float s1 = 0.0f, s2 = 0.0f;
    int s = 0;
    for (; s + 8 <= d.n_stats; s += 8) {  // eight slots' loads in flight; the sums keep the slot order
      float x1[8], x2[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        x1[u] = __ldcg(part + 2ll * (s + u) * C + j0 + j);
        x2[u] = __ldcg(part + 2ll * (s + u) * C + C + j0 + j);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) { s1 += x1[u]; s2 += x2[u]; }
    }
    for (; s < d.n_stats; ++s) {
      s1 += __ldcg(part + 2ll * s * C + j0 + j);
      s2 += __ldcg(part + 2ll * s * C + C + j0 + j);
    }
    const float mean = __fdiv_rn(s1, (float)d.rows);
    const float cn = lerp_torch(d.stat_b[j0 + j], mean, hp.w2, hp.w2m1, hp.small_w2 != 0);
    d.stat_b[j0 + j] = cn;
    cfac[j0 + j] = rsqrt_torch(cn);
    tl += (double)s2 / (double)cn;
  }
  const double tot = block_sum_d(tl, sm.red, tid);
  double* tpart = reinterpret_cast<double*>(pv.aux + aux_tpart(d));
  if (tid == 0) tpart[t.slot] = tot;
  __threadfence();
  __syncthreads();
  int last = 0;
  if (tid == 0) {
    unsigned old;
    asm volatile("atom.acq_rel.gpu.global.add.u32 %0, [%1], 1;" : "=r"(old) : "l"(pv.done + 1 * pv.n_tensors + t.tensor) : "memory");
    if (old == (unsigned)d.n_strips - 1u) {  // last strip: combine, in slot order
      last = 1;
      __threadfence();
      const volatile double* rowpart = reinterpret_cast<const volatile double*>(pv.aux + aux_rowpart(d));
      const volatile double* tp = tpart;
      double rs = 0.0, T = 0.0;
      for (int s = 0; s < d.n_stats; ++s) rs += rowpart[s];
      for (int s = 0; s < d.n_strips; ++s) T += tp[s];
      const float rowmean = __fdiv_rn((float)rs, (float)d.rows);
      const double ss = (double)rowmean * T;
      const float rms = __fdiv_rn((float)sqrt(ss), (float)sqrt((double)d.rows * (double)C));
      float* scal = pv.aux + aux_scal(d);
      scal[0] = rowmean;
      scal[1] = fmaxf(__fdiv_rn(rms, hp.clip), 1.0f);
      scal[2] = rms;
      sm.part_s[0] = rowmean;
    }
  }
  last = __syncthreads_or(last);
  if (last) {  // the whole CTA: r_i of every row, then release COUNT / APPLY
    const float rowmean = sm.part_s[0];
    float* rfac = pv.aux + aux_rfac(d);
    for (int r = tid; r < d.rows; r += AT) rfac[r] = rsqrt_torch(__fdiv_rn(__ldcg(d.stat_a + r), rowmean));
    if (hp.int8) {  // int8 momentum: COUNT starts from zeroed row maxima; APPLY decodes with the old scales
      unsigned* rowmax = reinterpret_cast<unsigned*>(pv.aux + aux_rowmax(d));
      float* oldsc = pv.aux + aux_oldsc(d);
      for (int r = tid; r < d.rows; r += AT) { rowmax[r] = 0u; oldsc[r] = d.m_scale[r]; }
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) signal_counter(pv.done + 2 * pv.n_tensors + t.tensor, 1u);
  }
}

// ----------------------------------------------------------------------------- COUNT / APPLY

// Per-item constants of the update chain.
struct Chain {
  float div, rcp_div;   // clip divisor and its reciprocal
  bool use_div;
};

// u for one element: ((g*r)*c) / divisor * scale  (reference src/kaon/adakaon.py:885-888)
__device__ __forceinline__ float update_of(float g, float r, float c, const Chain& ch, float scale) {
  float u = __fmul_rn(__fmul_rn(g, r), c);
  if (ch.use_div) u = div_shared(u, ch.div, ch.rcp_div);
  return __fmul_rn(u, scale);
}

// momentum EMA on one element in the stored dtype's arithmetic
// (reference src/kaon/_momentum_codec.py:266-270, 303-306)
template <int MK>
__device__ __forceinline__ float ema_of(float m_old, float u, const AdaDev& hp) {
  if constexpr (MK == KAON_M_NONE) return u;
  if constexpr (MK == KAON_M_BF16)
    return round_bf16(lerp_torch(m_old, round_bf16(u), hp.w1, hp.w1m1, hp.small_w1 != 0));
  return lerp_torch(m_old, u, hp.w1, hp.w1m1, hp.small_w1 != 0);
}

// MUON (AdaMuon's factored tensors): the signal is the orthogonalised momentum O (bf16, `pv.signal`), the
// momentum itself was already updated by the EMA pre-pass (so the chain carries none: delta = u), and
// the cautious mask compares delta with the RAW gradient, which is staged where the momentum bytes go
// otherwise (reference src/kaon/adamuon.py:460-497, 605-613).
template <typename PT, int MKP, bool APPLY, bool MUON>
__device__ void ada_rows(const PlanView& pv, const AdaDev& hp, const Task& t, Stage& st,
                         const AdaSmem& sm, int tid) {
  using E = Elems<PT>;
  using S = Elems<typename std::conditional<MUON, __nv_bfloat16, PT>::type>;
  using ST = typename std::conditional<MUON, __nv_bfloat16, PT>::type;
  constexpr int MK = MUON ? KAON_M_NONE : MKP;
  const DevTensor d = pv.tensors[t.tensor];
  const unsigned char* g = reinterpret_cast<const unsigned char*>(pv.grads[t.tensor]);
  const unsigned char* sig = g;
  if (MUON && g != nullptr) sig = reinterpret_cast<const unsigned char*>(pv.signal[t.tensor]);
  if (g == nullptr) {
    if (!APPLY) {
      __syncthreads();
      if (tid == 0) signal_counter(pv.done + 3 * pv.n_tensors + t.tensor, 1u);
    }
    return;
  }
  bool ok = true;
  if (tid == 0) {
    ok = wait_counter(pv.done + 2 * pv.n_tensors + t.tensor, 1u, pv.status, 12001u);
    if (ok && APPLY && hp.cautious)
      ok = wait_counter(pv.done + 3 * pv.n_tensors + t.tensor, (unsigned)d.n_count, pv.status, 13001u);
  }
  ok = __syncthreads_and(ok) != 0;
  const int C = d.cols;
  const int nrows = t.n / C;
  const bool gc = hp.gc != 0 && !MUON;
  // AdaMuon with gradient centralization: the statistics run on the orthogonalised matrix, which is not
  // centralised; the cautious mask compares with the CENTRALISED raw gradient (row means in the scratch)
  const bool gcr = hp.gc != 0 && MUON;
  const float* scal = pv.aux + aux_scal(d);
  const float rowmean = __ldcg(scal + 0);
  Chain ch;
  ch.div = __ldcg(scal + 1);
  ch.use_div = ch.div != 1.0f;
  ch.rcp_div = __fdiv_rn(1.0f, ch.div);
  float denom = 1.0f, rcp_denom = 1.0f;
  if (APPLY && hp.cautious) {
    const unsigned kept = __ldcg(pv.kept + t.tensor);
    denom = fmaxf(__fdiv_rn((float)kept, (float)d.numel), 1e-8f);
    rcp_denom = __fdiv_rn(1.0f, denom);
  }
  // column factors of this tensor -> shared memory (after the momentum bytes in region X)
  float* cfac_s = sm.x_s;
  if (ok) {
    const float* cf = pv.aux + aux_cfac(d);
    for (int j = tid; j < C; j += AT) cfac_s[j] = __ldcg(cf + j);
  }
  const bool row_uniform = (C & 7) == 0;
  SrStream s_upd{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_UPDATE};
  SrStream s_rem{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_REMOVE};
  SrStream s_clb{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_CLIMB};
  const bool sr = hp.sr != 0;
  const bool need_p = APPLY || hp.has_wd;
  unsigned kept_local = 0;

  auto chunk_src = [&](int c0, const unsigned char*& s0, unsigned& b0, const unsigned char*& s1, unsigned& b1) {
    const int nn = min(d.chunk_rows, nrows - c0) * C;
    const long long ee = t.e0 + (long long)c0 * C;
    if (MUON) { s0 = sig + ee * S::BYTES; b0 = (unsigned)nn * S::BYTES; s1 = g + ee * E::BYTES; b1 = (unsigned)nn * E::BYTES; }
    else { s0 = g + ee * E::BYTES; b0 = (unsigned)nn * E::BYTES; s1 = m_ptr<MK>(d, ee); b1 = m_bytes<MK>(nn); }
  };
  auto issue = [&](int c0, int b) {
    const unsigned char *s0, *s1; unsigned b0, b1;
    chunk_src(c0, s0, b0, s1, b1);
    stage_issue(st, b, s0, b0, s1, b1, tid);
  };
  if (ok && st.nbuf == 2) issue(0, 0);
  for (int c0 = 0, ci = 0; ok && c0 < nrows; c0 += d.chunk_rows, ++ci) {
    const int nrc = min(d.chunk_rows, nrows - c0);
    const int n = nrc * C;
    const long long e0 = t.e0 + (long long)c0 * C;
    const int b = st.nbuf == 2 ? (ci & 1) : 0;
    if (st.nbuf == 1) issue(c0, 0);
    else if (c0 + d.chunk_rows < nrows) issue(c0 + d.chunk_rows, b ^ 1);
    // per-row scalars of this chunk: loads go out before the wait for the staged data
    constexpr int RPT = MAX_TASK_ROWS / AT;  // rows per thread at most
    float pre_mu[RPT], pre_row[RPT], pre_sc[RPT];
    unsigned pre_max[RPT];
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
      pre_mu[j] = 0.0f; pre_row[j] = 1.0f; pre_sc[j] = 1.0f; pre_max[j] = 0u;
      const int r = tid + j * AT;
      if (r < nrc) {
        const int row = t.row0 + c0 + r;
        if (gc || gcr) pre_mu[j] = __ldcg(pv.aux + aux_mean(d) + row);
        pre_row[j] = __ldcg(d.stat_a + row);
        if constexpr (MK == KAON_M_INT8) {
          pre_sc[j] = d.m_scale[row];
          // with cautious on, COUNT has already found the row's absmax of the new momentum
          if (APPLY && hp.cautious) pre_max[j] = __ldcg(reinterpret_cast<const unsigned*>(pv.aux + aux_rowmax(d)) + row);
        }
      }
    }
    float pre_blk = 1.0f;
    if constexpr (MK == KAON_M_4BIT) {  // old block scales of the chunk (<= CAP/32 = 512 blocks, one per thread)
      const int nblk = d.bshift >= 31 ? 1 : (int)(blk_of(d, e0 + n - 1) - blk_of(d, e0) + 1);
      if (tid < nblk) pre_blk = d.m_scale[blk_of(d, e0) + tid];
    }
    {
      const unsigned char *s0, *s1; unsigned b0, b1;
      chunk_src(c0, s0, b0, s1, b1);
      ok = stage_wait(st, b, s0, b0, s1, b1, pv.status);
    }
    if (!ok) break;
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
      const int r = tid + j * AT;
      if (r < nrc) {
        sm.mean_s[r] = pre_mu[j];
        sm.rfac_s[r] = rsqrt_torch(__fdiv_rn(pre_row[j], rowmean));
        if constexpr (MK == KAON_M_INT8) {
          sm.scale_s[r] = pre_sc[j];
          sm.rowmax_s[r] = pre_max[j];
        }
      }
    }
    if constexpr (MK == KAON_M_4BIT) {
      const int nblk = d.bshift >= 31 ? 1 : (int)(blk_of(d, e0 + n - 1) - blk_of(d, e0) + 1);
      if (tid < nblk) sm.scale_s[tid] = pre_blk;
    }
    __syncthreads();
    unsigned char* pbase = reinterpret_cast<unsigned char*>(d.p) + e0 * E::BYTES;
    const int nvec = (n + 7) >> 3;
    const int nvec_pad = (nvec + 31) & ~31;

    // One vector of the chain: fills g', the new momentum mn[], the pre-update weights pc[] (after the
    // Nekaon removal) and delta dl[]; returns the kept bits.
    // the weights this thread will touch in this chunk: all loads go out before the first use
    constexpr int VPT = CAP / 8 / AT;
    constexpr int PW = E::BYTES / 2;  // 16-byte words per eight weights
    uint4 pre_p[VPT * PW];
    const bool preload = need_p && row_uniform && (n & 7) == 0;
    if (preload) {
#pragma unroll
      for (int j = 0; j < VPT; ++j) {
        const int v = tid + j * AT;
        if (v < nvec) {
#pragma unroll
          for (int w = 0; w < PW; ++w) pre_p[j * PW + w] = reinterpret_cast<const uint4*>(pbase + (size_t)v * 8 * E::BYTES)[w];
        }
      }
    }

    auto chain8 = [&](int v, int cnt, float gv[8], float mo[8], float mn[8], float pc[8], float dl[8]) -> unsigned {
      if (row_uniform && cnt == 8) {
        // full vector inside one row: one row lookup, vector loads, no guards
        S::load8(st.g_s + (size_t)v * 8 * S::BYTES, gv);
        float raw[8];
        if (MUON) E::load8(st.m_s + (size_t)v * 8 * E::BYTES, raw);
        const int r = row_of((unsigned)v * 8u, d);
        const float rf = sm.rfac_s[r], mu = sm.mean_s[r];
        if (MUON && gcr) {
#pragma unroll
          for (int k = 0; k < 8; ++k) raw[k] = centered<PT>(raw[k], mu, true);
        }
        const float4 c0 = *reinterpret_cast<const float4*>(cfac_s + (v * 8 - r * C));
        const float4 c1 = *reinterpret_cast<const float4*>(cfac_s + (v * 8 - r * C) + 4);
        const float cf[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
        if constexpr (MK == KAON_M_4BIT) decode8<MK>(st.m_s, v, 8, sm.scale_s[d.bshift >= 31 ? 0 : (v >> (d.bshift - 3))], mo);
        else if constexpr (MK == KAON_M_INT8) decode8<MK>(st.m_s, v, 8, sm.scale_s[r], mo);
        else if constexpr (MK == KAON_M_NONE) {
#pragma unroll
          for (int k = 0; k < 8; ++k) mo[k] = 0.0f;
        } else decode8<MK>(st.m_s, v, 8, 1.0f, mo);
        if (need_p) {
          if (preload) E::load8(&pre_p[((v - tid) / AT) * PW], pc);
          else E::load8(pbase + (size_t)v * 8 * E::BYTES, pc);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) pc[k] = 0.0f;
        }
        if (hp.remove && need_p) {
          uint32_t nz[4] = {0u, 0u, 0u, 0u};
          if (E::IS_BF16) s_rem.draw8(d.tensor_id, (uint64_t)((e0 >> 3) + v), nz);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            pc[k] = write_step<PT>(pc[k], climb_e(mo[k], hp.a_remove, hp.b_remove), 1.0f, E::IS_BF16, noise_lane(nz, k));
        }
        if (gc) {
#pragma unroll
          for (int k = 0; k < 8; k += 2) {
            const float x0 = __fsub_rn(gv[k], mu), x1 = __fsub_rn(gv[k + 1], mu);
            if (E::IS_BF16) {
              const uint32_t pk = pack_bf16_rn(x0, x1);
              gv[k] = bf16lo(pk); gv[k + 1] = bf16hi(pk);
            } else {
              gv[k] = x0; gv[k + 1] = x1;
            }
          }
        }
        unsigned keptf = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float u = update_of(gv[k], rf, cf[k], ch, hp.upd_scale);
          mn[k] = ema_of<MK>(mo[k], u, hp);
          const float dv = hp.has_wd ? __fmaf_rn(pc[k], hp.lrwd, mn[k]) : mn[k];
          dl[k] = dv;
          if (__fmul_rn(dv, MUON ? raw[k] : gv[k]) > 0.0f) keptf |= 1u << k;
        }
        return keptf;
      }
      load8_guard<ST>(st.g_s + (size_t)v * 8 * S::BYTES, cnt, gv);
      float raw[8];  // MUON: the raw gradient, the cautious mask's reference
      if (MUON) load8_guard<PT>(st.m_s + (size_t)v * 8 * E::BYTES, cnt, raw);
      int rl[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) rl[k] = row_uniform ? row_of((unsigned)v * 8u, d) : row_of((unsigned)(v * 8 + min(k, max(cnt - 1, 0))), d);
      if (MUON && gcr) {
#pragma unroll
        for (int k = 0; k < 8; ++k) raw[k] = (k < cnt) ? centered<PT>(raw[k], sm.mean_s[rl[k]], true) : 0.0f;
      }
      // old momentum
      if constexpr (MK == KAON_M_4BIT) {
        decode8<MK>(st.m_s, v, cnt, cnt > 0 ? sm.scale_s[d.bshift >= 31 ? 0 : (v >> (d.bshift - 3))] : 1.0f, mo);
      } else if constexpr (MK == KAON_M_INT8) {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          mo[k] = (k < cnt) ? __fmul_rn((float)(signed char)st.m_s[v * 8 + k], sm.scale_s[rl[k]]) : 0.0f;
      } else if constexpr (MK == KAON_M_NONE) {
#pragma unroll
        for (int k = 0; k < 8; ++k) mo[k] = 0.0f;
      } else {
        decode8<MK>(st.m_s, v, cnt, 1.0f, mo);
      }
      if (need_p && cnt > 0) load8_guard<PT>(pbase + (size_t)v * 8 * E::BYTES, cnt, pc);
      else {
#pragma unroll
        for (int k = 0; k < 8; ++k) pc[k] = 0.0f;
      }
      if (hp.remove && need_p && cnt > 0) {  // take the previous climb back out first
        uint32_t nz[4] = {0u, 0u, 0u, 0u};
        if (E::IS_BF16) s_rem.draw8(d.tensor_id, (uint64_t)((e0 >> 3) + v), nz);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          pc[k] = write_step<PT>(pc[k], climb_e(mo[k], hp.a_remove, hp.b_remove), 1.0f, true && E::IS_BF16, noise_lane(nz, k));
      }
      unsigned kept = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float col = cfac_s[(v * 8 + k) - rl[k] * C < C ? (v * 8 + k) - rl[k] * C : 0];
        const float x = (k < cnt) ? centered<PT>(gv[k], sm.mean_s[rl[k]], gc) : 0.0f;
        gv[k] = x;
        const float u = update_of(x, sm.rfac_s[rl[k]], col, ch, hp.upd_scale);
        mn[k] = (k < cnt) ? ema_of<MK>(mo[k], u, hp) : 0.0f;
        const float dv = hp.has_wd ? __fmaf_rn(pc[k], hp.lrwd, mn[k]) : mn[k];
        dl[k] = dv;
        if (k < cnt && __fmul_rn(dv, MUON ? raw[k] : x) > 0.0f) kept |= 1u << k;
      }
      return kept;
    };

    if constexpr (APPLY && MK == KAON_M_INT8) if (!hp.cautious) {  // row absmax of the new momentum first
      for (int v = tid; v < nvec; v += AT) {
        const int cnt = min(8, n - v * 8);
        float gv[8], mo[8], mn[8], pc[8], dl[8];
        chain8(v, cnt, gv, mo, mn, pc, dl);
        if (row_uniform) {
          float a = 0.0f;
#pragma unroll
          for (int k = 0; k < 8; ++k) a = fmaxf(a, fabsf(mn[k]));
          atomicMax(sm.rowmax_s + row_of((unsigned)v * 8u, d), __float_as_uint(a));
        } else {
          for (int k = 0; k < cnt; ++k) atomicMax(sm.rowmax_s + row_of((unsigned)(v * 8 + k), d), __float_as_uint(fabsf(mn[k])));
        }
      }
      __syncthreads();
    }

    for (int v = tid; v < nvec_pad; v += AT) {
      const int cnt = max(0, min(8, n - v * 8));
      float gv[8], mo[8], mn[8], pc[8], dl[8];
      unsigned kept = 0;
      if (cnt > 0) kept = chain8(v, cnt, gv, mo, mn, pc, dl);
      else {
#pragma unroll
        for (int k = 0; k < 8; ++k) { mn[k] = 0.0f; mo[k] = 0.0f; pc[k] = 0.0f; dl[k] = 0.0f; gv[k] = 0.0f; }
      }
      if constexpr (!APPLY) {
        kept_local += __popc(kept);
        if constexpr (MK == KAON_M_INT8) {  // leave the row absmax of the new momentum for APPLY
          if (cnt > 0) {
            if (row_uniform) {
              float a = 0.0f;
#pragma unroll
              for (int k = 0; k < 8; ++k) a = fmaxf(a, fabsf(mn[k]));
              atomicMax(sm.rowmax_s + row_of((unsigned)v * 8u, d), __float_as_uint(a));
            } else {
              for (int k = 0; k < cnt; ++k) atomicMax(sm.rowmax_s + row_of((unsigned)(v * 8 + k), d), __float_as_uint(fabsf(mn[k])));
            }
          }
        }
      } else {
        float md[8];  // the momentum as stored (decoded), for the Nekaon climb
        // ---- encode + store the new momentum ----
        if constexpr (MK == KAON_M_4BIT) {
          float a = 0.0f;
#pragma unroll
          for (int k = 0; k < 8; ++k) a = fmaxf(a, fabsf(mn[k]));
          a = fmaxf(group_max(a, blk_lanes(d)), 1e-12f);
          const float sc = __fdiv_rn(a, 7.0f);
          const float inv = __fdividef(1.0f, sc);
          uint32_t word = 0;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float q = quant_round(mn[k], sc, inv, 1e-4f);
            const int qi = min(max((int)q, -7), 7);
            md[k] = __fmul_rn((float)qi, sc);
            if (k < cnt) word |= (uint32_t)(qi + 8) << (4 * k);
          }
          if (cnt > 0) {
            unsigned char* mdst = (unsigned char*)d.m + (e0 >> 1) + (size_t)v * 4;
            if (cnt == 8) *reinterpret_cast<uint32_t*>(mdst) = word;
            else
              for (int b = 0; b < (cnt + 1) / 2; ++b) mdst[b] = (unsigned char)(word >> (8 * b));
            if ((v & (blk_lanes(d) - 1)) == 0) d.m_scale[blk_of(d, e0 + (long long)v * 8)] = sc;
          }
        } else if constexpr (MK == KAON_M_INT8) {
          if (cnt > 0) {
            unsigned char* mdst = (unsigned char*)d.m + e0 + (size_t)v * 8;
            uint32_t w0 = 0, w1 = 0;
            float sc = 0.0f, inv = 0.0f;
            int rprev = -1;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              md[k] = 0.0f;
              if (k < cnt) {
                const int r = row_uniform ? row_of((unsigned)v * 8u, d) : row_of((unsigned)(v * 8 + k), d);
                if (r != rprev) {
                  sc = __fdiv_rn(fmaxf(__uint_as_float(sm.rowmax_s[r]), 1e-12f), 127.0f);
                  inv = __fdividef(1.0f, sc);
                  rprev = r;
                  if ((unsigned)(v * 8 + k) == (unsigned)r * (unsigned)C) d.m_scale[t.row0 + c0 + r] = sc;
                }
                const int qi = min(max((int)quant_round(mn[k], sc, inv, 1e-3f), -127), 127);
                md[k] = __fmul_rn((float)qi, sc);
                const uint32_t byte = (uint32_t)(qi & 0xFF);
                if (k < 4) w0 |= byte << (8 * k); else w1 |= byte << (8 * (k - 4));
              }
            }
            if (cnt == 8) *reinterpret_cast<uint2*>(mdst) = make_uint2(w0, w1);
            else
              for (int k = 0; k < cnt; ++k) mdst[k] = (unsigned char)((k < 4 ? w0 >> (8 * k) : w1 >> (8 * (k - 4))) & 0xFF);
          }
        } else if constexpr (MK == KAON_M_BF16 || MK == KAON_M_F32) {
#pragma unroll
          for (int k = 0; k < 8; ++k) md[k] = mn[k];
          if (cnt > 0) {
            if constexpr (MK == KAON_M_BF16) store8<__nv_bfloat16>((unsigned char*)d.m + e0 * 2 + (size_t)v * 16, cnt, mn, nullptr);
            else store8<float>((unsigned char*)d.m + e0 * 4 + (size_t)v * 32, cnt, mn, nullptr);
          }
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) md[k] = 0.0f;
        }
        // ---- weights: update, then the new climb ----
        if (cnt > 0) {
          if (E::IS_BF16 && hp.kahan) {
            // compensated write: the tensor's shift buffer is read and written alongside the weights
            unsigned char* she = reinterpret_cast<unsigned char*>(d.shift) + (size_t)e0 * 2 + (size_t)v * 16;
            float sh[8];
            load8_guard<__nv_bfloat16>(she, cnt, sh);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              float f = dl[k];
              if (hp.cautious) f = ((kept >> k) & 1u) ? div_shared(f, denom, rcp_denom) : 0.0f;
              kahan_step(pc[k], sh[k], f);
            }
            store8<__nv_bfloat16>(she, cnt, sh, nullptr);
          } else {
            uint32_t nz[4] = {0u, 0u, 0u, 0u};
            if (sr) s_upd.draw8(d.tensor_id, (uint64_t)((e0 >> 3) + v), nz);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              float f = dl[k];
              if (hp.cautious) f = ((kept >> k) & 1u) ? div_shared(f, denom, rcp_denom) : 0.0f;
              pc[k] = write_step<PT>(pc[k], f, -1.0f, sr, noise_lane(nz, k));
            }
          }
          if (hp.climb && MK != KAON_M_NONE) {
            uint32_t nc[4] = {0u, 0u, 0u, 0u};
            if (E::IS_BF16) s_clb.draw8(d.tensor_id, (uint64_t)((e0 >> 3) + v), nc);
#pragma unroll
            for (int k = 0; k < 8; ++k)
              pc[k] = write_step<PT>(pc[k], climb_e(md[k], hp.a_climb, hp.b_climb), 1.0f, E::IS_BF16, noise_lane(nc, k));
          }
          store8<PT>(pbase + (size_t)v * 8 * E::BYTES, cnt, pc, &pv.peers);
        }
      }
    }
    __syncthreads();
    if constexpr (!APPLY && MK == KAON_M_INT8) {
      unsigned* rm = reinterpret_cast<unsigned*>(pv.aux + aux_rowmax(d)) + t.row0 + c0;
      for (int r = tid; r < nrc; r += AT) rm[r] = sm.rowmax_s[r];
      __syncthreads();
    }
  }
  if constexpr (!APPLY) {
    const unsigned tot = block_sum_u(kept_local, sm.red, tid);
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      if (ok) atomicAdd(pv.kept + t.tensor, tot);
      signal_counter(pv.done + 3 * pv.n_tensors + t.tensor, 1u);
    }
  }
}

// ----------------------------------------------------------------------------- COUNT / APPLY, streaming

// The same two work items for the common case - rows a multiple of 8 elements, gradient as the signal -
// without shared-memory staging and without a barrier in the loop: every thread streams its vectors
// straight from global memory (gradient, momentum, weights) and fetches what is per row or per column
// (centralization mean, row statistic, column factor, int8 scales) from L2, where the earlier stages
// left it.  Rows of an item belong to this CTA alone, so the int8 row maxima are reduced with
// atomicMax on the tensor's scratch (COUNT) and the old row scales are set aside once per item (APPLY).
// Results are bit-identical to ada_rows: same arithmetic, same noise indices.
template <typename PT, int MKP, bool APPLY, bool MUON>
__device__ void ada_stream(const PlanView& pv, const AdaDev& hp, const Task& t, const AdaSmem& sm, int tid) {
  using E = Elems<PT>;
  using S = Elems<typename std::conditional<MUON, __nv_bfloat16, PT>::type>;  // the signal's element type
  constexpr int MK = MUON ? KAON_M_NONE : MKP;
  const DevTensor d = pv.tensors[t.tensor];
  const unsigned char* g = reinterpret_cast<const unsigned char*>(pv.grads[t.tensor]);
  if (g == nullptr) {
    if (!APPLY) {
      __syncthreads();
      if (tid == 0) signal_counter(pv.done + 3 * pv.n_tensors + t.tensor, 1u);
    }
    return;
  }
  bool ok = true;
  if (tid == 0) {
    ok = wait_counter(pv.done + 2 * pv.n_tensors + t.tensor, 1u, pv.status, 12001u);
    if (ok && APPLY && hp.cautious)
      ok = wait_counter(pv.done + 3 * pv.n_tensors + t.tensor, (unsigned)d.n_count, pv.status, 13001u);
  }
  ok = __syncthreads_and(ok) != 0;
  const int C = d.cols;
  const int nrows = t.n / C;
  const bool gc = hp.gc != 0 && !MUON;
  // AdaMuon with gradient centralization: the statistics run on the orthogonalised matrix, which is not
  // centralised; the cautious mask compares with the CENTRALISED raw gradient (row means in the scratch)
  const bool gcr = hp.gc != 0 && MUON;
  // AdaMuon: the chain runs on the orthogonalised momentum, the cautious mask on the raw gradient
  const unsigned char* sig = MUON ? reinterpret_cast<const unsigned char*>(pv.signal[t.tensor]) : g;
  const float* scal = pv.aux + aux_scal(d);
  const float rowmean = __ldcg(scal + 0);
  Chain ch;
  ch.div = __ldcg(scal + 1);
  ch.use_div = ch.div != 1.0f;
  ch.rcp_div = __fdiv_rn(1.0f, ch.div);
  float denom = 1.0f, rcp_denom = 1.0f;
  if (APPLY && hp.cautious) {
    const unsigned kept = __ldcg(pv.kept + t.tensor);
    denom = fmaxf(__fdiv_rn((float)kept, (float)d.numel), 1e-8f);
    rcp_denom = __fdiv_rn(1.0f, denom);
  }
  const float* cfac = pv.aux + aux_cfac(d);
  const float* mean = pv.aux + aux_mean(d);
  unsigned* rowmax = reinterpret_cast<unsigned*>(pv.aux + aux_rowmax(d));
  float* oldsc = pv.aux + aux_oldsc(d);
  const float* rfac = pv.aux + aux_rfac(d);
  SrStream s_upd{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_UPDATE};
  SrStream s_rem{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_REMOVE};
  SrStream s_clb{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_CLIMB};
  const bool sr = hp.sr != 0;
  const bool need_p = APPLY || hp.has_wd;
  const int lane = tid & 31;
  unsigned kept_local = 0;

  for (int c0 = 0; ok && c0 < nrows; c0 += d.chunk_rows) {
    const int nrc = min(d.chunk_rows, nrows - c0);
    const int nvec = (nrc * C) >> 3;
    const int nvec_pad = (nvec + 31) & ~31;
    const long long e0 = t.e0 + (long long)c0 * C;
    const unsigned char* gbase = sig + e0 * S::BYTES;
    const unsigned char* rawbase = g + e0 * E::BYTES;
    const unsigned char* mbase = m_ptr<MK>(d, e0);
    unsigned char* pbase = reinterpret_cast<unsigned char*>(d.p) + e0 * E::BYTES;
    for (int v = tid; v < nvec_pad; v += AT) {
      const bool act = v < nvec;
      const int vv = act ? v : 0;
      const int r = row_of((unsigned)vv * 8u, d);
      const int row = t.row0 + c0 + r;
      const int col = vv * 8 - r * C;
      float gv[8], mo[8], mn[8], pc[8], dl[8];
      // ---- loads ----
      S::load8(gbase + (size_t)vv * 8 * S::BYTES, gv);
      float raw[8];
      if (MUON) E::load8(rawbase + (size_t)vv * 8 * E::BYTES, raw);
      if (need_p) E::load8(pbase + (size_t)vv * 8 * E::BYTES, pc);
      else {
#pragma unroll
        for (int k = 0; k < 8; ++k) pc[k] = 0.0f;
      }
      const float mu = (gc || gcr) ? __ldcg(mean + row) : 0.0f;
      if (MUON && gcr) {
#pragma unroll
        for (int k = 0; k < 8; ++k) raw[k] = centered<PT>(raw[k], mu, true);
      }
      const float rf = __ldcg(rfac + row);
      const float4 c0v = __ldcg(reinterpret_cast<const float4*>(cfac + col));
      const float4 c1v = __ldcg(reinterpret_cast<const float4*>(cfac + col + 4));
      const float cf[8] = {c0v.x, c0v.y, c0v.z, c0v.w, c1v.x, c1v.y, c1v.z, c1v.w};
      if constexpr (MK == KAON_M_4BIT) {
        const float sc_old = d.m_scale[d.block == 128u ? ((e0 >> 7) + (vv >> 4)) : 0];
        decode8<MK>(mbase, vv, 8, sc_old, mo);
      } else if constexpr (MK == KAON_M_INT8) {
        const float sc_old = APPLY ? __ldcg(oldsc + row) : d.m_scale[row];
        decode8<MK>(mbase, vv, 8, sc_old, mo);
      } else if constexpr (MK == KAON_M_NONE) {
#pragma unroll
        for (int k = 0; k < 8; ++k) mo[k] = 0.0f;
      } else {
        decode8<MK>(mbase, vv, 8, 1.0f, mo);
      }
      // ---- the chain ----
      if (hp.remove && need_p) {
        uint32_t nz[4] = {0u, 0u, 0u, 0u};
        if (E::IS_BF16) s_rem.draw8(d.tensor_id, (uint64_t)((e0 >> 3) + vv), nz);
#pragma unroll
        for (int k = 0; k < 8; ++k)
          pc[k] = write_step<PT>(pc[k], climb_e(mo[k], hp.a_remove, hp.b_remove), 1.0f, E::IS_BF16, noise_lane(nz, k));
      }
      if (gc) {
#pragma unroll
        for (int k = 0; k < 8; k += 2) {
          const float x0 = __fsub_rn(gv[k], mu), x1 = __fsub_rn(gv[k + 1], mu);
          if (E::IS_BF16) {
            const uint32_t pk = pack_bf16_rn(x0, x1);
            gv[k] = bf16lo(pk); gv[k + 1] = bf16hi(pk);
          } else {
            gv[k] = x0; gv[k + 1] = x1;
          }
        }
      }
      unsigned kept = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const float u = update_of(gv[k], rf, cf[k], ch, hp.upd_scale);
        mn[k] = ema_of<MK>(mo[k], u, hp);
        const float dv = hp.has_wd ? __fmaf_rn(pc[k], hp.lrwd, mn[k]) : mn[k];
        dl[k] = dv;
        if (__fmul_rn(dv, MUON ? raw[k] : gv[k]) > 0.0f) kept |= 1u << k;
      }
      if constexpr (!APPLY) {
        if (act) kept_local += __popc(kept);
        if constexpr (MK == KAON_M_INT8) {
          float a = 0.0f;
#pragma unroll
          for (int k = 0; k < 8; ++k) a = fmaxf(a, fabsf(mn[k]));
          unsigned bits = act ? __float_as_uint(a) : 0u;
          const int row_l0 = __shfl_sync(0xffffffffu, row, 0);
          if (__all_sync(0xffffffffu, !act || row == row_l0)) {
            bits = __reduce_max_sync(0xffffffffu, bits);
            if (lane == 0 && bits) atomicMax(rowmax + row_l0, bits);
          } else if (act) {
            atomicMax(rowmax + row, bits);
          }
        }
      } else {
        float md[8];  // the momentum as stored (decoded), for the Nekaon climb
        if constexpr (MK == KAON_M_4BIT) {
          float a = 0.0f;
#pragma unroll
          for (int k = 0; k < 8; ++k) a = fmaxf(a, act ? fabsf(mn[k]) : 0.0f);
          a = fmaxf(group_max(a, 16), 1e-12f);
          __syncwarp();  // every lane of the block has read the old scale before it is replaced
          const float sc = __fdiv_rn(a, 7.0f);
          const float inv = __fdividef(1.0f, sc);
          uint32_t word = 0;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float q = quant_round(mn[k], sc, inv, 1e-4f);
            const int qi = min(max((int)q, -7), 7);
            md[k] = __fmul_rn((float)qi, sc);
            word |= (uint32_t)(qi + 8) << (4 * k);
          }
          if (act) {
            *reinterpret_cast<uint32_t*>((unsigned char*)d.m + (e0 >> 1) + (size_t)v * 4) = word;
            if ((v & 15) == 0) d.m_scale[(d.block == 128u) ? ((e0 >> 7) + (v >> 4)) : 0] = sc;
          }
        } else if constexpr (MK == KAON_M_INT8) {
          const float sc = __fdiv_rn(fmaxf(__uint_as_float(__ldcg(rowmax + row)), 1e-12f), 127.0f);
          const float inv = __fdividef(1.0f, sc);
          uint32_t w0 = 0, w1 = 0;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int qi = min(max((int)quant_round(mn[k], sc, inv, 1e-3f), -127), 127);
            md[k] = __fmul_rn((float)qi, sc);
            const uint32_t byte = (uint32_t)(qi & 0xFF);
            if (k < 4) w0 |= byte << (8 * k); else w1 |= byte << (8 * (k - 4));
          }
          if (act) {
            *reinterpret_cast<uint2*>((unsigned char*)d.m + e0 + (size_t)v * 8) = make_uint2(w0, w1);
            if (col == 0) d.m_scale[row] = sc;
          }
        } else if constexpr (MK == KAON_M_BF16 || MK == KAON_M_F32) {
#pragma unroll
          for (int k = 0; k < 8; ++k) md[k] = mn[k];
          if (act) {
            if constexpr (MK == KAON_M_BF16) store8<__nv_bfloat16>((unsigned char*)d.m + e0 * 2 + (size_t)v * 16, 8, mn, nullptr);
            else store8<float>((unsigned char*)d.m + e0 * 4 + (size_t)v * 32, 8, mn, nullptr);
          }
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) md[k] = 0.0f;
        }
        if (act) {
          if (E::IS_BF16 && hp.kahan) {
            unsigned char* she = reinterpret_cast<unsigned char*>(d.shift) + (size_t)e0 * 2 + (size_t)v * 16;
            float sh[8];
            load8_guard<__nv_bfloat16>(she, 8, sh);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              float f = dl[k];
              if (hp.cautious) f = ((kept >> k) & 1u) ? div_shared(f, denom, rcp_denom) : 0.0f;
              kahan_step(pc[k], sh[k], f);
            }
            store8<__nv_bfloat16>(she, 8, sh, nullptr);
          } else {
            uint32_t nz[4] = {0u, 0u, 0u, 0u};
            if (sr) s_upd.draw8(d.tensor_id, (uint64_t)((e0 >> 3) + v), nz);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              float f = dl[k];
              if (hp.cautious) f = ((kept >> k) & 1u) ? div_shared(f, denom, rcp_denom) : 0.0f;
              pc[k] = write_step<PT>(pc[k], f, -1.0f, sr, noise_lane(nz, k));
            }
          }
          if (hp.climb && MK != KAON_M_NONE) {
            uint32_t nc[4] = {0u, 0u, 0u, 0u};
            if (E::IS_BF16) s_clb.draw8(d.tensor_id, (uint64_t)((e0 >> 3) + v), nc);
#pragma unroll
            for (int k = 0; k < 8; ++k)
              pc[k] = write_step<PT>(pc[k], climb_e(md[k], hp.a_climb, hp.b_climb), 1.0f, E::IS_BF16, noise_lane(nc, k));
          }
          store8<PT>(pbase + (size_t)v * 8 * E::BYTES, 8, pc, &pv.peers);
        }
      }
    }
  }
  if constexpr (!APPLY) {
    const unsigned tot = block_sum_u(kept_local, sm.red, tid);
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      if (ok) atomicAdd(pv.kept + t.tensor, tot);
      signal_counter(pv.done + 3 * pv.n_tensors + t.tensor, 1u);
    }
  }
}

// Whether the streaming form handles this tensor and these settings (otherwise: ada_rows).
template <int MK>
__device__ __forceinline__ bool stream_ok(const DevTensor& d, const AdaDev& hp, const void* g, const void* sig) {
  if ((d.cols & 7) != 0) return false;
  if ((reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(sig)) & 15) return false;  // 16-byte vector loads
  if (MK == KAON_M_4BIT && d.block != 128u) return false;
  if (MK == KAON_M_INT8 && !hp.cautious) return false;  // no COUNT item to find the row maxima
  return true;
}

// ----------------------------------------------------------------------------- FLAT (1-D tensors)

// reference src/kaon/adakaon.py:908-966: full second moment v, no factoring, no centralization.
// The whole tensor is one work item, so every tensor-wide reduction is CTA-local.  Up to CAP elements
// the gradient and the momentum are staged and the intermediate lives in shared memory; a longer
// tensor (t.slot != 0) is streamed from global memory pass by pass, with the intermediate and the
// block maxima in the tensor's scratch.
template <typename PT, int MK>
__device__ void ada_flat(const PlanView& pv, const AdaDev& hp, const Task& t, Stage& st,
                         const AdaSmem& sm, int tid) {
  using E = Elems<PT>;
  const DevTensor d = pv.tensors[t.tensor];
  const unsigned char* g = reinterpret_cast<const unsigned char*>(pv.grads[t.tensor]);
  if (g == nullptr) return;
  const int n = t.n;
  const bool lng = t.slot != 0;
  if (!lng) {
    stage_issue(st, 0, g, (unsigned)n * E::BYTES, m_ptr<MK>(d, 0), m_bytes<MK>(n), tid);
    if (!stage_wait(st, 0, g, (unsigned)n * E::BYTES, m_ptr<MK>(d, 0), m_bytes<MK>(n), pv.status)) return;
  }
  const unsigned char* g_src = lng ? g : st.g_s;
  const unsigned char* m_src = lng ? reinterpret_cast<const unsigned char*>(d.m) : st.m_s;
  float* f_s = lng ? pv.aux + d.aux_off + 8 : sm.x_s;  // u, then the new momentum
  float* v = d.stat_a;
  // 1. second moment, raw update, its rms
  double ss = 0.0;
  for (int i = tid; i < n; i += AT) {
    const float x = E::load1(g_src, i);
    float sq = __fmul_rn(x, x);
    if (hp.has_eps) sq = __fadd_rn(sq, hp.eps1);
    const float vn = lerp_torch(v[i], sq, hp.w2, hp.w2m1, hp.small_w2 != 0);
    v[i] = vn;
    const float u = __fmul_rn(x, rsqrt_torch(vn));
    f_s[i] = u;
    ss += (double)u * (double)u;
  }
  ss = block_sum_d(ss, sm.red, tid);
  const float rms = __fdiv_rn((float)sqrt(ss), (float)sqrt((double)n));
  const float div = fmaxf(__fdiv_rn(rms, hp.clip), 1.0f);
  // 2. momentum EMA (pre-requant value kept in f_s), absmax per scale group
  const bool one_block = MK == KAON_M_4BIT && d.bshift >= 31;
  const int bsh = one_block ? 0 : d.bshift;  // 4-bit: element -> block
  // 4bit: one entry per 128-block; int8: entry 0
  unsigned* blkmax = lng ? reinterpret_cast<unsigned*>(f_s + flat_long_pad(n)) : sm.rowmax_s;
  const int nblk = lng ? (n + 31) / 32 + 1 : MAX_TASK_ROWS;
  for (int i = tid; i < nblk; i += AT) blkmax[i] = 0u;
  __syncthreads();
  auto old_m = [&](int i) -> float {
    if constexpr (MK == KAON_M_4BIT) {
      const unsigned byte = m_src[i >> 1];
      const int nib = (i & 1) ? (byte >> 4) & 0xF : byte & 0xF;
      return __fmul_rn((float)(nib - 8), d.m_scale[one_block ? 0 : (i >> bsh)]);
    } else if constexpr (MK == KAON_M_INT8) {
      return __fmul_rn((float)(signed char)m_src[i], d.m_scale[0]);
    } else if constexpr (MK == KAON_M_BF16) {
      return Elems<__nv_bfloat16>::load1(m_src, i);
    } else if constexpr (MK == KAON_M_F32) {
      return reinterpret_cast<const float*>(m_src)[i];
    } else {
      return 0.0f;
    }
  };
  for (int i = tid; i < n; i += AT) {
    const float u = __fmul_rn(__fdiv_rn(f_s[i], div), hp.upd_scale);
    const float mn = ema_of<MK>(old_m(i), u, hp);
    f_s[i] = mn;
    if constexpr (MK == KAON_M_4BIT) atomicMax(blkmax + (one_block ? 0 : (i >> bsh)), __float_as_uint(fabsf(mn)));
    if constexpr (MK == KAON_M_INT8) atomicMax(blkmax, __float_as_uint(fabsf(mn)));
  }
  __syncthreads();
  // 3. weights before the update (Nekaon removal), delta, kept count
  SrStream s_upd{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_UPDATE};
  SrStream s_rem{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_REMOVE};
  SrStream s_clb{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_CLIMB};
  auto noise_of = [&](const SrStream& s, int i) -> uint32_t {
    uint32_t nz[4];
    s.draw8(d.tensor_id, (uint64_t)(i >> 3), nz);
    return noise_lane(nz, i & 7);
  };
  auto p_before = [&](int i) -> float {
    float pv0 = E::load1(d.p, i);
    if (hp.remove && MK != KAON_M_NONE)
      pv0 = write_step<PT>(pv0, climb_e(old_m(i), hp.a_remove, hp.b_remove), 1.0f, E::IS_BF16,
                           E::IS_BF16 ? noise_of(s_rem, i) : 0u);
    return pv0;
  };
  unsigned kept_local = 0;
  if (hp.cautious) {
    for (int i = tid; i < n; i += AT) {
      const float dv = hp.has_wd ? __fmaf_rn(p_before(i), hp.lrwd, f_s[i]) : f_s[i];
      if (__fmul_rn(dv, E::load1(g_src, i)) > 0.0f) ++kept_local;
    }
  }
  const unsigned kept = block_sum_u(kept_local, sm.red, tid);
  if (tid == 0) pv.kept[t.tensor] = kept;
  const float denom = fmaxf(__fdiv_rn((float)kept, (float)n), 1e-8f);
  // 4. encode the momentum, write the weights
  auto scale_of = [&](int i) -> float {
    if constexpr (MK == KAON_M_4BIT) return __fdiv_rn(fmaxf(__uint_as_float(blkmax[one_block ? 0 : (i >> bsh)]), 1e-12f), 7.0f);
    else if constexpr (MK == KAON_M_INT8) return __fdiv_rn(fmaxf(__uint_as_float(blkmax[0]), 1e-12f), 127.0f);
    else return 1.0f;
  };
  auto code_of = [&](int i, float sc) -> int {
    const float lim = MK == KAON_M_4BIT ? 7.0f : 127.0f;
    return (int)fminf(fmaxf(rintf(__fdiv_rn(f_s[i], sc)), -lim), lim);
  };
  for (int i = tid; i < n; i += AT) {
    const float pv0 = p_before(i);
    float dv = hp.has_wd ? __fmaf_rn(pv0, hp.lrwd, f_s[i]) : f_s[i];
    if (hp.cautious) dv = (__fmul_rn(dv, E::load1(g_src, i)) > 0.0f) ? __fdiv_rn(dv, denom) : 0.0f;
    float pn;
    if (E::IS_BF16 && hp.kahan) {
      uint16_t* shp = reinterpret_cast<uint16_t*>(d.shift) + i;
      float sh = __uint_as_float((uint32_t)*shp << 16);
      pn = pv0;
      kahan_step(pn, sh, dv);
      *shp = (uint16_t)(__float_as_uint(sh) >> 16);
    } else {
      pn = write_step<PT>(pv0, dv, -1.0f, hp.sr != 0, hp.sr ? noise_of(s_upd, i) : 0u);
    }
    if (hp.climb && MK != KAON_M_NONE) {
      float md;
      if constexpr (MK == KAON_M_4BIT || MK == KAON_M_INT8) {
        const float sc = scale_of(i);
        md = __fmul_rn((float)code_of(i, sc), sc);
      } else {
        md = f_s[i];
      }
      pn = write_step<PT>(pn, climb_e(md, hp.a_climb, hp.b_climb), 1.0f, E::IS_BF16, E::IS_BF16 ? noise_of(s_clb, i) : 0u);
    }
    if constexpr (E::IS_BF16) {
      uint16_t* dst = reinterpret_cast<uint16_t*>(d.p) + i;
      *dst = (uint16_t)(__float_as_uint(pn) >> 16);
      mirror_copy(&pv.peers, dst, 2);
    } else {
      float* dst = reinterpret_cast<float*>(d.p) + i;
      *dst = pn;
      mirror_copy(&pv.peers, dst, 4);
    }
  }
  __syncthreads();  // every read of the old scales is done before they are replaced
  if constexpr (MK == KAON_M_4BIT) {
    for (int b = tid; b < (n + 1) / 2; b += AT) {
      const int i0 = 2 * b, i1 = 2 * b + 1;
      unsigned lo = (unsigned)(code_of(i0, scale_of(i0)) + 8);
      unsigned hi = i1 < n ? (unsigned)(code_of(i1, scale_of(i1)) + 8) : 0u;
      reinterpret_cast<unsigned char*>(d.m)[b] = (unsigned char)(lo | (hi << 4));
    }
    const int nb = one_block ? 1 : (int)(((long long)n + (1 << bsh) - 1) >> bsh);
    for (int b = tid; b < nb; b += AT) d.m_scale[b] = scale_of(b << bsh);
  } else if constexpr (MK == KAON_M_INT8) {
    const float sc = scale_of(0);
    for (int i = tid; i < n; i += AT) reinterpret_cast<signed char*>(d.m)[i] = (signed char)code_of(i, sc);
    __syncthreads();  // every thread has read the old scale (old_m) before it is replaced
    if (tid == 0) d.m_scale[0] = sc;
  } else if constexpr (MK == KAON_M_BF16) {
    for (int i = tid; i < n; i += AT) reinterpret_cast<uint16_t*>(d.m)[i] = (uint16_t)(__float_as_uint(f_s[i]) >> 16);
  } else if constexpr (MK == KAON_M_F32) {
    for (int i = tid; i < n; i += AT) reinterpret_cast<float*>(d.m)[i] = f_s[i];
  }
}

// ----------------------------------------------------------------------------- kernels

#ifdef KAON_PHASE_TIMING
// development aid (off unless compiled in): busy cycles and item counts per work-item kind
__device__ unsigned long long g_phase_cycles[16];
#endif

template <typename PT, int MK, bool MUON>
__global__ void __launch_bounds__(AT, 1) adakaon_kernel(PlanView pv, AdaDev hp, int x_off_rows) {
  extern __shared__ __align__(128) unsigned char dyn[];
  __shared__ float mean_s[MAX_TASK_ROWS];
  __shared__ float rfac_s[MAX_TASK_ROWS];
  __shared__ unsigned rowmax_s[MAX_TASK_ROWS];
  __shared__ float scale_s[MAX_TASK_ROWS];
  __shared__ double red[AT / 32];
  __shared__ float part_s[AT / 32];
  __shared__ __align__(8) uint64_t bar[2];
  __shared__ int next_s[2];
  const int tid = threadIdx.x;
  // dynamic shared memory: [g buffer 0][g buffer 1][m buffer 0][m buffer 1][cfac / flat buffer];
  // x_off_rows = bytes of one m buffer (a multiple of 128) | 1 when there is room for two buffer sets.
  const int nbuf = (x_off_rows & 1) + 1;
  const size_t mcap = (size_t)(x_off_rows & ~127);
  const size_t gcap = (size_t)CAP * Elems<typename std::conditional<MUON, __nv_bfloat16, PT>::type>::BYTES;
  const size_t gcap_any = gcap > (size_t)CAP * Elems<PT>::BYTES ? gcap : (size_t)CAP * Elems<PT>::BYTES;
  Stage st;
  st.nbuf = nbuf;
  st.gbuf[0] = dyn; st.gbuf[1] = nbuf == 2 ? dyn + gcap_any : dyn;
  unsigned char* mbase = dyn + (size_t)nbuf * gcap_any;
  st.mbuf[0] = mbase; st.mbuf[1] = nbuf == 2 ? mbase + mcap : mbase;
  st.bar[0] = &bar[0]; st.bar[1] = &bar[1];
  st.parity[0] = st.parity[1] = 0u;
  st.g_s = st.gbuf[0]; st.m_s = st.mbuf[0];
  // STATS stages gradients only and overlays its column accumulators on the momentum buffers;
  // COUNT/APPLY/FLAT put cfac / the flat buffer after them.
  AdaSmem sm_stats{mean_s, rfac_s, rowmax_s, scale_s, reinterpret_cast<float*>(mbase), red, part_s};
  AdaSmem sm_rows{mean_s, rfac_s, rowmax_s, scale_s, reinterpret_cast<float*>(mbase + (size_t)nbuf * mcap), red, part_s};
  if (on_reserved_sm(pv.sm_reserve)) return;
  auto claim_next = [&](int slot) {
    if (tid == 0) {
      const unsigned s = *reinterpret_cast<volatile unsigned*>(pv.status);
      next_s[slot] = s ? 0x7fffffff : (int)atomicAdd(pv.task_counter, 1u);
    }
  };
  if (tid == 0) { mbar_init(&bar[0], 1); mbar_init(&bar[1], 1); }
  claim_next(0);
  __syncthreads();
  int slot = 0;
  int cur = next_s[0];
  while (cur < pv.n_tasks) {
    claim_next(slot ^ 1);
    const Task t = pv.tasks[cur];
#ifdef KAON_PHASE_TIMING
    const long long tk0 = clock64();
#endif
    switch (t.phase) {
      case PH_ADA_STATS: {
        using SST = typename std::conditional<MUON, __nv_bfloat16, PT>::type;
        const void* gsrc = (MUON && pv.grads[t.tensor] != nullptr) ? pv.signal[t.tensor] : pv.grads[t.tensor];
        if (stats_stream_ok(pv.tensors[t.tensor], gsrc, Elems<SST>::BYTES)) ada_stats_stream<SST>(pv, hp, t, sm_stats, dyn, tid);
        else ada_stats<SST>(pv, hp, t, st, sm_stats, tid);
        break;
      }
      case PH_ADA_FINAL: ada_final(pv, hp, t, sm_stats, tid); break;
      case PH_ADA_COUNT:
        if (stream_ok<MUON ? KAON_M_NONE : MK>(pv.tensors[t.tensor], hp, pv.grads[t.tensor], MUON && pv.grads[t.tensor] ? pv.signal[t.tensor] : nullptr))
          ada_stream<PT, MK, false, MUON>(pv, hp, t, sm_rows, tid);
        else ada_rows<PT, MK, false, MUON>(pv, hp, t, st, sm_rows, tid);
        break;
      case PH_ADA_APPLY:
        if (stream_ok<MUON ? KAON_M_NONE : MK>(pv.tensors[t.tensor], hp, pv.grads[t.tensor], MUON && pv.grads[t.tensor] ? pv.signal[t.tensor] : nullptr))
          ada_stream<PT, MK, true, MUON>(pv, hp, t, sm_rows, tid);
        else ada_rows<PT, MK, true, MUON>(pv, hp, t, st, sm_rows, tid);
        break;
      case PH_ADA_FLAT: ada_flat<PT, MK>(pv, hp, t, st, sm_rows, tid); break;
      default: break;
    }
    __syncthreads();
#ifdef KAON_PHASE_TIMING
    if (tid == 0) {
      atomicAdd(&g_phase_cycles[(t.phase - 10) & 7], (unsigned long long)(clock64() - tk0));
      atomicAdd(&g_phase_cycles[8 + ((t.phase - 10) & 7)], 1ull);
    }
#endif
    slot ^= 1;
    cur = next_s[slot];
  }
}

// Nekaon climb / removal / eval / train swap on its own (reference src/kaon/msam.py:201-235):
// p += clamp(nan_to_num(decode(m) * alpha), +-bound) over the plan's flat work items.
template <typename PT, int MK>
__global__ void __launch_bounds__(256) msam_axpy_kernel(PlanView pv, float alpha, float bound,
                                                        SrStream st) {
  using E = Elems<PT>;
  for (int ti = blockIdx.x; ti < pv.n_tasks; ti += gridDim.x) {
    const Task t = pv.tasks[ti];
    const DevTensor d = pv.tensors[t.tensor];
    const int nvec = (t.n + 7) >> 3;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const int cnt = min(8, t.n - v * 8);
      const long long e = t.e0 + (long long)v * 8;
      float md[8];
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float x = 0.0f;
        if (k < cnt) {
          const long long i = e + k;
          if constexpr (MK == KAON_M_4BIT) {
            const unsigned byte = reinterpret_cast<const unsigned char*>(d.m)[i >> 1];
            const int nib = (i & 1) ? (byte >> 4) & 0xF : byte & 0xF;
            x = __fmul_rn((float)(nib - 8), d.m_scale[blk_of(d, i)]);
          } else if constexpr (MK == KAON_M_INT8) {
            const int row = d.rows > 0 ? (int)(i / d.cols) : 0;
            x = __fmul_rn((float)reinterpret_cast<const signed char*>(d.m)[i], d.m_scale[row]);
          } else if constexpr (MK == KAON_M_BF16) {
            x = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(d.m)[i]);
          } else {
            x = reinterpret_cast<const float*>(d.m)[i];
          }
        }
        md[k] = climb_e(x, alpha, bound);
      }
      update8<PT>(reinterpret_cast<unsigned char*>(d.p) + e * E::BYTES, cnt, md, 1.0f, E::IS_BF16, st,
                  d.tensor_id, (uint64_t)(e >> 3), &pv.peers);
    }
  }
}

// ----------------------------------------------------------------------------- APPLY as its own kernel

// When every factored tensor of the plan takes the streaming form, the APPLY stage leaves the
// persistent kernel above and runs as a second launch built like the Lion kernel: 256-thread CTAs,
// several per SM, each bringing one flat item of at most APPLY_CAP elements (gradient, weights,
// momentum bytes) into shared memory with bulk copies while the other CTAs of the SM compute.  Stream
// order replaces the completion counters: every COUNT item has finished when this kernel starts.
// Items are flat runs (no row structure: what is per row or per column comes from the scratch in L2),
// so the int8 row scales of the previous step are read from the copy COUNT set aside.
constexpr int APPLY_CAP = 8192;
constexpr int APPLY_THREADS = 256;

// APPLY = false is the COUNT stage in the same form (kept count, int8 row maxima; no stores but those).
// MUON (AdaMuon): the chain runs on the orthogonalised momentum (bf16, `pv.signal`) with no momentum of
// its own, the cautious mask compares with the raw gradient, which is staged where the momentum bytes
// go otherwise.
template <typename PT, int MKP, bool APPLY, bool MUON>
__global__ void __launch_bounds__(APPLY_THREADS, 4) adakaon_apply_kernel(PlanView pv, AdaDev hp) {
  using E = Elems<PT>;
  using S = Elems<typename std::conditional<MUON, __nv_bfloat16, PT>::type>;
  constexpr int MK = MUON ? KAON_M_NONE : MKP;
  constexpr int GB = 8 * E::BYTES;
  constexpr int SB = 8 * S::BYTES;
  constexpr int MB = MUON ? GB : MK == KAON_M_4BIT ? 4 : MK == KAON_M_INT8 ? 8 : MK == KAON_M_BF16 ? 16 : MK == KAON_M_F32 ? 32 : 0;
  extern __shared__ __align__(128) unsigned char dyn[];
  __shared__ __align__(8) uint64_t bar;
  __shared__ int next_s[2];
  __shared__ unsigned red_s[APPLY_THREADS / 32];
  const bool need_p = APPLY || hp.has_wd;
  unsigned char* g_s = dyn;
  unsigned char* p_s = dyn + (size_t)APPLY_CAP * E::BYTES;
  unsigned char* m_s = dyn + (size_t)2 * APPLY_CAP * E::BYTES;
  const int tid = threadIdx.x;
  if (on_reserved_sm(pv.sm_reserve)) return;
  auto claim_next = [&](int slot) {
    if (tid == 0) {
      const unsigned st = *reinterpret_cast<volatile unsigned*>(pv.status);
      next_s[slot] = st ? 0x7fffffff : (int)atomicAdd(pv.task_counter, 1u);
    }
  };
  if (tid == 0) mbar_init(&bar, 1);
  claim_next(0);
  __syncthreads();
  unsigned parity = 0u;
  int slot = 0;
  int cur = next_s[0];
  SrStream s_upd{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_UPDATE};
  SrStream s_rem{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_REMOVE};
  SrStream s_clb{Philox{hp.k0, hp.k1}, hp.step, KAON_TAG_CLIMB};
  const bool sr = hp.sr != 0;
  const bool gc = hp.gc != 0 && !MUON;
  // AdaMuon with gradient centralization: the statistics run on the orthogonalised matrix, which is not
  // centralised; the cautious mask compares with the CENTRALISED raw gradient (row means in the scratch)
  const bool gcr = hp.gc != 0 && MUON;
  while (cur < pv.n_tasks) {
    claim_next(slot ^ 1);
    const Task t = pv.tasks[cur];
    const DevTensor d = pv.tensors[t.tensor];
    const unsigned char* g = reinterpret_cast<const unsigned char*>(pv.grads[t.tensor]);
    bool ok = g != nullptr;
    const int n = t.n;
    if (ok) {
      const unsigned char* gsrc = MUON ? reinterpret_cast<const unsigned char*>(pv.signal[t.tensor]) + t.e0 * S::BYTES
                                       : g + t.e0 * E::BYTES;
      const unsigned char* msrc = MUON ? g + t.e0 * E::BYTES : m_ptr<MK>(d, t.e0);
      const unsigned mbytes = MUON ? (unsigned)n * E::BYTES : m_bytes<MK>(n);
      const unsigned char* psrc = reinterpret_cast<const unsigned char*>(d.p) + t.e0 * E::BYTES;
      const unsigned ghead = stage_tail(g_s, gsrc, (unsigned)n * S::BYTES, tid);
      const unsigned phead = need_p ? stage_tail(p_s, psrc, (unsigned)n * E::BYTES, tid) : 0u;
      unsigned mhead = 0u;
      if constexpr (MB > 0) mhead = stage_tail(m_s, msrc, mbytes, tid);
      if (ghead + phead + mhead) {
        if (tid == 0) {
          fence_async_smem();
          mbar_expect_tx(&bar, ghead + phead + mhead);
          if (ghead) bulk_g2s(g_s, gsrc, ghead, &bar);
          if (phead) bulk_g2s(p_s, psrc, phead, &bar);
          if constexpr (MB > 0) { if (mhead) bulk_g2s(m_s, msrc, mhead, &bar); }
        }
        ok = mbar_wait(&bar, parity, pv.status, 15001u);
        parity ^= 1u;
      }
    }
    ok = __syncthreads_and(ok) != 0;
    unsigned kept_local = 0;
    if (ok) {
      const int C = d.cols;
      const long long row0 = t.e0 / C;
      const int col0 = (int)(t.e0 - row0 * C);
      const float* scal = pv.aux + aux_scal(d);
      Chain ch;
      ch.div = __ldcg(scal + 1);
      ch.use_div = ch.div != 1.0f;
      ch.rcp_div = __fdiv_rn(1.0f, ch.div);
      float denom = 1.0f, rcp_denom = 1.0f;
      if (APPLY && hp.cautious) {
        const unsigned kept_t = __ldcg(pv.kept + t.tensor);
        denom = fmaxf(__fdiv_rn((float)kept_t, (float)d.numel), 1e-8f);
        rcp_denom = __fdiv_rn(1.0f, denom);
      }
      const float* cfac = pv.aux + aux_cfac(d);
      const float* mean = pv.aux + aux_mean(d);
      unsigned* rowmax = reinterpret_cast<unsigned*>(pv.aux + aux_rowmax(d));
      const float* oldsc = pv.aux + aux_oldsc(d);
      const float* rfac = pv.aux + aux_rfac(d);
      unsigned char* pbase = reinterpret_cast<unsigned char*>(d.p) + t.e0 * E::BYTES;
      const int nvec = n >> 3;
      const int nvec_pad = (nvec + 31) & ~31;
      // ---- fast path: bf16 weights, int8 / 4-bit momentum (or AdaMuon's chain, which carries none and takes
      //      the orthogonalised matrix as its signal), stochastic-rounding write (or the COUNT stage), no Kahan buffer.  Same arithmetic as the general loop below, element for element, on packed
      //      pairs (f32x2), with the cautious mask and the quantised codes gathered by byte permutes and
      //      one exactness check per vector; the rare vectors that fail a check are redone the plain way. ----
      constexpr bool FASTABLE = E::IS_BF16 && (MUON || MK == KAON_M_INT8 || MK == KAON_M_4BIT);
      bool fast = false;
      if constexpr (FASTABLE) fast = !hp.kahan && (!APPLY || sr);
      if constexpr (FASTABLE) if (fast) {
        const f32x2 DIVN = pack2(-ch.div, -ch.div), RCPD = pack2(ch.rcp_div, ch.rcp_div);
        const f32x2 SCALE = pack2(hp.upd_scale, hp.upd_scale);
        const f32x2 W1 = pack2(hp.w1, hp.w1), W1M1 = pack2(hp.w1m1, hp.w1m1);
        const f32x2 LRWD = pack2(hp.lrwd, hp.lrwd);
        const f32x2 DENN = pack2(-denom, -denom), RCPN = pack2(rcp_denom, rcp_denom);
        const uint32_t* gsm = reinterpret_cast<const uint32_t*>(g_s);
        const uint32_t* psm = reinterpret_cast<const uint32_t*>(p_s);
        const long long blk0 = t.e0 >> 7;
        const uint64_t q0 = (uint64_t)(t.e0 >> 3);
        auto clamp2 = [](f32x2 e, float b) { return pack2(fminf(fmaxf(e.x, -b), b), fminf(fmaxf(e.y, -b), b)); };
        // one stochastic-rounding write of eight weights held as four pairs: P <- trunc16(bits(P + D) + noise)
        auto sr_write = [&](f32x2 P[4], const f32x2 D[4], const SrStream& stream, uint64_t q) {
          uint32_t nz[4];
          stream.draw8(d.tensor_id, q, nz);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const f32x2 r = add2(P[j], D[j]);
            P[j] = pack2(__uint_as_float((__float_as_uint(r.x) + (nz[j] & 0xffffu)) & 0xFFFF0000u),
                         __uint_as_float((__float_as_uint(r.y) + (nz[j] >> 16)) & 0xFFFF0000u));
          }
        };
        auto trip = [&](const int v, auto guard_tag, auto small_tag) {
          constexpr bool GUARD = decltype(guard_tag)::value;
          constexpr bool SMALL_W1 = decltype(small_tag)::value;
          const bool act = !GUARD || v < nvec;
          const int vv = act ? v : 0;
          const unsigned i = (unsigned)col0 + (unsigned)vv * 8u;
          const int r = row_of(i, d);
          const int row = (int)row0 + r;
          const int col = (int)i - r * C;
          const float rf = __ldcg(rfac + row);
          const float4 c0v = __ldcg(reinterpret_cast<const float4*>(cfac + col));
          const float4 c1v = __ldcg(reinterpret_cast<const float4*>(cfac + col + 4));
          const uint4 gq = *reinterpret_cast<const uint4*>(gsm + (size_t)vv * 4);
          uint32_t gw[4] = {gq.x, gq.y, gq.z, gq.w};
          if (gc) {
            const float mu = __ldcg(mean + row);
            const uint32_t mu2 = pack_bf16_rn(mu, mu);
#pragma unroll
            for (int j = 0; j < 4; ++j) gw[j] = sub_bf16x2(gw[j], mu2);
          }
          uint32_t mu2r = 0u;   // AdaMuon: the centralization mean of the raw gradient's row, two bf16 copies
          if (MUON && gcr) {
            const float mur = __ldcg(mean + row);
            mu2r = pack_bf16_rn(mur, mur);
          }
          f32x2 P[4];
          if (need_p) {
            const uint4 pq = *reinterpret_cast<const uint4*>(psm + (size_t)vv * 4);
            P[0] = pack2(bf16lo(pq.x), bf16hi(pq.x)); P[1] = pack2(bf16lo(pq.y), bf16hi(pq.y));
            P[2] = pack2(bf16lo(pq.z), bf16hi(pq.z)); P[3] = pack2(bf16lo(pq.w), bf16hi(pq.w));
          } else {
            P[0] = P[1] = P[2] = P[3] = pack2(0.0f, 0.0f);
          }
          // ---- old momentum ----
          f32x2 MO[4];
          float sc_old;
          if constexpr (MK == KAON_M_4BIT) {
            sc_old = d.m_scale[blk0 + (vv >> 4)];
            const uint32_t w = reinterpret_cast<const uint32_t*>(m_s)[vv];
            const uint32_t wl = w & 0x0F0F0F0Fu, wh = (w >> 4) & 0x0F0F0F0Fu;
            const f32x2 BIAS = pack2(-8388616.0f, -8388616.0f), SC = pack2(sc_old, sc_old);
#pragma unroll
            for (int j = 0; j < 4; ++j)
              MO[j] = mul2(add2(pack2(__uint_as_float(prmt(wl, 0x4B000000u, 0x7540u | (uint32_t)j)),
                                      __uint_as_float(prmt(wh, 0x4B000000u, 0x7540u | (uint32_t)j))), BIAS), SC);
          } else if constexpr (MK == KAON_M_NONE) {
            sc_old = 1.0f;
            MO[0] = MO[1] = MO[2] = MO[3] = pack2(0.0f, 0.0f);
          } else {
            sc_old = APPLY ? __ldcg(oldsc + row) : d.m_scale[row];
            const uint2 w = reinterpret_cast<const uint2*>(m_s)[vv];
            const uint32_t x0 = w.x ^ 0x80808080u, x1 = w.y ^ 0x80808080u;  // code + 128 in every byte
            const f32x2 BIAS = pack2(-8388736.0f, -8388736.0f), SC = pack2(sc_old, sc_old);  // -(2^23 + 128)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const uint32_t x = j < 2 ? x0 : x1;
              const uint32_t b = (uint32_t)(2 * (j & 1));
              MO[j] = mul2(add2(pack2(__uint_as_float(prmt(x, 0x4B000000u, 0x7540u | b)),
                                      __uint_as_float(prmt(x, 0x4B000000u, 0x7540u | (b + 1u)))), BIAS), SC);
            }
          }
          const uint64_t q = q0 + (uint64_t)vv;
          // a momentum that decodes to NaN or infinity (a corrupt scale) keeps the reference's nan_to_num
          const bool wild = !(fabsf(sc_old) <= 3.0e38f);
          if (hp.remove && need_p) {
            const f32x2 AR = pack2(hp.a_remove, hp.a_remove);
            f32x2 Dr[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              f32x2 e = mul2(MO[j], AR);
              if (wild) { if (e.x != e.x) e.x = 0.0f; if (e.y != e.y) e.y = 0.0f; }
              Dr[j] = clamp2(e, hp.b_remove);
            }
            sr_write(P, Dr, s_rem, q);
          }
          // ---- update chain: u = ((g r) c) / divisor * scale; m' = lerp(m, u); delta = m' + (lr wd) p ----
          // (a divisor of 1 and a zero weight decay go through the same operations: x/1 and fma(p, 0, m')
          //  give x and m' back; a delta of -0 that becomes +0 is masked out or subtracted either way)
          const f32x2 RF = pack2(rf, rf);
          const f32x2 CF[4] = {pack2(c0v.x, c0v.y), pack2(c0v.z, c0v.w), pack2(c1v.x, c1v.y), pack2(c1v.z, c1v.w)};
          f32x2 MN[4], DV[4];
          float a[8];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const f32x2 G = pack2(bf16lo(gw[j]), bf16hi(gw[j]));
            f32x2 U = mul2(mul2(G, RF), CF[j]);
            const f32x2 qq = mul2(U, RCPD);
            U = mul2(fma2(fma2(qq, DIVN, U), RCPD, qq), SCALE);
            if constexpr (MK == KAON_M_NONE) {
              MN[j] = U;  // no momentum of its own: delta = u
            } else {
              const f32x2 diff = sub2(U, MO[j]);
              MN[j] = SMALL_W1 ? fma2(W1, diff, MO[j]) : fma2(W1M1, diff, U);
            }
            DV[j] = fma2(P[j], LRWD, MN[j]);
            if constexpr (MUON) {  // the mask compares with the raw gradient, staged where the momentum goes otherwise
              uint32_t rw = reinterpret_cast<const uint32_t*>(m_s)[(size_t)vv * 4 + j];
              if (gcr) rw = sub_bf16x2(rw, mu2r);
              unpack2(mul2(DV[j], pack2(bf16lo(rw), bf16hi(rw))), a[2 * j], a[2 * j + 1]);
            } else {
              unpack2(mul2(DV[j], G), a[2 * j], a[2 * j + 1]);
            }
          }
          // ---- cautious mask: kept <=> delta * g > 0 (sign bits; a zero or underflowing product is rare
          //      and decided by the comparison itself) ----
          float amin = min3f(fabsf(a[0]), fabsf(a[1]), fabsf(a[2]));
          amin = min3f(amin, fabsf(a[3]), fabsf(a[4]));
          amin = min3f(amin, fabsf(a[5]), fabsf(a[6]));
          amin = fminf(amin, fabsf(a[7]));
          float amax = max3f(fabsf(MN[0].x), fabsf(MN[0].y), fabsf(MN[1].x));
          amax = max3f(amax, fabsf(MN[1].y), fabsf(MN[2].x));
          amax = max3f(amax, fabsf(MN[2].y), fabsf(MN[3].x));
          amax = fmaxf(amax, fabsf(MN[3].y));
          if constexpr (!APPLY) {
            unsigned kept = 0;
            if (amin > 0.0f) {
              const uint32_t am_lo = prmt(prmt(__float_as_uint(a[0]), __float_as_uint(a[1]), 0x00FBu),
                                          prmt(__float_as_uint(a[2]), __float_as_uint(a[3]), 0x00FBu), 0x5410u);
              const uint32_t am_hi = prmt(prmt(__float_as_uint(a[4]), __float_as_uint(a[5]), 0x00FBu),
                                          prmt(__float_as_uint(a[6]), __float_as_uint(a[7]), 0x00FBu), 0x5410u);
              kept = 8u - (unsigned)__popc(am_lo & 0x01010101u) - (unsigned)__popc(am_hi & 0x01010101u);
            } else {
#pragma unroll
              for (int k = 0; k < 8; ++k) kept += a[k] > 0.0f ? 1u : 0u;
            }
            if (act) kept_local += kept;
            if constexpr (MK == KAON_M_INT8) {
              unsigned bits = act ? __float_as_uint(amax) : 0u;
              const int row_l0 = __shfl_sync(0xffffffffu, row, 0);
              if (__all_sync(0xffffffffu, !act || row == row_l0)) {
                bits = __reduce_max_sync(0xffffffffu, bits);
                if ((tid & 31) == 0 && bits) atomicMax(rowmax + row_l0, bits);
              } else if (act) {
                atomicMax(rowmax + row, bits);
              }
            }
            return;
          } else {
            // ---- the update: delta, or under the cautious mask (delta if kept else 0) / denom ----
            f32x2 F[4];
            if (hp.cautious) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                const f32x2 qq = mul2(DV[j], RCPN);
                const f32x2 f = fma2(fma2(qq, DENN, DV[j]), RCPN, qq);
                // masked out where the product delta * g is negative (its sign bit spread over the word)
                F[j] = pack2(__uint_as_float(__float_as_uint(f.x) & ~(uint32_t)((int)__float_as_uint(a[2 * j]) >> 31)),
                             __uint_as_float(__float_as_uint(f.y) & ~(uint32_t)((int)__float_as_uint(a[2 * j + 1]) >> 31)));
              }
              if (!(amin > 0.0f)) {  // some product is zero: those elements are masked out as well
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  if (!(a[2 * j] > 0.0f)) F[j].x = 0.0f;
                  if (!(a[2 * j + 1] > 0.0f)) F[j].y = 0.0f;
                }
              }
            } else {
#pragma unroll
              for (int j = 0; j < 4; ++j) F[j] = DV[j];
            }
            // ---- quantise and store the new momentum; MD = the momentum as stored, decoded ----
            f32x2 MD[4];
            float sc = 1.0f;
            if constexpr (MK == KAON_M_NONE) {
              MD[0] = MD[1] = MD[2] = MD[3] = pack2(0.0f, 0.0f);
            } else {
            if constexpr (MK == KAON_M_4BIT) {
              const float am = fmaxf(half_warp_max(act ? amax : 0.0f, tid), 1e-12f);
              __syncwarp();  // every lane of the block has read the old scale before it is replaced
              sc = div7_exact(am);
            } else {
              sc = div127_exact(fmaxf(__uint_as_float(__ldcg(rowmax + row)), 1e-12f));
            }
            float inv;
            asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(sc));
            const f32x2 INV = pack2(inv, inv), NSC = pack2(-sc, -sc);
            // r = rint(n*inv) (+8) + magic in one rounding; T = -rint(n*inv); e = n*inv - rint(n*inv) exactly
            constexpr float MAGIC = MK == KAON_M_4BIT ? 12582920.0f : 12582912.0f;
            const f32x2 MG = pack2(MAGIC, MAGIC);
            f32x2 T[4], R[4];
            float e8[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              R[j] = fma2(MN[j], INV, MG);
              T[j] = sub2(MG, R[j]);
              unpack2(fma2(MN[j], INV, T[j]), e8[2 * j], e8[2 * j + 1]);
              MD[j] = mul2(T[j], NSC);
            }
            float worst = max3f(fabsf(e8[0]), fabsf(e8[1]), fabsf(e8[2]));
            worst = max3f(worst, fabsf(e8[3]), fabsf(e8[4]));
            worst = max3f(worst, fabsf(e8[5]), fabsf(e8[6]));
            worst = fmaxf(worst, fabsf(e8[7]));
            uint32_t w0, w1 = 0u;
            if constexpr (MK == KAON_M_4BIT) {
              const f32x2 K256 = pack2(256.0f, 256.0f);
              const f32x2 X = fma2(T[1], K256, T[0]), Y = fma2(T[3], K256, T[2]);
              const float lo4 = __fsub_rn(8423560.0f, __fmaf_rn(X.y, 16.0f, X.x));
              const float hi4 = __fsub_rn(8423560.0f, __fmaf_rn(Y.y, 16.0f, Y.x));
              w0 = prmt(__float_as_uint(lo4), __float_as_uint(hi4), 0x5410u);
            } else {  // the low byte of every r is the code in two's complement
              w0 = prmt(prmt(__float_as_uint(R[0].x), __float_as_uint(R[0].y), 0x0040u),
                        prmt(__float_as_uint(R[1].x), __float_as_uint(R[1].y), 0x0040u), 0x5410u);
              w1 = prmt(prmt(__float_as_uint(R[2].x), __float_as_uint(R[2].y), 0x0040u),
                        prmt(__float_as_uint(R[3].x), __float_as_uint(R[3].y), 0x0040u), 0x5410u);
            }
            // Rare: a product n*inv too close to a rounding boundary to trust the reciprocal (it is good to
            // 2^-22: |n*inv - n/sc| < 127 * 2^-22 = 3e-5, 7 * 2^-22 for 4 bits), or a scale that is not
            // finite: the codes of this vector again, by the true division.
            if (worst > 0.5f - (MK == KAON_M_4BIT ? 1e-5f : 1e-4f) || !(sc <= 3.0e38f)) {
              const float inv2 = __fdividef(1.0f, sc);
              float n8[8], md8[8];
#pragma unroll
              for (int j = 0; j < 4; ++j) unpack2(MN[j], n8[2 * j], n8[2 * j + 1]);
              w0 = 0u; w1 = 0u;
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                if constexpr (MK == KAON_M_4BIT) {
                  const int qi = min(max((int)quant_round(n8[k], sc, inv2, 1e-4f), -7), 7);
                  md8[k] = __fmul_rn((float)qi, sc);
                  w0 |= (uint32_t)(qi + 8) << (4 * k);
                } else {
                  const int qi = min(max((int)quant_round(n8[k], sc, inv2, 1e-3f), -127), 127);
                  md8[k] = __fmul_rn((float)qi, sc);
                  const uint32_t byte = (uint32_t)(qi & 0xFF);
                  if (k < 4) w0 |= byte << (8 * k); else w1 |= byte << (8 * (k - 4));
                }
              }
#pragma unroll
              for (int j = 0; j < 4; ++j) MD[j] = pack2(md8[2 * j], md8[2 * j + 1]);
            }
            if (act) {
              if constexpr (MK == KAON_M_4BIT) {
                stg_u32(reinterpret_cast<unsigned char*>(d.m) + (t.e0 >> 1) + (size_t)v * 4, w0);
                if ((v & 15) == 0) stg_f32(d.m_scale + blk0 + (v >> 4), sc);
              } else {
                *reinterpret_cast<uint2*>(reinterpret_cast<unsigned char*>(d.m) + t.e0 + (size_t)v * 8) = make_uint2(w0, w1);
                if (col == 0) d.m_scale[row] = sc;
              }
            }
            }  // MK != NONE
            // ---- weights: p <- SR(p - update), then the Nekaon climb from the momentum as stored ----
#pragma unroll
            for (int j = 0; j < 4; ++j) F[j] = pack2(-F[j].x, -F[j].y);
            sr_write(P, F, s_upd, q);
            if (hp.climb && MK != KAON_M_NONE) {
              const f32x2 AC = pack2(hp.a_climb, hp.a_climb);
              const bool wild2 = !(sc <= 3.0e38f);
              f32x2 Dc[4];
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                f32x2 e = mul2(MD[j], AC);
                if (wild2) { if (e.x != e.x) e.x = 0.0f; if (e.y != e.y) e.y = 0.0f; }
                Dc[j] = clamp2(e, hp.b_climb);
              }
              sr_write(P, Dc, s_clb, q);
            }
            if (act) {
              const uint4 out = make_uint4(prmt(__float_as_uint(P[0].x), __float_as_uint(P[0].y), 0x7632u),
                                           prmt(__float_as_uint(P[1].x), __float_as_uint(P[1].y), 0x7632u),
                                           prmt(__float_as_uint(P[2].x), __float_as_uint(P[2].y), 0x7632u),
                                           prmt(__float_as_uint(P[3].x), __float_as_uint(P[3].y), 0x7632u));
              *reinterpret_cast<uint4*>(pbase + (size_t)v * 16) = out;
              mirror16(&pv.peers, pbase + (size_t)v * 16, out);
            }
          }
        };
        const int nfull = nvec & ~31;
        if (hp.small_w1) {
          for (int v = tid; v < nfull; v += APPLY_THREADS) trip(v, std::false_type{}, std::true_type{});
          if (nfull != nvec && tid < 32) trip(nfull + tid, std::true_type{}, std::true_type{});
        } else {
          for (int v = tid; v < nfull; v += APPLY_THREADS) trip(v, std::false_type{}, std::false_type{});
          if (nfull != nvec && tid < 32) trip(nfull + tid, std::true_type{}, std::false_type{});
        }
      }
      if (!fast)
      for (int v = tid; v < nvec_pad; v += APPLY_THREADS) {
        const bool act = v < nvec;
        const int vv = act ? v : 0;
        const unsigned i = (unsigned)col0 + (unsigned)vv * 8u;  // < APPLY_CAP + cols: row_of is exact
        const int r = row_of(i, d);
        const int row = (int)row0 + r;
        const int col = (int)i - r * C;
        float gv[8], mo[8], mn[8], pc[8], dl[8];
        const float mu = (gc || gcr) ? __ldcg(mean + row) : 0.0f;
        const float rf = __ldcg(rfac + row);
        const float4 c0v = __ldcg(reinterpret_cast<const float4*>(cfac + col));
        const float4 c1v = __ldcg(reinterpret_cast<const float4*>(cfac + col + 4));
        const float cf[8] = {c0v.x, c0v.y, c0v.z, c0v.w, c1v.x, c1v.y, c1v.z, c1v.w};
        S::load8(g_s + (size_t)vv * SB, gv);
        float raw[8];
        if (MUON) E::load8(m_s + (size_t)vv * GB, raw);
        if (MUON && gcr) {
#pragma unroll
          for (int k = 0; k < 8; ++k) raw[k] = centered<PT>(raw[k], mu, true);
        }
        if (need_p) E::load8(p_s + (size_t)vv * GB, pc);
        else {
#pragma unroll
          for (int k = 0; k < 8; ++k) pc[k] = 0.0f;
        }
        if constexpr (MK == KAON_M_4BIT) {
          decode8<MK>(m_s, vv, 8, d.m_scale[(t.e0 >> 7) + (vv >> 4)], mo);
        } else if constexpr (MK == KAON_M_INT8) {
          decode8<MK>(m_s, vv, 8, APPLY ? __ldcg(oldsc + row) : d.m_scale[row], mo);
        } else if constexpr (MK == KAON_M_NONE) {
#pragma unroll
          for (int k = 0; k < 8; ++k) mo[k] = 0.0f;
        } else {
          decode8<MK>(m_s, vv, 8, 1.0f, mo);
        }
        if (hp.remove && need_p) {
          uint32_t nz[4] = {0u, 0u, 0u, 0u};
          if (E::IS_BF16) s_rem.draw8(d.tensor_id, (uint64_t)((t.e0 >> 3) + vv), nz);
#pragma unroll
          for (int k = 0; k < 8; ++k)
            pc[k] = write_step<PT>(pc[k], climb_e(mo[k], hp.a_remove, hp.b_remove), 1.0f, E::IS_BF16, noise_lane(nz, k));
        }
        if (gc) {
#pragma unroll
          for (int k = 0; k < 8; k += 2) {
            const float x0 = __fsub_rn(gv[k], mu), x1 = __fsub_rn(gv[k + 1], mu);
            if (E::IS_BF16) {
              const uint32_t pk = pack_bf16_rn(x0, x1);
              gv[k] = bf16lo(pk); gv[k + 1] = bf16hi(pk);
            } else {
              gv[k] = x0; gv[k + 1] = x1;
            }
          }
        }
        unsigned kept = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float u = update_of(gv[k], rf, cf[k], ch, hp.upd_scale);
          mn[k] = ema_of<MK>(mo[k], u, hp);
          const float dv = hp.has_wd ? __fmaf_rn(pc[k], hp.lrwd, mn[k]) : mn[k];
          dl[k] = dv;
          if (__fmul_rn(dv, MUON ? raw[k] : gv[k]) > 0.0f) kept |= 1u << k;
        }
        if constexpr (!APPLY) {
          if (act) kept_local += __popc(kept);
          if constexpr (MK == KAON_M_INT8) {
            float a = 0.0f;
#pragma unroll
            for (int k = 0; k < 8; ++k) a = fmaxf(a, fabsf(mn[k]));
            unsigned bits = act ? __float_as_uint(a) : 0u;
            const int row_l0 = __shfl_sync(0xffffffffu, row, 0);
            if (__all_sync(0xffffffffu, !act || row == row_l0)) {
              bits = __reduce_max_sync(0xffffffffu, bits);
              if ((tid & 31) == 0 && bits) atomicMax(rowmax + row_l0, bits);
            } else if (act) {
              atomicMax(rowmax + row, bits);
            }
          }
          continue;
        }
        float md[8];  // the momentum as stored (decoded), for the Nekaon climb
        if constexpr (MK == KAON_M_4BIT) {
          float a = 0.0f;
#pragma unroll
          for (int k = 0; k < 8; ++k) a = fmaxf(a, act ? fabsf(mn[k]) : 0.0f);
          a = fmaxf(group_max(a, 16), 1e-12f);
          __syncwarp();  // every lane of the block has read the old scale before it is replaced
          const float sc = __fdiv_rn(a, 7.0f);
          const float inv = __fdividef(1.0f, sc);
          uint32_t word = 0;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const float q = quant_round(mn[k], sc, inv, 1e-4f);
            const int qi = min(max((int)q, -7), 7);
            md[k] = __fmul_rn((float)qi, sc);
            word |= (uint32_t)(qi + 8) << (4 * k);
          }
          if (act) {
            *reinterpret_cast<uint32_t*>((unsigned char*)d.m + (t.e0 >> 1) + (size_t)v * 4) = word;
            if ((v & 15) == 0) d.m_scale[(t.e0 >> 7) + (v >> 4)] = sc;
          }
        } else if constexpr (MK == KAON_M_INT8) {
          const float sc = __fdiv_rn(fmaxf(__uint_as_float(__ldcg(rowmax + row)), 1e-12f), 127.0f);
          const float inv = __fdividef(1.0f, sc);
          uint32_t w0 = 0, w1 = 0;
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const int qi = min(max((int)quant_round(mn[k], sc, inv, 1e-3f), -127), 127);
            md[k] = __fmul_rn((float)qi, sc);
            const uint32_t byte = (uint32_t)(qi & 0xFF);
            if (k < 4) w0 |= byte << (8 * k); else w1 |= byte << (8 * (k - 4));
          }
          if (act) {
            *reinterpret_cast<uint2*>((unsigned char*)d.m + t.e0 + (size_t)v * 8) = make_uint2(w0, w1);
            if (col == 0) d.m_scale[row] = sc;
          }
        } else if constexpr (MK == KAON_M_BF16 || MK == KAON_M_F32) {
#pragma unroll
          for (int k = 0; k < 8; ++k) md[k] = mn[k];
          if (act) {
            if constexpr (MK == KAON_M_BF16) store8<__nv_bfloat16>((unsigned char*)d.m + t.e0 * 2 + (size_t)v * 16, 8, mn, nullptr);
            else store8<float>((unsigned char*)d.m + t.e0 * 4 + (size_t)v * 32, 8, mn, nullptr);
          }
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) md[k] = 0.0f;
        }
        if (act) {
          if (E::IS_BF16 && hp.kahan) {
            unsigned char* she = reinterpret_cast<unsigned char*>(d.shift) + (size_t)t.e0 * 2 + (size_t)v * 16;
            float sh[8];
            load8_guard<__nv_bfloat16>(she, 8, sh);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              float f = dl[k];
              if (hp.cautious) f = ((kept >> k) & 1u) ? div_shared(f, denom, rcp_denom) : 0.0f;
              kahan_step(pc[k], sh[k], f);
            }
            store8<__nv_bfloat16>(she, 8, sh, nullptr);
          } else {
            uint32_t nz[4] = {0u, 0u, 0u, 0u};
            if (sr) s_upd.draw8(d.tensor_id, (uint64_t)((t.e0 >> 3) + v), nz);
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              float f = dl[k];
              if (hp.cautious) f = ((kept >> k) & 1u) ? div_shared(f, denom, rcp_denom) : 0.0f;
              pc[k] = write_step<PT>(pc[k], f, -1.0f, sr, noise_lane(nz, k));
            }
          }
          if (hp.climb && MK != KAON_M_NONE) {
            uint32_t nc[4] = {0u, 0u, 0u, 0u};
            if (E::IS_BF16) s_clb.draw8(d.tensor_id, (uint64_t)((t.e0 >> 3) + v), nc);
#pragma unroll
            for (int k = 0; k < 8; ++k)
              pc[k] = write_step<PT>(pc[k], climb_e(md[k], hp.a_climb, hp.b_climb), 1.0f, E::IS_BF16, noise_lane(nc, k));
          }
          store8<PT>(pbase + (size_t)v * 8 * E::BYTES, 8, pc, &pv.peers);
        }
      }
    }
    if constexpr (!APPLY) {  // the item's kept count
      for (int o = 16; o > 0; o >>= 1) kept_local += __shfl_xor_sync(0xffffffffu, kept_local, o);
      if ((tid & 31) == 0) red_s[tid >> 5] = kept_local;
    }
    __syncthreads();
    if constexpr (!APPLY) {
      if (tid == 0 && ok) {
        unsigned tot = 0;
        for (int w = 0; w < APPLY_THREADS / 32; ++w) tot += red_s[w];
        if (tot) atomicAdd(pv.kept + t.tensor, tot);
      }
    }
    slot ^= 1;
    cur = next_s[slot];
  }
}

typedef void (*ApplyKernel)(PlanView, AdaDev);

template <typename PT, bool APPLY>
static ApplyKernel pick_apply_pt(int mk) {
  switch (mk) {
    case KAON_M_F32: return adakaon_apply_kernel<PT, KAON_M_F32, APPLY, false>;
    case KAON_M_BF16: return adakaon_apply_kernel<PT, KAON_M_BF16, APPLY, false>;
    case KAON_M_INT8: return adakaon_apply_kernel<PT, KAON_M_INT8, APPLY, false>;
    case KAON_M_4BIT: return adakaon_apply_kernel<PT, KAON_M_4BIT, APPLY, false>;
    case KAON_M_NONE: return adakaon_apply_kernel<PT, KAON_M_NONE, APPLY, false>;
    default: return nullptr;
  }
}

static ApplyKernel pick_apply(int pdt, int mk, bool apply, bool muon) {
  if (muon) {
    if (pdt == KAON_DT_BF16) return apply ? adakaon_apply_kernel<__nv_bfloat16, KAON_M_NONE, true, true>
                                          : adakaon_apply_kernel<__nv_bfloat16, KAON_M_NONE, false, true>;
    return apply ? adakaon_apply_kernel<float, KAON_M_NONE, true, true> : adakaon_apply_kernel<float, KAON_M_NONE, false, true>;
  }
  if (apply) return pdt == KAON_DT_BF16 ? pick_apply_pt<__nv_bfloat16, true>(mk) : pick_apply_pt<float, true>(mk);
  return pdt == KAON_DT_BF16 ? pick_apply_pt<__nv_bfloat16, false>(mk) : pick_apply_pt<float, false>(mk);
}

typedef void (*AxpyKernel)(PlanView, float, float, SrStream);

template <typename PT, bool MUON>
static AdaKernel pick_ada_pt(int mk) {
  switch (mk) {
    case KAON_M_F32: return adakaon_kernel<PT, KAON_M_F32, MUON>;
    case KAON_M_BF16: return adakaon_kernel<PT, KAON_M_BF16, MUON>;
    case KAON_M_INT8: return adakaon_kernel<PT, KAON_M_INT8, MUON>;
    case KAON_M_4BIT: return adakaon_kernel<PT, KAON_M_4BIT, MUON>;
    case KAON_M_NONE: return adakaon_kernel<PT, KAON_M_NONE, MUON>;
    default: return nullptr;
  }
}
AdaKernel pick_ada(int pdt, int mk, bool muon) {
  if (muon) return pdt == KAON_DT_BF16 ? pick_ada_pt<__nv_bfloat16, true>(mk) : pick_ada_pt<float, true>(mk);
  return pdt == KAON_DT_BF16 ? pick_ada_pt<__nv_bfloat16, false>(mk) : pick_ada_pt<float, false>(mk);
}

template <typename PT>
static AxpyKernel pick_axpy_pt(int mk) {
  switch (mk) {
    case KAON_M_F32: return msam_axpy_kernel<PT, KAON_M_F32>;
    case KAON_M_BF16: return msam_axpy_kernel<PT, KAON_M_BF16>;
    case KAON_M_INT8: return msam_axpy_kernel<PT, KAON_M_INT8>;
    case KAON_M_4BIT: return msam_axpy_kernel<PT, KAON_M_4BIT>;
    default: return nullptr;
  }
}

// bytes reserved after the gradient stage for the momentum bytes (AdaMuon: the raw gradient) of a chunk
size_t x_offset_rows(const kaon_plan* pl) {
  size_t b = momentum_bytes_per_cap(pl->momentum_kind);
  if (pl->optimizer == KAON_OPT_ADAMUON) b = std::max<size_t>(b, (size_t)CAP * (pl->param_dtype == KAON_DT_BF16 ? 2 : 4));
  return (b + 127) / 128 * 128;
}

int configure_launch_adakaon(kaon_plan* pl, const cudaDeviceProp& prop, int max_cols) {
  const size_t esz = pl->param_dtype == KAON_DT_BF16 ? 2 : 4;
  const size_t xr = x_offset_rows(pl);
  // the gradient stage holds the parameter dtype, or bf16 for AdaMuon's orthogonalised signal (FLAT still
  // stages the gradient itself there): size it for the larger
  const size_t gcap = (size_t)CAP * esz;
  auto total = [&](int nbuf) {
    const size_t region = std::max<size_t>((size_t)nbuf * xr + (size_t)max_cols * 4, (size_t)max_cols * 8);
    return (size_t)nbuf * gcap + region + 128;
  };
  pl->threads = AT;
  AdaKernel k = pick_ada(pl->param_dtype, pl->momentum_kind, pl->optimizer == KAON_OPT_ADAMUON);
  if (!k) return fail(KAON_E_INVALID, "no Adakaon kernel for this dtype combination");
  cudaFuncAttributes fa;
  KAON_CUDA(cudaFuncGetAttributes(&fa, (const void*)k));
  pl->double_buffer = total(2) + fa.sharedSizeBytes <= (size_t)prop.sharedMemPerBlockOptin;
  pl->smem_bytes = total(pl->double_buffer ? 2 : 1);
  if (pl->smem_bytes + fa.sharedSizeBytes > (size_t)prop.sharedMemPerBlockOptin)
    return fail(KAON_E_UNSUPPORTED, "Adakaon kernel needs %zu + %zu bytes of shared memory for rows of %d elements (limit %zu)",
                pl->smem_bytes, (size_t)fa.sharedSizeBytes, max_cols, (size_t)prop.sharedMemPerBlockOptin);
  // The limit belongs to the kernel function, not to the plan: plans with narrower rows must not lower
  // it under a plan that is still stepping, so it only ever goes up (per device).
  {
    static std::mutex mu;
    static std::map<std::pair<int, const void*>, size_t> high;
    std::lock_guard<std::mutex> lock(mu);
    size_t& h = high[std::make_pair(pl->device, (const void*)k)];
    if (pl->smem_bytes > h) {
      KAON_CUDA(cudaFuncSetAttribute((const void*)k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl->smem_bytes));
      h = pl->smem_bytes;
    }
  }
  int per_sm = 1;
  KAON_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void*)k, AT, pl->smem_bytes));
  if (per_sm < 1) return fail(KAON_E_UNSUPPORTED, "Adakaon kernel does not fit on an SM");
  pl->grid = prop.multiProcessorCount * per_sm;
  return KAON_OK;
}

// One-time set-up of the launches beside the persistent kernel.  Per factored tensor: its COUNT and
// APPLY items go to the flat COUNT / APPLY launches when its rows stream (a multiple of 8 elements; 16
// with int8 momentum; 4-bit block 128), and its STATS items to the STATS launch when they qualify
// (stats_item_ok, bf16 gradients or AdaMuon's bf16 signal).  Everything else - FINAL, the 1-D tensors,
// the stages of tensors that do not qualify - stays in the persistent kernel, whose two lists (with
// COUNT items for the cautious mask, without them otherwise) are the plan's lists minus what left.
int ensure_apply2(kaon_plan* pl) {
  if (pl->apply2 != 0) return KAON_OK;
  pl->apply2 = -1;
  const bool muon = pl->optimizer == KAON_OPT_ADAMUON;
  const int mk = muon ? KAON_M_NONE : pl->momentum_kind;
  std::vector<Task> items;
  std::vector<char> elig((size_t)pl->n_tensors, 0);
  for (int i = 0; i < pl->n_tensors; ++i) {
    const DevTensor& t = pl->h_tensors[i];
    if (t.rows <= 0 || t.numel == 0) continue;
    if ((t.cols & 7) != 0) continue;
    if (mk == KAON_M_4BIT && t.block != 128u) continue;
    if (mk == KAON_M_INT8 && (t.cols & 15) != 0) continue;
    elig[i] = 1;
    for (long long e = 0; e < t.numel; e += APPLY_CAP)
      items.push_back(Task{i, PH_ADA_APPLY, e, (int)std::min<long long>(APPLY_CAP, t.numel - e), 0, 0, 0});
  }
  if (items.empty()) return KAON_OK;
  ApplyKernel k = pick_apply(pl->param_dtype, mk, true, muon);
  ApplyKernel kc = pick_apply(pl->param_dtype, mk, false, muon);
  if (!k || !kc) return KAON_OK;
  const size_t esz = pl->param_dtype == KAON_DT_BF16 ? 2 : 4;
  const size_t mb = muon ? APPLY_CAP * esz
                         : mk == KAON_M_4BIT ? APPLY_CAP / 2 : mk == KAON_M_INT8 ? APPLY_CAP : mk == KAON_M_BF16 ? APPLY_CAP * 2
                         : mk == KAON_M_F32 ? APPLY_CAP * 4 : 0;
  pl->apply_smem = 2 * (size_t)APPLY_CAP * esz + mb;
  KAON_CUDA(cudaFuncSetAttribute((const void*)k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl->apply_smem));
  KAON_CUDA(cudaFuncSetAttribute((const void*)kc, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl->apply_smem));
  int per_sm = 0;
  KAON_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void*)k, APPLY_THREADS, pl->apply_smem));
  if (per_sm < 1) return KAON_OK;
  pl->apply_grid = pl->sm_count * per_sm;
  // the persistent kernel's lists and the STATS launch's
  const bool stats_dtype = muon || pl->param_dtype == KAON_DT_BF16;
  std::vector<Task> stats;
  pl->long_rows_ok = true;
  for (int variant = 0; variant < 2; ++variant) {   // 0: from the list without COUNT items; 1: from the full list
    const Task* src = variant ? pl->d_tasks_full : pl->d_tasks_main;
    const int ns = variant ? pl->n_tasks_full : pl->n_tasks_main;
    std::vector<Task> h((size_t)ns), keep;
    KAON_CUDA(cudaMemcpy(h.data(), src, sizeof(Task) * h.size(), cudaMemcpyDeviceToHost));
    for (const Task& t : h) {
      const bool el = elig[t.tensor] != 0;
      if ((t.phase == PH_ADA_APPLY || t.phase == PH_ADA_COUNT) && el) continue;
      if (t.phase == PH_ADA_STATS && stats_dtype && stats_item_ok(pl, t)) {
        if (variant == 0) stats.push_back(t);
        continue;
      }
      // what stays here is staged row by row: a tensor whose rows exceed a work item cannot stay
      if (t.phase != PH_ADA_FINAL && t.phase != PH_ADA_FLAT && pl->h_tensors[t.tensor].cols > CAP) pl->long_rows_ok = false;
      keep.push_back(t);
    }
    KAON_CUDA(cudaMalloc((void**)&pl->d_tasks_na[variant], sizeof(Task) * std::max<size_t>(keep.size(), 1)));
    KAON_CUDA(cudaMemcpy(pl->d_tasks_na[variant], keep.data(), sizeof(Task) * keep.size(), cudaMemcpyHostToDevice));
    pl->n_tasks_na[variant] = (int)keep.size();
    pl->device_bytes += (int64_t)(sizeof(Task) * keep.size());
  }
  if (!stats.empty()) {
    KAON_CUDA(cudaMalloc((void**)&pl->d_tasks_stats, sizeof(Task) * stats.size()));
    KAON_CUDA(cudaMemcpy(pl->d_tasks_stats, stats.data(), sizeof(Task) * stats.size(), cudaMemcpyHostToDevice));
    pl->n_tasks_stats = (int)stats.size();
    pl->device_bytes += (int64_t)(sizeof(Task) * stats.size());
  }
  KAON_CUDA(cudaMalloc((void**)&pl->d_tasks_apply2, sizeof(Task) * items.size()));
  KAON_CUDA(cudaMemcpy(pl->d_tasks_apply2, items.data(), sizeof(Task) * items.size(), cudaMemcpyHostToDevice));
  pl->n_tasks_apply2 = (int)items.size();
  pl->device_bytes += (int64_t)(sizeof(Task) * items.size());
  pl->apply2 = 1;
  return KAON_OK;
}

// The COUNT (cautious mask on) and APPLY launches over the plan's flat items; `base` carries the
// plan's pointers (and AdaMuon's signal column).
// STATS as a launch of its own over the plan's qualifying STATS items (the persistent kernel's lists
// do not hold them); KAON_OK also when there are none.
int launch_stats(kaon_plan* pl, const PlanView& base, const AdaDev& hp, cudaStream_t s) {
  if (pl->n_tasks_stats == 0) return KAON_OK;
  return launch_stats_tasks(pl, base, hp, pl->d_tasks_stats, pl->n_tasks_stats, s);
}

bool stats_item_ok(const kaon_plan* pl, const Task& t) {
  const DevTensor& dt = pl->h_tensors[t.tensor];
  return dt.cols >= 256 && (dt.cols & 7) == 0 && t.n / dt.cols <= ST_MAXROWS && (dt.aux_off & 3) == 0;
}

int launch_stats_tasks(kaon_plan* pl, const PlanView& base, const AdaDev& hp, const Task* tasks, int n, cudaStream_t s) {
  if (pl->d_counter2 == nullptr) {
    KAON_CUDA(cudaMalloc((void**)&pl->d_counter2, 256));
    pl->device_bytes += 256;
  }
  if (pl->stats_grid == 0) {
    int per_sm = 0;
    KAON_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, (const void*)ada_stats_kernel, STT, 0));
    pl->stats_grid = pl->sm_count * std::max(per_sm, 1);
  }
  PlanView vs = base;
  vs.tasks = tasks;
  vs.n_tasks = n;
  vs.task_counter = pl->d_counter2;
  KAON_CUDA(cudaMemsetAsync(pl->d_counter2, 0, sizeof(unsigned), s));
  ada_stats_kernel<<<pl->stats_grid, STT, 0, s>>>(vs, hp);
  KAON_CUDA(cudaGetLastError());
  pl->launches += 1;
  return KAON_OK;
}

int launch_count_apply(kaon_plan* pl, const PlanView& base, const AdaDev& hp, cudaStream_t s) {
  if (pl->d_counter2 == nullptr) {
    KAON_CUDA(cudaMalloc((void**)&pl->d_counter2, 256));
    pl->device_bytes += 256;
  }
  const bool muon = pl->optimizer == KAON_OPT_ADAMUON;
  const int mk = muon ? KAON_M_NONE : pl->momentum_kind;
  PlanView va = base;
  va.tasks = pl->d_tasks_apply2;
  va.n_tasks = pl->n_tasks_apply2;
  va.task_counter = pl->d_counter2;
  if (hp.cautious) {
    KAON_CUDA(cudaMemsetAsync(pl->d_counter2, 0, sizeof(unsigned), s));
    pick_apply(pl->param_dtype, mk, false, muon)<<<pl->apply_grid, APPLY_THREADS, pl->apply_smem, s>>>(va, hp);
    KAON_CUDA(cudaGetLastError());
    pl->launches += 1;
  }
  KAON_CUDA(cudaMemsetAsync(pl->d_counter2, 0, sizeof(unsigned), s));
  pick_apply(pl->param_dtype, mk, true, muon)<<<pl->apply_grid, APPLY_THREADS, pl->apply_smem, s>>>(va, hp);
  KAON_CUDA(cudaGetLastError());
  pl->launches += 1;
  return KAON_OK;
}

}  // namespace kaon

using namespace kaon;

extern "C" int kaon_adakaon_step(kaon_plan* pl, const kaon_adakaon_hparams* h, uint64_t seed,
                                 uint32_t step, void* stream) {
  if (!pl || !h) return fail(KAON_E_INVALID, "kaon_adakaon_step: null argument");
  if (pl->optimizer != KAON_OPT_ADAKAON) return fail(KAON_E_INVALID, "plan was not built for Adakaon");
  if (int rc = check_device(pl)) return rc;
  if (h->bf16_method < KAON_W_NONE || h->bf16_method > KAON_W_KAHAN) return fail(KAON_E_UNSUPPORTED, "bf16_method %d", h->bf16_method);
  if (int rc = check_kahan(pl, h->bf16_method)) return rc;
  if (!(h->clip_threshold > 0.0)) return fail(KAON_E_INVALID, "clip_threshold must be > 0");
  const bool has_m = pl->momentum_kind != KAON_M_NONE;
  if (has_m != (h->beta1 > 0.0)) return fail(KAON_E_INVALID, "beta1 %g does not match the plan's momentum kind", h->beta1);
  AdaDev hp{};
  hp.w1 = (float)(1.0 - h->beta1); hp.w1m1 = hp.w1 - 1.0f; hp.small_w1 = hp.w1 < 0.5f;
  hp.w2 = (float)(1.0 - h->beta2); hp.w2m1 = hp.w2 - 1.0f; hp.small_w2 = hp.w2 < 0.5f;
  hp.eps1 = (float)h->eps1; hp.has_eps = h->eps1 > 0.0;
  hp.clip = (float)h->clip_threshold;
  hp.lrwd = (float)(h->lr * h->weight_decay); hp.has_wd = h->weight_decay != 0.0;
  hp.upd_scale = (float)h->lr;
  hp.cautious = h->cautious != 0;
  hp.gc = h->gradient_centralization != 0;
  hp.sr = h->bf16_method == KAON_W_SR && pl->param_dtype == KAON_DT_BF16;
  hp.kahan = h->bf16_method == KAON_W_KAHAN && pl->param_dtype == KAON_DT_BF16;
  hp.int8 = pl->momentum_kind == KAON_M_INT8;
  hp.has_m = has_m;
  hp.remove = h->msam_remove != 0 && has_m;
  hp.climb = h->msam_climb != 0 && has_m;
  hp.a_remove = (float)h->msam_alpha_remove; hp.b_remove = (float)h->msam_bound_remove;
  hp.a_climb = (float)h->msam_alpha_climb; hp.b_climb = (float)h->msam_bound_climb;
  hp.step = step; hp.k0 = (uint32_t)seed; hp.k1 = (uint32_t)(seed >> 32);
  cudaStream_t s = (cudaStream_t)stream;
  PlanView v = pl->view;
  if (int rc = ensure_apply2(pl)) return rc;
  // two launches when the plan is eligible (int8 momentum also needs the COUNT stage's row maxima)
  const bool two = pl->apply2 == 1 && (pl->momentum_kind != KAON_M_INT8 || hp.cautious);
  if (pl->has_long_rows && !(two && pl->long_rows_ok))
    return fail(KAON_E_UNSUPPORTED,
                "a tensor's rows exceed a work item of %d elements: such rows are stepped by the streaming launches "
                "only (bf16 weights, a row length that is a multiple of 8 (16 with int8 momentum), 4-bit block 128, "
                "int8 momentum with the cautious mask on)", CAP);
  // the persistent kernel: FINAL, the 1-D tensors and the stages of tensors that do not stream; beside it
  // the STATS launch before and the COUNT / APPLY launches after
  if (two) { v.tasks = pl->d_tasks_na[hp.cautious ? 1 : 0]; v.n_tasks = pl->n_tasks_na[hp.cautious ? 1 : 0]; }
  else if (hp.cautious) { v.tasks = pl->d_tasks_full; v.n_tasks = pl->n_tasks_full; }
  else { v.tasks = pl->d_tasks_main; v.n_tasks = pl->n_tasks_main; }
  KAON_CUDA(cudaMemsetAsync(v.task_counter, 0, pl->counters_bytes - sizeof(unsigned), s));
  if (two)
    if (int rc = launch_stats(pl, pl->view, hp, s)) return rc;
  AdaKernel k = pick_ada(pl->param_dtype, pl->momentum_kind, false);
  k<<<pl->grid, AT, pl->smem_bytes, s>>>(v, hp, (int)x_offset_rows(pl) | (pl->double_buffer ? 1 : 0));
  KAON_CUDA(cudaGetLastError());
  pl->launches += 1;
  if (two) {
    if (int rc = launch_count_apply(pl, pl->view, hp, s)) return rc;
  }
  return KAON_OK;
}

extern "C" int kaon_msam_apply(kaon_plan* pl, double alpha, double bound, uint32_t tag, uint64_t seed,
                               uint32_t step, void* stream) {
  if (!pl) return fail(KAON_E_INVALID, "kaon_msam_apply: null plan");
  if (int rc = check_device(pl)) return rc;
  if (pl->momentum_kind == KAON_M_NONE || pl->n_tasks_axpy == 0) return KAON_OK;  // nothing carries a momentum
  AxpyKernel k = pl->param_dtype == KAON_DT_BF16 ? pick_axpy_pt<__nv_bfloat16>(pl->momentum_kind)
                                                 : pick_axpy_pt<float>(pl->momentum_kind);
  if (!k) return fail(KAON_E_INVALID, "no climb kernel for this dtype combination");
  PlanView v = pl->view;
  v.tasks = pl->d_tasks_axpy; v.n_tasks = pl->n_tasks_axpy;
  SrStream st{Philox{(uint32_t)seed, (uint32_t)(seed >> 32)}, step, tag};
  const int grid = std::min(pl->n_tasks_axpy, pl->sm_count * 8);
  k<<<grid, 256, 0, (cudaStream_t)stream>>>(v, (float)alpha, (float)bound, st);
  KAON_CUDA(cudaGetLastError());
  pl->launches += 1;
  return KAON_OK;
}

#ifdef KAON_PHASE_TIMING
extern "C" int kaon_debug_phase_cycles(unsigned long long* host16, int reset) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(host16, kaon::g_phase_cycles, sizeof(unsigned long long) * 16);
  if (reset) { unsigned long long z[16] = {0}; cudaMemcpyToSymbol(kaon::g_phase_cycles, z, sizeof z); }
  return 0;
}
#endif
