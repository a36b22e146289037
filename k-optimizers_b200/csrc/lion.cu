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
#include <type_traits>

#include "kaon_host.h"
#include "kaon_ops.cuh"
#include "kaon_packed.cuh"

namespace kaon {

struct LionDev {
  float lr, b1, w1, b2, w2, wd;
  int cautious, gc, sr, has_wd;
  uint32_t step, k0, k1;
  uint32_t rk0[KAON_PHILOX_ROUNDS], rk1[KAON_PHILOX_ROUNDS];  // Philox round keys (k + r * Weyl), from the host
  int kahan;
};

// Philox4x32-7 with the round keys read from the kernel's parameter block.
__device__ __forceinline__ void philox_rk(const LionDev& hp, uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                          uint32_t out[4]) {
#pragma unroll
  for (int r = 0; r < KAON_PHILOX_ROUNDS; ++r) {
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

// ---- update codes: 16 bits per eight elements, one nibble per element pair ----
// Nibble j covers elements 2j (e) and 2j+1 (o): bit 0 = kept_e, bit 1 = kept_o, bit 2 = neg_e, bit 3 = neg_o.
// Per element (kept, neg): (0,0) masked out; (1,0) kept, update sign +1; (1,1) kept, sign -1;
// (0,1) kept with update sign 0 (possible only with weight decay, where the mask looks at sign + wd*p).
__device__ __forceinline__ constexpr uint32_t code_bit(int k) { return 1u << (4 * (k >> 1) + (k & 1)); }
constexpr uint32_t CODE_KEPT_BITS = 0x3333u;

// MAIN item, fast path for bf16 weights/gradients: 4-bit momentum in blocks of 128, no weight decay,
// cautious on, rows a multiple of 8 elements.  Eight elements per thread and trip, arithmetic on packed
// pairs: gradient centralization as one bf16x2 subtract per pair; decode, direction c and new momentum as
// f32x2 multiplies and FMAs; the block maximum by a half-warp reduction; the 4-bit codes packed with FMAs
// (codes are small integers, exact in fp32) and one exactness check per vector; the update codes gathered
// from sign bytes (byte permutes with sign replication) instead of per-element compares.
template <bool GC>
__device__ __forceinline__ unsigned lion_fast4_bf16(const PlanView& pv, const LionDev& hp, const Task& t,
                                                    const DevTensor& d, const unsigned char* g_s,
                                                    const unsigned char* m_s, const uint32_t* mean2_s,
                                                    const float* sc_s, int tid) {
  const int nvec = t.n >> 3;
  uint16_t* cdst = reinterpret_cast<uint16_t*>(pv.codes + d.code_off + (t.e0 >> 2));
  uint32_t* mdst = reinterpret_cast<uint32_t*>(reinterpret_cast<unsigned char*>(d.m) + (t.e0 >> 1));
  const uint32_t* msrc = reinterpret_cast<const uint32_t*>(m_s);
  const long long blk0 = t.e0 >> 7;
  const f32x2 B1 = pack2(hp.b1, hp.b1), W1 = pack2(hp.w1, hp.w1), B2 = pack2(hp.b2, hp.b2), W2 = pack2(hp.w2, hp.w2);
  const f32x2 BIAS = pack2(-8388616.0f, -8388616.0f);   // -(2^23 + 8): nibble bits under 2^23 -> nibble - 8
  const f32x2 M8 = pack2(12582920.0f, 12582920.0f);     // 1.5 * 2^23 + 8: adding it rounds to integer, half to even
  const f32x2 K256 = pack2(256.0f, 256.0f);
  unsigned kept_local = 0;
  // one trip: eight elements of this thread.  GUARD = false: every lane of the warp has a vector.
  auto trip = [&](const int v, auto guard_tag) {
    constexpr bool GUARD = decltype(guard_tag)::value;
    const bool act = !GUARD || v < nvec;
    uint32_t gw[4] = {0u, 0u, 0u, 0u};
    uint32_t w = 0x88888888u;
    float sc_old = 1.0f;
    if (act) {
      const uint4 q = *reinterpret_cast<const uint4*>(g_s + (size_t)v * 16);
      gw[0] = q.x; gw[1] = q.y; gw[2] = q.z; gw[3] = q.w;
      w = msrc[v];
      sc_old = sc_s[v >> 4];
      if (GC) {
        const uint32_t mu2 = mean2_s[row_of((unsigned)t.pad + (unsigned)v * 8u, d)];
#pragma unroll
        for (int j = 0; j < 4; ++j) gw[j] = sub_bf16x2(gw[j], mu2);
      }
    }
    // nibble 2j as the low mantissa bits of 2^23 (even nibbles are the bytes of wl, odd ones of wh)
    const uint32_t wl = w & 0x0F0F0F0Fu, wh = (w >> 4) & 0x0F0F0F0Fu;
    const f32x2 SC = pack2(sc_old, sc_old);
    f32x2 G[4], C[4], N[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      G[j] = pack2(bf16lo(gw[j]), bf16hi(gw[j]));
      const f32x2 raw = pack2(__uint_as_float(__byte_perm(wl, 0x4B000000u, 0x7540u | (uint32_t)j)),
                              __uint_as_float(__byte_perm(wh, 0x4B000000u, 0x7540u | (uint32_t)j)));
      const f32x2 mo = mul2(add2(raw, BIAS), SC);
      C[j] = fma2(G[j], W1, mul2(mo, B1));
      N[j] = fma2(G[j], W2, mul2(mo, B2));
    }
    float n[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) unpack2(N[j], n[2 * j], n[2 * j + 1]);
    float amax = max3f(fabsf(n[0]), fabsf(n[1]), fabsf(n[2]));
    amax = max3f(amax, fabsf(n[3]), fabsf(n[4]));
    amax = max3f(amax, fabsf(n[5]), fabsf(n[6]));
    amax = fmaxf(amax, fabsf(n[7]));
    amax = fmaxf(half_warp_max(amax, tid), 1e-12f);
    const float sc = div7_exact(amax);
    float inv;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inv) : "f"(sc));
    const f32x2 INV = pack2(inv, inv);
    // r = rint(n*inv) + 8 + magic in one rounding; t = -(rint(n*inv)); e = n*inv - rint(n*inv) exactly
    f32x2 T[4];
    float e[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const f32x2 r = fma2(N[j], INV, M8);
      T[j] = sub2(M8, r);
      unpack2(fma2(N[j], INV, T[j]), e[2 * j], e[2 * j + 1]);
    }
    float worst = max3f(fabsf(e[0]), fabsf(e[1]), fabsf(e[2]));
    worst = max3f(worst, fabsf(e[3]), fabsf(e[4]));
    worst = max3f(worst, fabsf(e[5]), fabsf(e[6]));
    worst = fmaxf(worst, fabsf(e[7]));
    // t_k = -q_k in [-7, 7]: sum_k (8 - t_k) 16^k = 0x8888 - (t0 + 16 t1 + 256 t2 + 4096 t3), exact in fp32;
    // adding 2^23 leaves it in the low 16 mantissa bits
    float xl, xh, yl, yh;
    unpack2(fma2(T[1], K256, T[0]), xl, xh);   // (t0 + 256 t2, t1 + 256 t3)
    unpack2(fma2(T[3], K256, T[2]), yl, yh);
    const float lo4 = __fsub_rn(8423560.0f, __fmaf_rn(xh, 16.0f, xl));  // 2^23 + 0x8888 - ...
    const float hi4 = __fsub_rn(8423560.0f, __fmaf_rn(yh, 16.0f, yl));
    uint32_t word = prmt(__float_as_uint(lo4), __float_as_uint(hi4), 0x5410u);
    // ---- update codes: kept <=> c*g > 0; the update's sign is then the sign of g ----
    float a[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) unpack2(mul2(C[j], G[j]), a[2 * j], a[2 * j + 1]);
    float amin = min3f(fabsf(a[0]), fabsf(a[1]), fabsf(a[2]));
    amin = min3f(amin, fabsf(a[3]), fabsf(a[4]));
    amin = min3f(amin, fabsf(a[5]), fabsf(a[6]));
    amin = fminf(amin, fabsf(a[7]));
    // bytes 0xFF where the product is negative (masked out) / where g is negative
    const uint32_t am_lo = prmt(prmt(__float_as_uint(a[0]), __float_as_uint(a[1]), 0x00FBu),
                                prmt(__float_as_uint(a[2]), __float_as_uint(a[3]), 0x00FBu), 0x5410u);
    const uint32_t am_hi = prmt(prmt(__float_as_uint(a[4]), __float_as_uint(a[5]), 0x00FBu),
                                prmt(__float_as_uint(a[6]), __float_as_uint(a[7]), 0x00FBu), 0x5410u);
    const uint32_t gm_lo = prmt(gw[0], gw[1], 0xFDB9u), gm_hi = prmt(gw[2], gw[3], 0xFDB9u);
    // element b of each group of four lives in byte b: kept bits 0,1,4,5 and neg bits 2,3,6,7 of the code byte
    const uint32_t t_lo = ~am_lo & ((gm_lo & 0x80400804u) | 0x20100201u);
    const uint32_t t_hi = ~am_hi & ((gm_hi & 0x80400804u) | 0x20100201u);
    // the four bytes of t have disjoint bits: their sum (top byte of t * 0x01010101) is their OR
    uint32_t code16 = prmt(t_lo * 0x01010101u, t_hi * 0x01010101u, 0x0073u);
    // Rare cases, decided element by element: a product n*inv within 1e-5 of a rounding boundary (the
    // reciprocal is good to 2^-22, so |n*inv - n/sc| < 2e-6: farther out both round alike) is redone with
    // the true division; a zero gradient, a zero direction or an underflowing product c*g gets its
    // update codes from the comparisons themselves.
    if (worst > 0.5f - 1e-5f || !(amin > 0.0f)) {
      float c[8], g[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) { unpack2(C[j], c[2 * j], c[2 * j + 1]); unpack2(G[j], g[2 * j], g[2 * j + 1]); }
      word = 0;
      code16 = 0;
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int qi = min(max((int)rintf(__fdiv_rn(n[k], sc)), -7), 7);
        word |= (uint32_t)(qi + 8) << (4 * k);
        if (c[k] > 0.0f && g[k] > 0.0f) code16 |= code_bit(k);
        if (c[k] < 0.0f && g[k] < 0.0f) code16 |= 5u * code_bit(k);
      }
    }
    if (act) {
      stg_u32(mdst + v, word);
      if ((v & 15) == 0) stg_f32(d.m_scale + blk0 + (v >> 4), sc);
      stg_u16(cdst + v, code16);
      kept_local += __popc(code16 & CODE_KEPT_BITS);
    }
  };
  const int nfull = nvec & ~31;  // vectors in trips whose whole warp is active
  for (int v = tid; v < nfull; v += NTHREADS) trip(v, std::false_type{});
  if (nfull != nvec && tid < 32) trip(nfull + tid, std::true_type{});
  return kept_local;
}

// Full-vector fast path of the MAIN item for fp32 weights (4-bit momentum, no weight decay, cautious on,
// rows a multiple of 8 elements): no per-element guards, the eight 4-bit codes assembled with one
// shift-add each, one exactness check per vector.
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
        const float mu = mean_s[row_of((unsigned)t.pad + (unsigned)v * 8u, d)];
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
      if (fminf(c, g[k]) > 0.0f) pos |= code_bit(k);
      if (fmaxf(c, g[k]) < 0.0f) neg |= 5u * code_bit(k);
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
      cdst[v] = (uint16_t)(pos | neg);
      kept_local += __popc((pos | neg) & CODE_KEPT_BITS);
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
  bool fast = false;
  if constexpr (MK == KAON_M_4BIT)  // the fast paths know blocks of 128 (or one block in the first 16 lanes)
    fast = !hp.has_wd && hp.cautious && (n & 7) == 0 && ((d.rows <= 0) || ((C & 7) == 0)) && (d.bshift == 7 || d.bshift >= 31);
  // the bf16 fast path subtracts the mean from packed pairs: it reads the mean as two bf16 copies
  const bool mean_packed = fast && E::IS_BF16;
  if (do_gc && d.chunk_rows < 0) {
    // a tensor cut into flat runs (rows longer than a work item, or rows that cannot be grouped on block
    // boundaries): the run touches parts of a few rows, whose means lion_rowmean_kernel left in the scratch
    const int touched = (int)(((long long)t.pad + n + C - 1) / C);
    for (int r = tid; r < touched; r += NTHREADS) {
      const float mean = __ldcg(pv.aux + d.aux_off + t.row0 + r);
      if (mean_packed) reinterpret_cast<uint32_t*>(mean_s)[r] = pack_bf16_rn(mean, mean);
      else mean_s[r] = mean;
    }
  } else if (do_gc) {
    const int warp = tid >> 5, lane = tid & 31;
    for (int r = warp; r < nrows; r += NTHREADS / 32) {
      const unsigned char* rowp = g_s + (size_t)r * C * E::BYTES;
      float s = 0.0f;
      if ((C & 7) == 0) {
        if constexpr (E::IS_BF16) {
          f32x2 acc = pack2(0.0f, 0.0f), acc2 = pack2(0.0f, 0.0f);
          for (int v = lane; v < (C >> 3); v += 32) {
            const uint4 q = *reinterpret_cast<const uint4*>(rowp + (size_t)v * 16);
            acc = add2(acc, add2(pack2(bf16lo(q.x), bf16hi(q.x)), pack2(bf16lo(q.y), bf16hi(q.y))));
            acc2 = add2(acc2, add2(pack2(bf16lo(q.z), bf16hi(q.z)), pack2(bf16lo(q.w), bf16hi(q.w))));
          }
          acc = add2(acc, acc2);
          s = acc.x + acc.y;
        } else {
          for (int v = lane; v < (C >> 3); v += 32) {
            float x[8];
            E::load8(rowp + (size_t)v * 8 * E::BYTES, x);
            s += ((x[0] + x[1]) + (x[2] + x[3])) + ((x[4] + x[5]) + (x[6] + x[7]));
          }
        }
      } else {
        for (int i = lane; i < C; i += 32) s += E::load1(rowp, i);
      }
      s = warp_sum(s);
      if (lane == 0) {
        float mean = __fdiv_rn(s, (float)C);
        if (mean_packed) reinterpret_cast<uint32_t*>(mean_s)[r] = pack_bf16_rn(mean, mean);
        else mean_s[r] = E::IS_BF16 ? round_bf16(mean) : mean;
      }
    }
  }
  if constexpr (MK == KAON_M_4BIT) {  // old block scales of the chunk (the fast path reads them from here)
    if (fast) {
      const int nblk = d.block == 128u ? (n + 127) >> 7 : 1;
      const long long b0 = d.block == 128u ? (t.e0 >> 7) : 0;
      for (int b = tid; b < nblk; b += NTHREADS) sc_s[b] = d.m_scale[b0 + b];
    }
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
        float mu = mean_s[row_of((unsigned)t.pad + (unsigned)v * 8u, d)];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float x = __fsub_rn(gv[k], mu);
          gv[k] = (k < cnt) ? (E::IS_BF16 ? round_bf16(x) : x) : 0.0f;
        }
      } else {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          float x = __fsub_rn(gv[k], mean_s[k < cnt ? row_of((unsigned)t.pad + (unsigned)(v * 8 + k), d) : 0]);
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
  if (fast) {
    if constexpr (MK == KAON_M_4BIT) {
      if constexpr (E::IS_BF16)
        kept_local = do_gc ? lion_fast4_bf16<true>(pv, hp, t, d, g_s, m_s, reinterpret_cast<const uint32_t*>(mean_s), sc_s, tid)
                           : lion_fast4_bf16<false>(pv, hp, t, d, g_s, m_s, reinterpret_cast<const uint32_t*>(mean_s), sc_s, tid);
      else
        kept_local = do_gc ? lion_fast4<PT, true>(pv, hp, t, d, g_s, m_s, mean_s, sc_s, tid)
                           : lion_fast4<PT, false>(pv, hp, t, d, g_s, m_s, mean_s, sc_s, tid);
    }
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
      blk = blk_of(d, t.e0 + (long long)v * 8);
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
      const int lanes = blk_lanes(d);  // threads that share a block: consecutive lanes of one warp
      a = group_max(a, lanes);
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
        if ((v & (lanes - 1)) == 0) d.m_scale[blk] = sc;
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
        uint32_t code16 = 0;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          if ((kept >> k) & 1u) code16 |= sg[k] > 0 ? code_bit(k) : (sg[k] < 0 ? 5u * code_bit(k) : 4u * code_bit(k));
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
  __syncthreads();
  if (tid == 0) {
    __threadfence();  // the CTA's stores of this item (ordered before the barrier) go out before the signal
    if (hp.cautious) {
      unsigned tot = 0;
      for (int w = 0; w < NTHREADS / 32; ++w) tot += red_s[w];
      atomicAdd(pv.kept + t.tensor, tot);
    }
    signal_counter(pv.done + t.tensor, 1u);
  }
}

// APPLY item: weights of the run [e0, e0+n) once the tensor's kept count is complete.
// lut_s (16 entries): for the fast path, the fp32 update pair of every value a code nibble can take.
template <typename PT, bool MIRROR>
__device__ void lion_apply(const PlanView& pv, const LionDev& hp, const Task& t, float2* lut_s, int tid) {
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
    lut_s += (tid >> 5) * 16;  // this warp's copy of the table
    const int lane = tid & 31;
    if (lane < 16) {  // nibble = kept_e | kept_o << 1 | neg_e << 2 | neg_o << 3
      const float de = (lane & 1) ? ((lane & 4) ? -vpos : vpos) : 0.0f;
      const float dd = (lane & 2) ? ((lane & 8) ? -vpos : vpos) : 0.0f;
      lut_s[lane] = make_float2(de, dd);
    }
    __syncwarp();
    // full vectors, four per trip: all loads are issued before the first use.  Per pair: the update pair
    // from the table, p - update as one packed subtract, 16 noise bits added below the kept mantissa.
    const int nfull = n >> 3;
    auto one = [&](const uint4 pw4, const uint32_t c16, const int vv) {
      const uint64_t q = (uint64_t)((t.e0 >> 3) + vv);
      uint32_t nz[4];
      philox_rk(hp, (uint32_t)q, d.tensor_id, hp.step, (uint32_t)KAON_TAG_UPDATE | ((uint32_t)(q >> 32) << 8), nz);
      uint32_t pw[4] = {pw4.x, pw4.y, pw4.z, pw4.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 dl = lut_s[(c16 >> (4 * j)) & 15u];
        float r0, r1;
        unpack2(sub2(pack2(bf16lo(pw[j]), bf16hi(pw[j])), pack2(dl.x, dl.y)), r0, r1);
        const uint32_t b0 = __float_as_uint(r0) + (nz[j] & 0xffffu);
        const uint32_t b1 = __float_as_uint(r1) + (nz[j] >> 16);
        pw[j] = __byte_perm(b0, b1, 0x7632);
      }
      const uint4 out = make_uint4(pw[0], pw[1], pw[2], pw[3]);
      *reinterpret_cast<uint4*>(pbase + (size_t)vv * 16) = out;
      mirror16(MIRROR ? &pv.peers : nullptr, pbase + (size_t)vv * 16, out);
    };
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
      for (int u = 0; u < 4; ++u) one(pw4[u], c16[u], v + u * NTHREADS);
    }
    for (; v < nfull; v += NTHREADS)
      one(*reinterpret_cast<const uint4*>(pbase + (size_t)v * 16),
          __ldcg(reinterpret_cast<const unsigned short*>(cbase + (size_t)v * 2)), v);
    v_begin = v;   // only a ragged last vector can be left
  }
  for (int v = v_begin; v < nvec; v += NTHREADS) {
    const int cnt = min(8, n - v * 8);
    const uint32_t c16 = __ldcg(reinterpret_cast<const unsigned short*>(cbase + (size_t)v * 2));
    float dl[8];
    float pvals[8];
    if (hp.has_wd) load8_guard<PT>(pbase + (size_t)v * 8 * E::BYTES, cnt, pvals);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const uint32_t kb = (c16 >> (4 * (k >> 1) + (k & 1))) & 1u, nb = (c16 >> (4 * (k >> 1) + (k & 1) + 2)) & 1u;
      if (hp.has_wd) {
        // kept elements: (kept, neg) = (1,0) sign +1, (1,1) sign -1, (0,1) sign 0
        const float sgn = kb ? (nb ? -1.0f : 1.0f) : 0.0f;
        const float dv = __fmaf_rn(pvals[k], hp.wd, sgn);
        dl[k] = (kb | nb) ? __fmul_rn(__fdiv_rn(dv, denom), hp.lr) : 0.0f;
      } else {
        dl[k] = kb ? (nb ? -vpos : vpos) : 0.0f;
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
  __shared__ float2 lut_s[(NTHREADS / 32) * 16];
  unsigned char* g_s = dyn;
  unsigned char* m_s = dyn + (size_t)CAP * Elems<PT>::BYTES;
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
  unsigned parity = 0;
  int slot = 0;
  int cur = next_s[0];
  while (cur < pv.n_tasks) {
    claim_next(slot ^ 1);
    const Task t = pv.tasks[cur];
    if (t.phase == PH_LION_MAIN) {
      lion_main<PT, MK, MIRROR>(pv, hp, t, g_s, m_s, mean_s, rowmax_s, scale_s, sc_s, &bar, parity, red_s, tid);
    } else {  // (a MAIN item ends with a barrier of its own)
      lion_apply<PT, MIRROR>(pv, hp, t, lut_s, tid);
      __syncthreads();
    }
    slot ^= 1;
    cur = next_s[slot];
  }
}

// Row means (gradient centralization) of the tensors that are cut into flat runs, one warp per row, into
// the plan's scratch: bf16-rounded for bf16 gradients, as the staged rows' means are.
template <typename PT>
__global__ void lion_rowmean_kernel(PlanView pv, const int* tensor_ids, int n_ids) {
  using E = Elems<PT>;
  const int lane = threadIdx.x & 31;
  const long long warp0 = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
  for (int k = 0; k < n_ids; ++k) {
    const DevTensor d = pv.tensors[tensor_ids[k]];
    const unsigned char* g = reinterpret_cast<const unsigned char*>(pv.grads[tensor_ids[k]]);
    if (g == nullptr) continue;
    const int C = d.cols;
    for (long long r = warp0; r < d.rows; r += nwarps) {
      const unsigned char* rowp = g + (size_t)r * C * E::BYTES;
      float s = 0.0f;
      if ((C & 7) == 0 && ((reinterpret_cast<uintptr_t>(rowp) & 15) == 0)) {
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
        const float mean = __fdiv_rn(s, (float)C);
        pv.aux[d.aux_off + r] = E::IS_BF16 ? round_bf16(mean) : mean;
      }
    }
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
  for (int r = 0; r < KAON_PHILOX_ROUNDS; ++r) { hp.rk0[r] = hp.k0 + 0x9E3779B9u * (uint32_t)r; hp.rk1[r] = hp.k1 + 0xBB67AE85u * (uint32_t)r; }
  cudaStream_t s = (cudaStream_t)stream;
  PlanView v = pl->view;
  if (hp.cautious) { v.tasks = pl->d_tasks_full; v.n_tasks = pl->n_tasks_full; }
  else { v.tasks = pl->d_tasks_main; v.n_tasks = pl->n_tasks_main; }
  KAON_CUDA(cudaMemsetAsync(v.task_counter, 0, pl->counters_bytes - sizeof(unsigned), s));
  if (pl->n_flat_tensors > 0 && hp.gc) {  // row means of the tensors cut into flat runs
    if (pl->param_dtype == KAON_DT_BF16) lion_rowmean_kernel<__nv_bfloat16><<<pl->sm_count * 4, 256, 0, s>>>(v, pl->d_flat_tensors, pl->n_flat_tensors);
    else lion_rowmean_kernel<float><<<pl->sm_count * 4, 256, 0, s>>>(v, pl->d_flat_tensors, pl->n_flat_tensors);
    KAON_CUDA(cudaGetLastError());
    pl->launches += 1;
  }
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
  d.tensor_id = t->tensor_id; d.block = t->block; d.bshift = t->block == 128 ? 7 : 31;
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
  for (int r = 0; r < KAON_PHILOX_ROUNDS; ++r) { hp.rk0[r] = hp.k0 + 0x9E3779B9u * (uint32_t)r; hp.rk1[r] = hp.k1 + 0xBB67AE85u * (uint32_t)r; }

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
