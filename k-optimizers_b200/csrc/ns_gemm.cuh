// bf16 GEMM for the Newton–Schulz iteration on sm_100a tensor cores:
//   out[M,N] = bf16( alpha * sum_k A(m,k) * B(n,k)  +  beta * aux[M,N] )
// tcgen05.mma (cta_group::1, kind::f16, M=128, N<=256, K=16) issued by one thread, operands staged in
// shared memory by TMA (128-byte swizzle, no multicast), fp32 accumulators in tensor memory, read back
// with tcgen05.ld for the fused epilogue.  Either operand may be K-major (matrix stored [MN, K], K
// contiguous) or MN-major (stored [K, MN], MN contiguous), which is what lets the iteration run on a
// matrix in its native orientation without ever transposing it in memory.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "kaon_stage.cuh"

namespace kaon {

constexpr int G_BM = 128;          // rows of the output tile = UMMA M
constexpr int G_BK = 64;           // K elements per stage (one 128-byte swizzle atom of bf16)
constexpr int G_STAGES = 2;
constexpr int G_A_BYTES = G_BM * G_BK * 2;  // 16 KiB
constexpr int G_MAX_BN = 256;
constexpr int G_THREADS = 128;
constexpr unsigned G_WAIT_LIMIT = 1u << 22;

struct GemmParams {
  int M, N, K;
  int a_mn, b_mn;    // 0 = K-major operand, 1 = MN-major operand
  int BN;            // 64, 128, 192 or 256
  float alpha, beta;
  const float* dev_scale;    // optional device pair {alpha multiplier, beta multiplier} (e.g. 1/norm)
  const __nv_bfloat16* aux;  // [M, ld_aux] or null (beta ignored)
  long long ld_aux;
  __nv_bfloat16* out;        // [M, ld_out]
  long long ld_out;
  unsigned* status;          // device status word (bounded waits)
  int sym;                   // the product is symmetric (M == N, same operand on both sides): tiles that lie
                             // wholly below the diagonal are not computed; every computed tile also stores
                             // its transpose, which fills them
};

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
          smem_u32(dst)),
      "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

__device__ __forceinline__ bool mbar_wait_limit(uint64_t* bar, unsigned parity) {
  for (unsigned i = 0; i < G_WAIT_LIMIT; ++i)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}

// 64-bit shared-memory matrix descriptor, 128-byte swizzle.
//  K-major : rows of 128 B (64 bf16 of K), 8-row groups 1024 B apart (SBO); LBO unused (1).
//  MN-major: K rows of 128 B (64 bf16 of MN), 8-K-row groups 1024 B apart (SBO), the next 64 MN
//            elements LBO bytes further (one 64x64 TMA box = 8192 B).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr, bool mn_major) {
  const uint64_t lbo = mn_major ? (8192u >> 4) : 1u;
  const uint64_t sbo = 1024u >> 4;
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (lbo << 16) | (sbo << 32) | (1ull << 46) | (2ull << 61);
}

__device__ __forceinline__ uint32_t umma_idesc(int n, bool a_mn, bool b_mn) {
  return (1u << 4) /* D = f32 */ | (1u << 7) /* A = bf16 */ | (1u << 10) /* B = bf16 */ |
         ((a_mn ? 1u : 0u) << 15) | ((b_mn ? 1u : 0u) << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(G_BM >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t tmem_c, uint64_t da, uint64_t db, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_c), "l"(da), "l"(db), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t v[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32"
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15,"
      " %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}

// ---- persistent, warp-specialised kernel ----
// One CTA per SM walks the output tiles (128 x BN) in a fixed stride.  Warp 0 (one lane) feeds a ring of
// G_STAGES shared-memory stages by TMA; warp 1 (one lane) issues the MMAs into one of two accumulators in
// tensor memory (2 x 256 columns, allocated once per CTA); warps 2-5 drain the other accumulator
// (tcgen05.ld, fused epilogue, bf16 stores), so that a tile's epilogue runs under the next tile's MMAs.
// In symmetric mode only the tiles that reach the diagonal are enumerated.
// Every wait is bounded: a wait that runs out raises a flag in shared memory, every role leaves its
// loops when it sees the flag, the CTA records the status code and frees its tensor memory.

constexpr int G2_THREADS = 192;
constexpr int G2_STAGES = 4;
constexpr int G2_ACC_COLS = 256;   // tensor-memory columns of one accumulator

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// wait with a poll limit, giving up early when another role has failed
__device__ __forceinline__ bool mbar_wait_or_fail(uint64_t* bar, unsigned parity, volatile int* fail) {
  for (unsigned i = 0; i < G_WAIT_LIMIT; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 1023u) == 1023u && *fail) return false;
  }
  *fail = 1;
  return false;
}

// computed-tile index c -> tile coordinates (rows of tiles are walked in order; in symmetric mode a row
// starts at the first tile that reaches the diagonal)
__device__ __forceinline__ void tile_coords(const GemmParams& p, int tn, int c, int& mi, int& ni) {
  mi = 0;
  while (true) {
    const int skip = p.sym ? min(tn, (mi * G_BM) / p.BN) : 0;
    const int cnt = tn - skip;
    if (c < cnt) { ni = skip + c; return; }
    c -= cnt;
    ++mi;
  }
}

__global__ void __launch_bounds__(G2_THREADS, 1)
ns_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, GemmParams p,
               int total_tiles) {
  extern __shared__ __align__(1024) unsigned char gsm[];
  __shared__ __align__(8) uint64_t full_bar[G2_STAGES];
  __shared__ __align__(8) uint64_t empty_bar[G2_STAGES];
  __shared__ __align__(8) uint64_t accf_bar[2];   // accumulator complete (MMA -> epilogue)
  __shared__ __align__(8) uint64_t acce_bar[2];   // accumulator drained (epilogue -> MMA)
  __shared__ uint32_t tmem_base_s;
  __shared__ int fail_s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b_bytes = p.BN * G_BK * 2;
  const int stage_bytes = G_A_BYTES + b_bytes;
  // 1024-byte aligned tile base (the swizzle pattern is a function of address bits 4..9)
  unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(gsm) + 1023) & ~uintptr_t(1023));
  const int kblocks = (p.K + G_BK - 1) / G_BK;
  const int tn = (p.N + p.BN - 1) / p.BN;
  volatile int* fail = &fail_s;

  if (tid == 0) {
    for (int s = 0; s < G2_STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&accf_bar[b], 1); mbar_init(&acce_bar[b], 4); }
    fail_s = 0;
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_s)), "r"(2u * G2_ACC_COLS) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;

  if (warp == 0) {
    // ---- TMA producer ----
    if (lane == 0) {
      unsigned it = 0;
      for (int c = blockIdx.x; c < total_tiles && !*fail; c += gridDim.x) {
        int mi, ni;
        tile_coords(p, tn, c, mi, ni);
        const int m0 = mi * G_BM, n0 = ni * p.BN;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % G2_STAGES;
          const unsigned use = it / G2_STAGES;
          if (use > 0 && !mbar_wait_or_fail(&empty_bar[s], (use - 1u) & 1u, fail)) break;
          unsigned char* a_dst = tiles + (size_t)s * stage_bytes;
          unsigned char* b_dst = a_dst + G_A_BYTES;
          mbar_expect_tx(&full_bar[s], (unsigned)stage_bytes);
          const int k0 = kb * G_BK;
          if (p.a_mn) {
            for (int j = 0; j < G_BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, m0 + 64 * j, k0, &full_bar[s]);
          } else {
            tma_load_2d(a_dst, &tmA, k0, m0, &full_bar[s]);
          }
          if (p.b_mn) {
            for (int j = 0; j < p.BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, n0 + 64 * j, k0, &full_bar[s]);
          } else {
            tma_load_2d(b_dst, &tmB, k0, n0, &full_bar[s]);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---- MMA issuer ----
    if (lane == 0) {
      const uint32_t idesc = umma_idesc(p.BN, p.a_mn != 0, p.b_mn != 0);
      unsigned it = 0, tcount = 0;
      for (int c = blockIdx.x; c < total_tiles && !*fail; c += gridDim.x, ++tcount) {
        const unsigned buf = tcount & 1u, use = tcount >> 1;
        if (use > 0 && !mbar_wait_or_fail(&acce_bar[buf], (use - 1u) & 1u, fail)) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t tmem_acc = tmem_base + buf * G2_ACC_COLS;
        bool ok = true;
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % G2_STAGES;
          if (!mbar_wait_or_fail(&full_bar[s], (it / G2_STAGES) & 1u, fail)) { ok = false; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(tiles + (size_t)s * stage_bytes);
          const uint32_t b_addr = a_addr + G_A_BYTES;
#pragma unroll
          for (int k = 0; k < G_BK / 16; ++k) {
            const uint64_t da = umma_desc(a_addr + (p.a_mn ? k * 2048 : k * 32), p.a_mn != 0);
            const uint64_t db = umma_desc(b_addr + (p.b_mn ? k * 2048 : k * 32), p.b_mn != 0);
            umma_f16(tmem_acc, da, db, idesc, (kb | k) ? 1u : 0u);
          }
          umma_commit(&empty_bar[s]);  // frees the stage once these MMAs have read it
        }
        if (!ok) break;
        umma_commit(&accf_bar[buf]);   // accumulator complete
      }
    }
  } else {
    // ---- epilogue: warps 2..5; a warp may touch the 32 tensor-memory lanes of its quarter (warp % 4) ----
    const int quarter = warp & 3;
    const float alpha = p.dev_scale ? p.alpha * p.dev_scale[0] : p.alpha;
    const float beta = p.dev_scale ? p.beta * p.dev_scale[1] : p.beta;
    unsigned tcount = 0;
    for (int c = blockIdx.x; c < total_tiles; c += gridDim.x, ++tcount) {
      int mi, ni;
      tile_coords(p, tn, c, mi, ni);
      const int m0 = mi * G_BM, n0 = ni * p.BN;
      const unsigned buf = tcount & 1u, use = tcount >> 1;
      if (!mbar_wait_or_fail(&accf_bar[buf], use & 1u, fail)) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t tmem_acc = tmem_base + buf * G2_ACC_COLS;
      const int row = m0 + quarter * 32 + lane;
      for (int c0 = 0; c0 < p.BN; c0 += 32) {
        uint32_t v[32];
        tmem_ld32(tmem_acc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const int col = n0 + c0;
        if (row < p.M && col < p.N) {
          __nv_bfloat16* orow = p.out + (long long)row * p.ld_out + col;
          const __nv_bfloat16* arow = p.aux ? p.aux + (long long)row * p.ld_aux + col : nullptr;
          const bool full = (col + 32 <= p.N) && ((reinterpret_cast<uintptr_t>(orow) & 15) == 0) &&
                            (!arow || (reinterpret_cast<uintptr_t>(arow) & 15) == 0);
          if (full) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              float x[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
              if (arow) Elems<__nv_bfloat16>::load8(arow + q * 8, x);
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e) {
                const float r0 = __uint_as_float(v[q * 8 + 2 * e]) * alpha + beta * x[2 * e];
                const float r1 = __uint_as_float(v[q * 8 + 2 * e + 1]) * alpha + beta * x[2 * e + 1];
                w[e] = pack_bf16_rn(r0, r1);
              }
              *reinterpret_cast<uint4*>(orow + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
              if (p.sym) {  // transpose: out[col + j, row]; lanes are consecutive rows, i.e. consecutive addresses
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  unsigned short* mlo = reinterpret_cast<unsigned short*>(p.out + (long long)(col + q * 8 + 2 * e) * p.ld_out + row);
                  unsigned short* mhi = reinterpret_cast<unsigned short*>(p.out + (long long)(col + q * 8 + 2 * e + 1) * p.ld_out + row);
                  *mlo = (unsigned short)(w[e] & 0xffffu);
                  *mhi = (unsigned short)(w[e] >> 16);
                }
              }
            }
          } else {
            for (int e = 0; e < 32 && col + e < p.N; ++e) {
              const float x = arow ? __bfloat162float(arow[e]) : 0.0f;
              const __nv_bfloat16 r = __float2bfloat16_rn(__uint_as_float(v[e]) * alpha + beta * x);
              orow[e] = r;
              if (p.sym) p.out[(long long)(col + e) * p.ld_out + row] = r;
            }
          }
        }
      }
      // this warp has read its part of the accumulator: hand the buffer back to the MMA issuer
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&acce_bar[buf]);
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (tid == 0 && fail_s) atomicCAS(p.status, 0u, 20001u);
  if (warp == 1) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(2u * G2_ACC_COLS) : "memory");
  }
}

}  // namespace kaon
