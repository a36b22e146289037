// Newton–Schulz orthogonalisation (reference src/kaon/adamuon.py:97-149) as a chain of tcgen05 GEMMs.
//
//   X = M / (||M||_F + 1e-7);  steps x { A = X X^T;  B = b A + c A A;  X = a X + B X }
// run on the matrix in its stored orientation: for a wide matrix [r, k] (r <= k) X is used as stored;
// for a tall one [k, r] the stored matrix is X^T, A = (X^T)^T (X^T) takes both operands MN-major and
// X^T <- a X^T + X^T B uses that B is symmetric.  The 1/norm scaling is folded into the epilogues of
// the first iteration (A = s^2 M M^T, X1 = s (a M + B M)), so the unnormalised bf16 matrix is read
// directly and no normalisation pass exists.  Every product rounds to bf16 once, after the fused fp32
// epilogue (the reference rounds after every op; both sit within its own 2e-2 tolerance).
#include <cuda.h>

#include <algorithm>
#include <cmath>

#include "kaon_host.h"
#include "ns_gemm.cuh"

namespace kaon {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Tensor map of a row-major bf16 matrix [outer, inner] with row stride ld (elements), box = [box_outer, 64].
static int make_map(CUtensorMap* m, const void* base, long long inner, long long outer, long long ld, int box_outer) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return fail(KAON_E_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_outer};
  cuuint32_t es[2] = {1u, 1u};
  CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(KAON_E_CUDA, "cuTensorMapEncodeTiled failed with %d (inner %lld outer %lld ld %lld)", (int)r, inner, outer, ld);
  return KAON_OK;
}

// Plain fp32-accumulate GEMM for shapes TMA cannot describe (row stride not a multiple of 16 bytes).
__global__ void ns_gemm_simple_kernel(const __nv_bfloat16* A, int a_mn, long long lda, const __nv_bfloat16* B,
                                      int b_mn, long long ldb, GemmParams p) {
  const long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (idx >= (long long)p.M * p.N) return;
  const int i = (int)(idx / p.N), j = (int)(idx % p.N);
  float acc = 0.0f;
  for (int k = 0; k < p.K; ++k) {
    const float a = __bfloat162float(a_mn ? A[(long long)k * lda + i] : A[(long long)i * lda + k]);
    const float b = __bfloat162float(b_mn ? B[(long long)k * ldb + j] : B[(long long)j * ldb + k]);
    acc += a * b;
  }
  const float alpha = p.dev_scale ? p.alpha * p.dev_scale[0] : p.alpha;
  const float beta = p.dev_scale ? p.beta * p.dev_scale[1] : p.beta;
  const float x = p.aux ? __bfloat162float(p.aux[(long long)i * p.ld_aux + j]) : 0.0f;
  p.out[(long long)i * p.ld_out + j] = __float2bfloat16_rn(acc * alpha + beta * x);
}

static int g_gemm_sms[64] = {0};  // multiprocessors per device, once the kernel's shared-memory limit is set

// out[M,N] = bf16(alpha * A(m,:) . B(n,:) + beta * aux)
int launch_ns_gemm(const __nv_bfloat16* A, bool a_mn, long long lda, const __nv_bfloat16* B, bool b_mn, long long ldb,
                   int M, int N, int K, float alpha, float beta, const float* dev_scale, const __nv_bfloat16* aux,
                   long long ld_aux, __nv_bfloat16* out, long long ld_out, unsigned* status, cudaStream_t stream,
                   long long* launches, bool sym = false) {
  GemmParams p{};
  p.sym = sym && M == N ? 1 : 0;
  p.M = M; p.N = N; p.K = K; p.a_mn = a_mn; p.b_mn = b_mn;
  p.alpha = alpha; p.beta = aux ? beta : 0.0f; p.dev_scale = dev_scale;
  p.aux = aux; p.ld_aux = ld_aux; p.out = out; p.ld_out = ld_out; p.status = status;
  const bool tma_ok = (lda % 8 == 0) && (ldb % 8 == 0) && ((uintptr_t)A % 16 == 0) && ((uintptr_t)B % 16 == 0);
  if (launches) *launches += 1;
  if (!tma_ok) {
    const long long total = (long long)M * N;
    ns_gemm_simple_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(A, a_mn, lda, B, b_mn, ldb, p);
    KAON_CUDA(cudaGetLastError());
    return KAON_OK;
  }
  p.BN = N >= 256 ? 256 : (N > 64 ? 128 : 64);
  if (p.sym && N >= 256) {
    // Persistent CTAs share the computed tiles out evenly: take the tile width whose busiest SM has the
    // least work (tiles per SM x width); narrower tiles balance better but feed the tensor cores worse,
    // so 256 keeps a 10 % edge.
    int dev = 0, sms = 148;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    auto cost = [&](int bn) {
      long long tiles = 0;
      for (int m0 = 0; m0 < M; m0 += G_BM)
        for (int n0 = 0; n0 < N; n0 += bn)
          if (n0 + bn > m0) ++tiles;
      return ((tiles + sms - 1) / sms) * (long long)bn;
    };
    if (cost(192) * 100 < cost(256) * 90) p.BN = 192;
  }
  CUtensorMap ma, mb;
  int rc;
  if (a_mn) rc = make_map(&ma, A, M, K, lda, 64); else rc = make_map(&ma, A, K, M, lda, G_BM);
  if (rc) return rc;
  if (b_mn) rc = make_map(&mb, B, N, K, ldb, 64); else rc = make_map(&mb, B, K, N, ldb, p.BN);
  if (rc) return rc;
  // always the shared memory of the widest tile: one CTA per SM, whose tensor-memory allocation (all 512
  // columns) then never waits for a neighbour
  const size_t smem = 1024 + (size_t)G2_STAGES * (G_A_BYTES + (size_t)G_MAX_BN * G_BK * 2);
  int dev = 0;
  KAON_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(KAON_E_UNSUPPORTED, "device index %d", dev);
  if (!g_gemm_sms[dev]) {
    KAON_CUDA(cudaFuncSetAttribute((const void*)ns_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                   (int)(1024 + (size_t)G2_STAGES * (G_A_BYTES + (size_t)G_MAX_BN * G_BK * 2))));
    int sms = 0;
    KAON_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    g_gemm_sms[dev] = sms;
  }
  // computed tiles: all of them, or in symmetric mode those that reach the diagonal
  const int tm = (M + G_BM - 1) / G_BM, tn = (N + p.BN - 1) / p.BN;
  int total = 0;
  for (int mi = 0; mi < tm; ++mi) total += tn - (p.sym ? std::min(tn, (mi * G_BM) / p.BN) : 0);
  const int grid = std::min(total, g_gemm_sms[dev]);
  ns_gemm_kernel<<<grid, G2_THREADS, smem, stream>>>(ma, mb, p, total);
  KAON_CUDA(cudaGetLastError());
  return KAON_OK;
}

// sum of squares of a bf16 matrix -> scal = {s*s, 0, s, s} with s = 1 / bf16(bf16(||x||) + 1e-7)
__global__ void ns_sumsq_kernel(const __nv_bfloat16* x, long long n, double* partial) {
  __shared__ double red[8];
  double acc = 0.0;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float v = __bfloat162float(x[i]);
    acc += (double)v * (double)v;
  }
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    double t = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
    partial[blockIdx.x] = t;
  }
}

__global__ void ns_scale_kernel(const double* partial, int n, float* scal) {
  if (threadIdx.x == 0 && blockIdx.x == 0) {
    double t = 0.0;
    for (int i = 0; i < n; ++i) t += partial[i];
    const float nrm = round_bf16((float)sqrt(t));
    const float den = round_bf16(nrm + 1e-7f);
    const float s = 1.0f / den;
    scal[0] = s * s; scal[1] = 0.0f; scal[2] = s; scal[3] = s;
  }
}

constexpr int NS_PARTIALS = 296;

size_t ns_workspace_bytes(long long R, long long C) {
  const long long r = std::min(R, C);
  auto up = [](size_t x) { return (x + 255) / 256 * 256; };
  return up((size_t)R * C * 2) + 2 * up((size_t)r * r * 2) + up(NS_PARTIALS * 8) + 256;
}

// x_in [R,C] bf16 (unnormalised) -> out [R,C] bf16.  out may not alias x_in.  ws >= ns_workspace_bytes.
int ns_run(const __nv_bfloat16* x_in, long long R, long long C, int steps, __nv_bfloat16* out, void* ws,
           unsigned* status, cudaStream_t stream, long long* launches) {
  const bool tall = R > C;             // stored matrix is X^T (k rows, r columns)
  const long long r = tall ? C : R, k = tall ? R : C;
  auto up = [](size_t x) { return (x + 255) / 256 * 256; };
  unsigned char* w = reinterpret_cast<unsigned char*>(ws);
  __nv_bfloat16* xb = reinterpret_cast<__nv_bfloat16*>(w); w += up((size_t)R * C * 2);
  __nv_bfloat16* Am = reinterpret_cast<__nv_bfloat16*>(w); w += up((size_t)r * r * 2);
  __nv_bfloat16* Bm = reinterpret_cast<__nv_bfloat16*>(w); w += up((size_t)r * r * 2);
  double* partial = reinterpret_cast<double*>(w); w += up(NS_PARTIALS * 8);
  float* scal = reinterpret_cast<float*>(w);
  ns_sumsq_kernel<<<NS_PARTIALS, 256, 0, stream>>>(x_in, R * C, partial);
  ns_scale_kernel<<<1, 32, 0, stream>>>(partial, NS_PARTIALS, scal);
  KAON_CUDA(cudaGetLastError());
  if (launches) *launches += 2;
  const float a = 3.4445f, b = -4.7750f, c = 2.0315f;
  // ping-pong so that the last iteration lands in `out`
  const __nv_bfloat16* cur = x_in;
  for (int it = 0; it < steps; ++it) {
    __nv_bfloat16* nxt = ((steps - 1 - it) % 2 == 0) ? out : xb;
    const float* sc_a = it == 0 ? scal : nullptr;
    const float* sc_x = it == 0 ? scal + 2 : nullptr;
    int rc;
    // A = X X^T  [r, r]
    // (symmetric: only the tiles on and above the diagonal are computed)
    if (tall) rc = launch_ns_gemm(cur, true, C, cur, true, C, (int)r, (int)r, (int)k, 1.0f, 0.0f, sc_a, nullptr, 0, Am, r, status, stream, launches, true);
    else      rc = launch_ns_gemm(cur, false, C, cur, false, C, (int)r, (int)r, (int)k, 1.0f, 0.0f, sc_a, nullptr, 0, Am, r, status, stream, launches, true);
    if (rc) return rc;
    // B = b A + c A A   (A symmetric: A A = A A^T, both operands K-major)
    rc = launch_ns_gemm(Am, false, r, Am, false, r, (int)r, (int)r, (int)r, c, b, nullptr, Am, r, Bm, r, status, stream, launches, true);
    if (rc) return rc;
    // X <- a X + B X
    if (tall)  // X^T <- a X^T + X^T B : out[kk, j] = sum_i X^T[kk, i] B[j, i]
      rc = launch_ns_gemm(cur, false, C, Bm, false, r, (int)k, (int)r, (int)r, 1.0f, a, sc_x, cur, C, nxt, C, status, stream, launches);
    else       // out[i, j] = sum_l B[i, l] X[l, j] : second operand MN-major
      rc = launch_ns_gemm(Bm, false, r, cur, true, C, (int)r, (int)k, (int)r, 1.0f, a, sc_x, cur, C, nxt, C, status, stream, launches);
    if (rc) return rc;
    cur = nxt;
  }
  return KAON_OK;
}

}  // namespace kaon

using namespace kaon;

extern "C" int64_t kaon_newton_schulz_workspace_bytes(int64_t rows, int64_t cols) {
  return (int64_t)ns_workspace_bytes(rows, cols) + 256;
}

extern "C" int kaon_newton_schulz(const void* x_bf16, int64_t rows, int64_t cols, int steps, void* out_bf16,
                                  void* workspace, int64_t workspace_bytes, void* stream) {
  if (!x_bf16 || !out_bf16 || !workspace || rows <= 0 || cols <= 0 || steps < 1) return fail(KAON_E_INVALID, "kaon_newton_schulz: bad argument");
  if (x_bf16 == out_bf16) return fail(KAON_E_INVALID, "kaon_newton_schulz: output may not alias the input");
  if (workspace_bytes < kaon_newton_schulz_workspace_bytes(rows, cols)) return fail(KAON_E_INVALID, "kaon_newton_schulz: workspace too small");
  if (rows >= (1ll << 31) || cols >= (1ll << 31)) return fail(KAON_E_UNSUPPORTED, "matrix too large");
  // the first 4 bytes of the workspace are the status word of this call
  unsigned* status = reinterpret_cast<unsigned*>(workspace);
  KAON_CUDA(cudaMemsetAsync(status, 0, 4, (cudaStream_t)stream));
  return ns_run(reinterpret_cast<const __nv_bfloat16*>(x_bf16), rows, cols, steps,
                reinterpret_cast<__nv_bfloat16*>(out_bf16), reinterpret_cast<unsigned char*>(workspace) + 256,
                status, (cudaStream_t)stream, nullptr);
}
