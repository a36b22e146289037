// Standalone momentum codec and weight-write kernels (off the step's hot path: state tooling,
// CodecBuffer-style reads, tests of the primitives in isolation).
#include "kaon_host.h"
#include "kaon_ops.cuh"

namespace kaon {

// ---- int8: one CTA per row (or one CTA for a 1-D tensor): absmax, then encode ----
__global__ void encode_int8_kernel(const float* __restrict__ m, long long C, signed char* codes,
                                   float* scale) {
  __shared__ float red[32];
  const long long r = blockIdx.x;
  const float* row = m + r * C;
  float a = 0.0f;
  for (long long i = threadIdx.x; i < C; i += blockDim.x) a = fmaxf(a, fabsf(row[i]));
  a = group_max(a, 32);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = a;
  __syncthreads();
  a = 0.0f;
  for (int w = 0; w < (int)(blockDim.x >> 5); ++w) a = fmaxf(a, red[w]);
  const float sc = __fdiv_rn(fmaxf(a, 1e-12f), 127.0f);
  if (threadIdx.x == 0) scale[r] = sc;
  for (long long i = threadIdx.x; i < C; i += blockDim.x) {
    float q = rintf(__fdiv_rn(row[i], sc));
    q = fminf(fmaxf(q, -127.0f), 127.0f);
    codes[r * C + i] = (signed char)(int)q;
  }
}

__global__ void decode_int8_kernel(const signed char* __restrict__ codes, const float* __restrict__ scale,
                                   long long n, long long C, float* m) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    m[i] = __fmul_rn((float)codes[i], scale[i / C]);
}

// ---- 4-bit: scales per block first, then one thread per output byte (two nibbles) ----
__global__ void scale_4bit_kernel(const float* __restrict__ m, long long n, long long block,
                                  long long nblocks, float* scale) {
  const long long b = blockIdx.x * (long long)(blockDim.x >> 5) + (threadIdx.x >> 5);
  if (b >= nblocks) return;
  const int lane = threadIdx.x & 31;
  const long long e0 = b * block, e1 = min(e0 + block, n);
  float a = 0.0f;
  for (long long i = e0 + lane; i < e1; i += 32) a = fmaxf(a, fabsf(m[i]));
  a = group_max(a, 32);
  if (lane == 0) scale[b] = __fdiv_rn(fmaxf(a, 1e-12f), 7.0f);
}

__device__ __forceinline__ unsigned nibble_of(float x, float sc) {
  float q = rintf(__fdiv_rn(x, sc));
  q = fminf(fmaxf(q, -7.0f), 7.0f);
  return (unsigned)((int)q + 8);
}

__global__ void pack_4bit_kernel(const float* __restrict__ m, const float* __restrict__ scale,
                                 long long n, long long block, unsigned char* packed) {
  const long long nbytes = (n + 1) / 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < nbytes;
       i += (long long)gridDim.x * blockDim.x) {
    const long long e = 2 * i;
    unsigned lo = nibble_of(m[e], scale[e / block]);
    unsigned hi = (e + 1 < n) ? nibble_of(m[e + 1], scale[(e + 1) / block]) : 0u;
    packed[i] = (unsigned char)(lo | (hi << 4));
  }
}

__global__ void decode_4bit_kernel(const unsigned char* __restrict__ packed, const float* __restrict__ scale,
                                   long long n, long long block, float* m) {
  for (long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x; e < n;
       e += (long long)gridDim.x * blockDim.x) {
    const unsigned byte = packed[e >> 1];
    const int nib = (e & 1) ? (byte >> 4) & 0xF : byte & 0xF;
    m[e] = __fmul_rn((float)(nib - 8), scale[e / block]);
  }
}

// ---- p += alpha * delta with the configured bf16 rounding ----
template <typename PT>
__global__ void sr_add_kernel(void* p, const float* __restrict__ delta, long long n, float alpha,
                              int sr, SrStream st, uint32_t tensor_id) {
  const long long nvec = (n + 7) >> 3;
  for (long long v = blockIdx.x * (long long)blockDim.x + threadIdx.x; v < nvec;
       v += (long long)gridDim.x * blockDim.x) {
    const int cnt = (int)min(8ll, n - v * 8);
    float d[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) d[k] = (k < cnt) ? delta[v * 8 + k] : 0.0f;
    update8<PT>(reinterpret_cast<unsigned char*>(p) + v * 8 * Elems<PT>::BYTES, cnt, d, alpha, sr != 0,
                st, tensor_id, (uint64_t)v, nullptr);
  }
}

static int grid_for(long long work, int threads) {
  long long g = (work + threads - 1) / threads;
  return (int)std::max<long long>(1, std::min<long long>(g, 148 * 16));
}

}  // namespace kaon

using namespace kaon;

extern "C" {

int kaon_codec_encode_int8(const float* m, int64_t numel, int64_t rows, int8_t* codes, float* scale,
                           void* stream) {
  if (!m || !codes || !scale || numel < 0) return fail(KAON_E_INVALID, "kaon_codec_encode_int8: bad argument");
  if (numel == 0) return KAON_OK;
  const long long R = rows > 0 ? rows : 1;
  if (numel % R) return fail(KAON_E_INVALID, "numel not divisible by rows");
  if (R > 0x7fffffffll) return fail(KAON_E_UNSUPPORTED, "too many rows");
  encode_int8_kernel<<<(unsigned)R, 256, 0, (cudaStream_t)stream>>>(m, numel / R, (signed char*)codes, scale);
  KAON_CUDA(cudaGetLastError());
  return KAON_OK;
}

int kaon_codec_decode_int8(const int8_t* codes, const float* scale, int64_t numel, int64_t rows,
                           float* m, void* stream) {
  if (!m || !codes || !scale || numel < 0) return fail(KAON_E_INVALID, "kaon_codec_decode_int8: bad argument");
  if (numel == 0) return KAON_OK;
  const long long R = rows > 0 ? rows : 1;
  decode_int8_kernel<<<grid_for(numel, 256), 256, 0, (cudaStream_t)stream>>>((const signed char*)codes, scale, numel, numel / R, m);
  KAON_CUDA(cudaGetLastError());
  return KAON_OK;
}

int kaon_codec_encode_4bit(const float* m, int64_t numel, int64_t block, uint8_t* packed,
                           float* scale, void* stream) {
  if (!m || !packed || !scale || numel < 0 || block <= 0) return fail(KAON_E_INVALID, "kaon_codec_encode_4bit: bad argument");
  if (numel == 0) return KAON_OK;
  const long long nb = (numel + block - 1) / block;
  scale_4bit_kernel<<<(unsigned)((nb + 7) / 8), 256, 0, (cudaStream_t)stream>>>(m, numel, block, nb, scale);
  pack_4bit_kernel<<<grid_for((numel + 1) / 2, 256), 256, 0, (cudaStream_t)stream>>>(m, scale, numel, block, packed);
  KAON_CUDA(cudaGetLastError());
  return KAON_OK;
}

int kaon_codec_decode_4bit(const uint8_t* packed, const float* scale, int64_t numel, int64_t block,
                           float* m, void* stream) {
  if (!m || !packed || !scale || numel < 0 || block <= 0) return fail(KAON_E_INVALID, "kaon_codec_decode_4bit: bad argument");
  if (numel == 0) return KAON_OK;
  decode_4bit_kernel<<<grid_for(numel, 256), 256, 0, (cudaStream_t)stream>>>(packed, scale, numel, block, m);
  KAON_CUDA(cudaGetLastError());
  return KAON_OK;
}

int kaon_sr_add(void* p, int param_dtype, const float* delta, int64_t numel, float alpha,
                int bf16_method, uint64_t seed, uint32_t step, uint32_t tensor_id, uint32_t tag,
                void* stream) {
  if (!p || !delta || numel < 0) return fail(KAON_E_INVALID, "kaon_sr_add: bad argument");
  if (((uintptr_t)p) & 15) return fail(KAON_E_INVALID, "kaon_sr_add: weights not 16-byte aligned");
  if (numel == 0) return KAON_OK;
  SrStream st{Philox{(uint32_t)seed, (uint32_t)(seed >> 32)}, step, tag};
  const int g = grid_for((numel + 7) / 8, 256);
  if (param_dtype == KAON_DT_BF16)
    sr_add_kernel<__nv_bfloat16><<<g, 256, 0, (cudaStream_t)stream>>>(p, delta, numel, alpha, bf16_method == KAON_W_SR, st, tensor_id);
  else if (param_dtype == KAON_DT_F32)
    sr_add_kernel<float><<<g, 256, 0, (cudaStream_t)stream>>>(p, delta, numel, alpha, 0, st, tensor_id);
  else
    return fail(KAON_E_INVALID, "param_dtype %d", param_dtype);
  KAON_CUDA(cudaGetLastError());
  return KAON_OK;
}

}  // extern "C"
