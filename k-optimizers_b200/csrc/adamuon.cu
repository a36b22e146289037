// AdaMuon step for sm_100a (reference src/kaon/adamuon.py:327-352, 434-615).
//
// Per >=2-D tensor:  (1) EMA pre-pass: m <- lerp(decode(m), g, 1-b1) with g optionally centralised (each
// row less its mean, adamuon.py:334-335), re-encode and store m, write the fp32 pre-requant momentum as
// bf16 into the workspace;  (2) Newton-Schulz of that matrix on the tensor
// cores (ns.cu);  (3) the Adakaon STATS/FINAL/COUNT/APPLY work items with the orthogonalised matrix O as
// the signal, no further momentum, scale 0.2*lr, and the cautious mask taken against the raw gradient.
// 1-D tensors run the FLAT work item (Adam-style, momentum of the update) inside step (3)'s kernel.
#include <algorithm>

#include "adakaon_dev.h"
#include "kaon_host.h"
#include "kaon_ops.cuh"

namespace kaon {

int ns_run(const __nv_bfloat16* x_in, long long R, long long C, int steps, __nv_bfloat16* out, void* ws,
           unsigned* status, cudaStream_t stream, long long* launches);
size_t ns_workspace_bytes(long long R, long long C);

constexpr int ET = 256;

// Row-chunk items [t0, t1) of ONE tensor: gradient and momentum straight from global memory.
template <typename PT, int MK>
__global__ void __launch_bounds__(ET) muon_ema_kernel(PlanView pv, const Task* tasks, int t0, int t1,
                                                      float w1, float w1m1, int small_w1, int gc,
                                                      __nv_bfloat16* x_out) {
  using E = Elems<PT>;
  __shared__ unsigned rowmax_s[MAX_TASK_ROWS];
  __shared__ float scale_s[MAX_TASK_ROWS];
  __shared__ float mean_s[MAX_TASK_ROWS];  // centralization mean of each row of the item
  const int tid = threadIdx.x;
  for (int ti = t0 + blockIdx.x; ti < t1; ti += gridDim.x) {
    const Task t = tasks[ti];
    const DevTensor d = pv.tensors[t.tensor];
    const unsigned char* g = reinterpret_cast<const unsigned char*>(pv.grads[t.tensor]) + t.e0 * E::BYTES;
    const int n = t.n, C = d.cols;
    const int nrows = n / C;
    const int nvec = (n + 7) >> 3, nvec_pad = (nvec + 31) & ~31;
    const bool row_uniform = (C & 7) == 0;
    const unsigned char* mbase = reinterpret_cast<const unsigned char*>(d.m);
    if (gc) {
      // one warp per row; the mean also goes to the scratch, where the cautious mask of the weight stage
      // finds it (the mask compares with the centralised gradient)
      for (int r = tid >> 5; r < nrows; r += ET / 32) {
        const unsigned char* rowp = g + (size_t)r * C * E::BYTES;
        float sum = 0.0f;
        if (row_uniform) {
          for (int v = tid & 31; v < (C >> 3); v += 32) {
            float x[8];
            E::load8(rowp + (size_t)v * 8 * E::BYTES, x);
            sum += ((x[0] + x[1]) + (x[2] + x[3])) + ((x[4] + x[5]) + (x[6] + x[7]));
          }
        } else {
          for (int i = tid & 31; i < C; i += 32) sum += E::load1(rowp, i);
        }
        sum = warp_sum(sum);
        const float mean = __fdiv_rn(sum, (float)C);
        const float mu = E::IS_BF16 ? round_bf16(mean) : mean;
        if ((tid & 31) == 0) { mean_s[r] = mu; pv.aux[aux_mean(d) + t.row0 + r] = mu; }
      }
      __syncthreads();
    }
    auto m_new8 = [&](int v, int cnt, float mn[8]) {
      float gv[8], mo[8];
      load8_guard<PT>(g + (size_t)v * 8 * E::BYTES, cnt, gv);
      if (gc) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const float x = __fsub_rn(gv[k], mean_s[row_uniform ? row_of((unsigned)v * 8u, d) : row_of((unsigned)(v * 8 + min(k, max(cnt - 1, 0))), d)]);
          gv[k] = E::IS_BF16 ? round_bf16(x) : x;
        }
      }
      if constexpr (MK == KAON_M_4BIT) {
        const long long blk = blk_of(d, t.e0 + (long long)v * 8);
        decode8<MK>(mbase + (t.e0 >> 1), v, cnt, d.m_scale[blk], mo);
      } else if constexpr (MK == KAON_M_INT8) {
#pragma unroll
        for (int k = 0; k < 8; ++k)
          mo[k] = (k < cnt) ? __fmul_rn((float)(signed char)mbase[t.e0 + v * 8 + k],
                                        scale_s[row_uniform ? row_of((unsigned)v * 8u, d) : row_of((unsigned)(v * 8 + k), d)])
                            : 0.0f;
      } else if constexpr (MK == KAON_M_BF16) {
        decode8<MK>(mbase + t.e0 * 2, v, cnt, 1.0f, mo);
      } else if constexpr (MK == KAON_M_F32) {
        decode8<MK>(mbase + t.e0 * 4, v, cnt, 1.0f, mo);
      }
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        float r;
        if constexpr (MK == KAON_M_NONE) r = gv[k];
        else if constexpr (MK == KAON_M_BF16) r = round_bf16(lerp_torch(mo[k], round_bf16(gv[k]), w1, w1m1, small_w1 != 0));
        else r = lerp_torch(mo[k], gv[k], w1, w1m1, small_w1 != 0);
        mn[k] = (k < cnt) ? r : 0.0f;
      }
    };
    if constexpr (MK == KAON_M_INT8) {
      for (int r = tid; r < nrows; r += ET) { rowmax_s[r] = 0u; scale_s[r] = d.m_scale[t.row0 + r]; }
      __syncthreads();
      for (int v = tid; v < nvec; v += ET) {
        const int cnt = min(8, n - v * 8);
        float mn[8];
        m_new8(v, cnt, mn);
        if (row_uniform) {
          float a = 0.0f;
#pragma unroll
          for (int k = 0; k < 8; ++k) a = fmaxf(a, fabsf(mn[k]));
          atomicMax(rowmax_s + row_of((unsigned)v * 8u, d), __float_as_uint(a));
        } else {
          for (int k = 0; k < cnt; ++k) atomicMax(rowmax_s + row_of((unsigned)(v * 8 + k), d), __float_as_uint(fabsf(mn[k])));
        }
      }
      __syncthreads();
    }
    for (int v = tid; v < nvec_pad; v += ET) {
      const int cnt = max(0, min(8, n - v * 8));
      float mn[8];
      if (cnt > 0) m_new8(v, cnt, mn);
      else {
#pragma unroll
        for (int k = 0; k < 8; ++k) mn[k] = 0.0f;
      }
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
          const int qi = min(max((int)quant_round(mn[k], sc, inv, 1e-4f), -7), 7);
          if (k < cnt) word |= (uint32_t)(qi + 8) << (4 * k);
        }
        if (cnt > 0) {
          unsigned char* mdst = (unsigned char*)d.m + (t.e0 >> 1) + (size_t)v * 4;
          if (cnt == 8) *reinterpret_cast<uint32_t*>(mdst) = word;
          else
            for (int b = 0; b < (cnt + 1) / 2; ++b) mdst[b] = (unsigned char)(word >> (8 * b));
          if ((v & (blk_lanes(d) - 1)) == 0) d.m_scale[blk_of(d, t.e0 + (long long)v * 8)] = sc;
        }
      } else if constexpr (MK == KAON_M_INT8) {
        if (cnt > 0) {
          unsigned char* mdst = (unsigned char*)d.m + t.e0 + (size_t)v * 8;
          float sc = 0.0f, inv = 0.0f;
          int rprev = -1;
          for (int k = 0; k < cnt; ++k) {
            const int r = row_uniform ? row_of((unsigned)v * 8u, d) : row_of((unsigned)(v * 8 + k), d);
            if (r != rprev) {
              sc = __fdiv_rn(fmaxf(__uint_as_float(rowmax_s[r]), 1e-12f), 127.0f);
              inv = __fdividef(1.0f, sc);
              rprev = r;
              if ((unsigned)(v * 8 + k) == (unsigned)r * (unsigned)C) d.m_scale[t.row0 + r] = sc;
            }
            mdst[k] = (unsigned char)(min(max((int)quant_round(mn[k], sc, inv, 1e-3f), -127), 127) & 0xFF);
          }
        }
      } else if constexpr (MK == KAON_M_BF16) {
        if (cnt > 0)
          for (int k = 0; k < cnt; ++k)
            reinterpret_cast<uint16_t*>((unsigned char*)d.m + t.e0 * 2)[v * 8 + k] = (uint16_t)(__float_as_uint(mn[k]) >> 16);
      } else if constexpr (MK == KAON_M_F32) {
        if (cnt > 0)
          for (int k = 0; k < cnt; ++k) reinterpret_cast<float*>((unsigned char*)d.m + t.e0 * 4)[v * 8 + k] = mn[k];
      }
      // the matrix Newton-Schulz reads: bf16 of the fp32 pre-requant momentum
      if (cnt > 0) {
        __nv_bfloat16* xo = x_out + t.e0 + (size_t)v * 8;
        if (cnt == 8 && (reinterpret_cast<uintptr_t>(xo) & 15) == 0) {
          *reinterpret_cast<uint4*>(xo) = make_uint4(pack_bf16_rn(mn[0], mn[1]), pack_bf16_rn(mn[2], mn[3]),
                                                    pack_bf16_rn(mn[4], mn[5]), pack_bf16_rn(mn[6], mn[7]));
        } else {
          for (int k = 0; k < cnt; ++k) xo[k] = __float2bfloat16_rn(mn[k]);
        }
      }
    }
    __syncthreads();
  }
}

typedef void (*EmaKernel)(PlanView, const Task*, int, int, float, float, int, int, __nv_bfloat16*);

template <typename PT>
static EmaKernel pick_ema_pt(int mk) {
  switch (mk) {
    case KAON_M_F32: return muon_ema_kernel<PT, KAON_M_F32>;
    case KAON_M_BF16: return muon_ema_kernel<PT, KAON_M_BF16>;
    case KAON_M_INT8: return muon_ema_kernel<PT, KAON_M_INT8>;
    case KAON_M_4BIT: return muon_ema_kernel<PT, KAON_M_4BIT>;
    case KAON_M_NONE: return muon_ema_kernel<PT, KAON_M_NONE>;
    default: return nullptr;
  }
}

static size_t up256(size_t x) { return (x + 255) / 256 * 256; }

// Matrices are independent of each other until the second-moment stage, so their EMA pre-pass and
// Newton-Schulz chains run round robin on NS_LANES internal streams, each with a staging matrix and a
// Newton-Schulz scratch of its own: when the last tiles of one matrix's GEMM leave most SMs idle, the next
// matrix's kernels start on them.
constexpr int NS_LANES = 3;

struct MuonLayout {
  std::vector<size_t> o_off;  // per tensor: byte offset of O in the workspace (factored tensors)
  size_t x0_off = 0, ns_off = 0, lane_stride = 0, total = 0;  // lane l: x0_off + l * lane_stride, ns_off + l * lane_stride
};

static MuonLayout muon_layout(const kaon_plan* pl) {
  MuonLayout L;
  L.o_off.assign(pl->n_tensors, 0);
  size_t cur = 0, max_x = 0, max_ns = 0;
  for (int i = 0; i < pl->n_tensors; ++i) {
    const DevTensor& t = pl->h_tensors[i];
    if (t.rows <= 0 || t.numel == 0) continue;
    L.o_off[i] = cur;
    cur += up256((size_t)t.numel * 2);
    max_x = std::max(max_x, up256((size_t)t.numel * 2));
    max_ns = std::max(max_ns, up256(ns_workspace_bytes(t.rows, t.cols)));
  }
  L.x0_off = cur;
  L.ns_off = cur + max_x;
  L.lane_stride = max_x + max_ns;
  cur += (size_t)NS_LANES * L.lane_stride;
  L.total = cur + 256;
  return L;
}

}  // namespace kaon

using namespace kaon;

extern "C" int64_t kaon_adamuon_workspace_bytes(const kaon_plan* pl) {
  if (!pl || pl->optimizer != KAON_OPT_ADAMUON) return 0;
  return (int64_t)muon_layout(pl).total;
}

extern "C" int64_t kaon_adamuon_signal_offset(const kaon_plan* pl, int tensor) {
  if (!pl || pl->optimizer != KAON_OPT_ADAMUON || tensor < 0 || tensor >= pl->n_tensors) return -1;
  if (pl->h_tensors[tensor].rows <= 0) return -1;
  return (int64_t)muon_layout(pl).o_off[tensor];
}

extern "C" int kaon_adamuon_step(kaon_plan* pl, const kaon_adamuon_hparams* h, void* workspace,
                                 int64_t workspace_bytes, uint64_t seed, uint32_t step, void* stream) {
  if (!pl || !h) return fail(KAON_E_INVALID, "kaon_adamuon_step: null argument");
  if (pl->optimizer != KAON_OPT_ADAMUON) return fail(KAON_E_INVALID, "plan was not built for AdaMuon");
  if (int rc = check_device(pl)) return rc;
  if (h->bf16_method < KAON_W_NONE || h->bf16_method > KAON_W_KAHAN) return fail(KAON_E_UNSUPPORTED, "bf16_method %d", h->bf16_method);
  if (int rc = check_kahan(pl, h->bf16_method)) return rc;
  if (!(h->clip_threshold > 0.0)) return fail(KAON_E_INVALID, "clip_threshold must be > 0");
  if (h->ns_steps < 1) return fail(KAON_E_INVALID, "ns_steps must be >= 1");
  const bool has_m = pl->momentum_kind != KAON_M_NONE;
  if (has_m != (h->beta1 > 0.0)) return fail(KAON_E_INVALID, "beta1 %g does not match the plan's momentum kind", h->beta1);
  const MuonLayout L = muon_layout(pl);
  if (!workspace || ((uintptr_t)workspace & 255) || workspace_bytes < (int64_t)L.total)
    return fail(KAON_E_INVALID, "kaon_adamuon_step: workspace missing, misaligned or smaller than %zu bytes", L.total);
  cudaStream_t s = (cudaStream_t)stream;
  unsigned char* ws = reinterpret_cast<unsigned char*>(workspace);
  const int n = pl->n_tensors;

  // one-time: row-chunk work list of the factored tensors; per-workspace: the O pointers
  if (!pl->d_tasks_ema) {
    std::vector<Task> list;
    pl->ema_begin.assign(n + 1, 0);
    for (int i = 0; i < n; ++i) {
      pl->ema_begin[i] = (int)list.size();
      const DevTensor& t = pl->h_tensors[i];
      if (t.rows <= 0 || t.numel == 0) continue;
      for (long long r = 0; r < t.rows; r += t.chunk_rows) {
        const long long nr = std::min<long long>(t.chunk_rows, t.rows - r);
        list.push_back(Task{i, 0, r * t.cols, (int)(nr * t.cols), (int)r, 0, 0});
      }
    }
    pl->ema_begin[n] = (int)list.size();
    KAON_CUDA(cudaMalloc((void**)&pl->d_tasks_ema, sizeof(Task) * std::max<size_t>(list.size(), 1)));
    KAON_CUDA(cudaMemcpy(pl->d_tasks_ema, list.data(), sizeof(Task) * list.size(), cudaMemcpyHostToDevice));
    KAON_CUDA(cudaMalloc((void**)&pl->d_signal, sizeof(void*) * (size_t)n));
    pl->device_bytes += (int64_t)(sizeof(Task) * list.size() + sizeof(void*) * n);
  }
  if (pl->signal_base != workspace) {
    std::vector<const void*> sig(n, nullptr);
    for (int i = 0; i < n; ++i)
      if (pl->h_tensors[i].rows > 0 && pl->h_tensors[i].numel) sig[i] = ws + L.o_off[i];
    KAON_CUDA(cudaMemcpyAsync((void*)pl->d_signal, sig.data(), sizeof(void*) * (size_t)n, cudaMemcpyHostToDevice, s));
    pl->signal_base = workspace;
  }

  const float w1 = (float)(1.0 - h->beta1);
  EmaKernel ek = pl->param_dtype == KAON_DT_BF16 ? pick_ema_pt<__nv_bfloat16>(pl->momentum_kind)
                                                 : pick_ema_pt<float>(pl->momentum_kind);
  if (!ek) return fail(KAON_E_INVALID, "no AdaMuon EMA kernel for this dtype combination");
  PlanView v = pl->view;
  v.signal = pl->d_signal;
  KAON_CUDA(cudaMemsetAsync(v.task_counter, 0, pl->counters_bytes - sizeof(unsigned), s));

  // (1) + (2): per factored tensor with a gradient: EMA pre-pass, then Newton-Schulz into its O slot,
  // round robin over the lanes (forked from the caller's stream, joined before stage 3)
  if (!pl->muon_lanes_ready) {
    for (int l = 0; l < NS_LANES; ++l) {
      KAON_CUDA(cudaStreamCreateWithFlags(&pl->muon_stream[l], cudaStreamNonBlocking));
      KAON_CUDA(cudaEventCreateWithFlags(&pl->muon_join[l], cudaEventDisableTiming));
    }
    KAON_CUDA(cudaEventCreateWithFlags(&pl->muon_fork, cudaEventDisableTiming));
    pl->muon_lanes_ready = true;
  }
  KAON_CUDA(cudaEventRecord(pl->muon_fork, s));
  for (int l = 0; l < NS_LANES; ++l) KAON_CUDA(cudaStreamWaitEvent(pl->muon_stream[l], pl->muon_fork, 0));
  int turn = 0;
  for (int i = 0; i < n; ++i) {
    const DevTensor& t = pl->h_tensors[i];
    if (t.rows <= 0 || t.numel == 0 || pl->h_grads[i] == nullptr) continue;
    const int lane = turn++ % NS_LANES;
    cudaStream_t sl = pl->muon_stream[lane];
    __nv_bfloat16* x0 = reinterpret_cast<__nv_bfloat16*>(ws + L.x0_off + (size_t)lane * L.lane_stride);
    const int t0 = pl->ema_begin[i], t1 = pl->ema_begin[i + 1];
    const int grid = std::min(t1 - t0, pl->sm_count * 8);
    ek<<<grid, ET, 0, sl>>>(v, pl->d_tasks_ema, t0, t1, w1, w1 - 1.0f, w1 < 0.5f, h->gradient_centralization != 0, x0);
    KAON_CUDA(cudaGetLastError());
    pl->launches += 1;
    long long nl = 0;
    int rc = ns_run(x0, t.rows, t.cols, h->ns_steps, reinterpret_cast<__nv_bfloat16*>(ws + L.o_off[i]),
                    ws + L.ns_off + (size_t)lane * L.lane_stride, v.status, sl, &nl);
    pl->launches += nl;
    if (rc) return rc;
  }
  for (int l = 0; l < NS_LANES; ++l) {
    KAON_CUDA(cudaEventRecord(pl->muon_join[l], pl->muon_stream[l]));
    KAON_CUDA(cudaStreamWaitEvent(s, pl->muon_join[l], 0));
  }

  // (3) second moment of O, clip, scale, cautious, weight write (and the whole 1-D branch)
  AdaDev hp{};
  hp.w1 = w1; hp.w1m1 = w1 - 1.0f; hp.small_w1 = w1 < 0.5f;
  hp.w2 = (float)(1.0 - h->beta2); hp.w2m1 = hp.w2 - 1.0f; hp.small_w2 = hp.w2 < 0.5f;
  hp.eps1 = (float)h->eps1; hp.has_eps = h->eps1 > 0.0;
  hp.clip = (float)h->clip_threshold;
  hp.lrwd = (float)(h->lr * h->weight_decay); hp.has_wd = h->weight_decay != 0.0;
  hp.upd_scale = (float)(0.2 * h->lr);  // _UPDATE_RMS * lr, product taken in double (adamuon.py:88, 489)
  hp.cautious = h->cautious != 0;
  hp.gc = h->gradient_centralization != 0;  // the statistics of O ignore it; the mask centres the raw gradient
  hp.sr = h->bf16_method == KAON_W_SR && pl->param_dtype == KAON_DT_BF16;
  hp.kahan = h->bf16_method == KAON_W_KAHAN && pl->param_dtype == KAON_DT_BF16;
  hp.has_m = has_m;
  hp.step = step; hp.k0 = (uint32_t)seed; hp.k1 = (uint32_t)(seed >> 32);
  if (int rc = ensure_apply2(pl)) return rc;
  const bool three = pl->apply2 == 1;  // STATS/FINAL/FLAT here, COUNT and APPLY as launches of their own
  if (three) { v.tasks = pl->d_tasks_na[hp.cautious ? 1 : 0]; v.n_tasks = pl->n_tasks_na[hp.cautious ? 1 : 0]; }
  else if (hp.cautious) { v.tasks = pl->d_tasks_full; v.n_tasks = pl->n_tasks_full; }
  else { v.tasks = pl->d_tasks_main; v.n_tasks = pl->n_tasks_main; }
  if (three)
    if (int rc = launch_stats(pl, v, hp, s)) return rc;
  AdaKernel k = pick_ada(pl->param_dtype, pl->momentum_kind, true);
  if (!k) return fail(KAON_E_INVALID, "no AdaMuon kernel for this dtype combination");
  k<<<pl->grid, ADA_THREADS, pl->smem_bytes, s>>>(v, hp, (int)x_offset_rows(pl) | (pl->double_buffer ? 1 : 0));
  KAON_CUDA(cudaGetLastError());
  pl->launches += 1;
  if (three) {
    if (int rc = launch_count_apply(pl, v, hp, s)) return rc;
  }
  return KAON_OK;
}
