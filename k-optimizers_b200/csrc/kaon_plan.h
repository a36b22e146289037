// Internal layout of a plan: the device-side descriptor table, the work list and the scratch.
// Shared by the host planner (plan.cu) and the kernels.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <vector>

#include "../../include/kaon_b200.h"

namespace kaon {

// Elements one work item stages in shared memory at most.  A work item of a >=2-D tensor is a run of
// whole rows, so the widest row a plan accepts is CAP elements.
constexpr int CAP = 16384;
constexpr int MAX_TASK_ROWS = 2048;  // rows per work item (bounds the shared row-mean array)
constexpr int NTHREADS = 256;

// Work-item kinds.  Lion: MAIN does everything up to the momentum store and records, per element,
// a 2-bit code (sign of the update / masked out); APPLY turns the codes into the weight write once
// the tensor's kept count is complete.
enum : int { PH_LION_MAIN = 0, PH_LION_APPLY = 1, PH_AXPY = 2,
              // Adakaon / AdaMuon (factored tensors): STATS = row statistics + column partial sums over a
              // run of rows; FINAL = column statistics, clip divisor (one item per column strip);
              // COUNT = cautious kept count; APPLY = momentum store + weight write.  FLAT = a whole 1-D
              // tensor in one item.
              PH_ADA_STATS = 10, PH_ADA_FINAL = 11, PH_ADA_COUNT = 12, PH_ADA_APPLY = 13, PH_ADA_FLAT = 14 };

constexpr int ADA_THREADS = 512;
constexpr int FINAL_STRIP = 2048;  // columns per FINAL item

// One tensor as the kernels see it (device copy of kaon_tensor_desc plus planner-derived fields).
struct DevTensor {
  void* p;
  void* m;
  float* m_scale;
  float* stat_a;
  float* stat_b;
  long long numel;
  long long code_off;   // byte offset of this tensor's 2-bit codes in the code scratch (16-aligned)
  int rows;             // shape[0] for ndim >= 2, else 0
  int cols;             // numel / rows, or numel for 1-D
  unsigned row_magic;   // ceil(2^32 / cols): floor(i / cols) == umulhi(i, row_magic) for i*cols < 2^32
  unsigned tensor_id;
  unsigned block;       // 4-bit block size in use
  int bshift;           // 4-bit: log2(block) for a power-of-two block of 32..256 elements; 31 when one block
                        // covers the whole tensor
  int n_main;           // number of MAIN work items of this tensor (what `done` must reach)
  // Adakaon / AdaMuon only
  int chunk_rows;       // rows staged at a time (chunk_rows * cols <= CAP, aligned); -1: a Lion tensor cut into
                        // flat runs instead of whole rows (its row means are in `aux` at aux_off)
  int n_stats;          // STATS items (= slots of column partials)
  int n_strips;         // FINAL items
  int n_count;          // COUNT items
  long long aux_off;    // float index of this tensor's scratch in `aux`:
                        //   colpart[n_stats][2][cols] | cfac[cols] | rowpart[n_stats] (double) |
                        //   tpart[n_strips] (double) | scal[4] = {rowmean, divisor, rms, -} | rowmax[rows] | mean[rows]
  void* shift;          // Kahan compensation buffer (bf16 [numel]) or null
};

// 4-bit block geometry: the block an element belongs to, and how many threads (eight elements each) share one
__host__ __device__ inline long long blk_of(const DevTensor& d, long long i) { return d.bshift >= 31 ? 0 : (i >> d.bshift); }
__host__ __device__ inline int blk_lanes(const DevTensor& d) { return d.bshift >= 31 ? 16 : (1 << (d.bshift - 3)); }

// float offsets inside a tensor's aux block
__host__ __device__ inline long long aux_cfac(const DevTensor& d) { return d.aux_off + 2ll * d.n_stats * d.cols; }
__host__ __device__ inline long long aux_rowpart(const DevTensor& d) { return (aux_cfac(d) + d.cols + 1) / 2 * 2; }
__host__ __device__ inline long long aux_tpart(const DevTensor& d) { return aux_rowpart(d) + 2ll * d.n_stats; }
__host__ __device__ inline long long aux_scal(const DevTensor& d) { return aux_tpart(d) + 2ll * d.n_strips; }
// int8 momentum: bits of each row's absmax of the new momentum, left by COUNT for APPLY
__host__ __device__ inline long long aux_rowmax(const DevTensor& d) { return aux_scal(d) + 4; }
// centralization mean of every row, left by STATS for COUNT / APPLY
__host__ __device__ inline long long aux_mean(const DevTensor& d) { return aux_rowmax(d) + d.rows; }
// int8 momentum: the row scales as they were before this step, copied by an APPLY item for its rows
__host__ __device__ inline long long aux_oldsc(const DevTensor& d) { return aux_mean(d) + d.rows; }
// r_i = rsqrt(row_i / mean(row)) of every row, left by the last FINAL strip for COUNT / APPLY
__host__ __device__ inline long long aux_rfac(const DevTensor& d) { return aux_oldsc(d) + d.rows; }
// scratch of a 1-D tensor stepped from global memory: 8 floats | n floats (padded) | one word per 4-bit block (>= 32 elements)
__host__ __device__ inline long long flat_long_pad(long long n) { return (n + 63) / 64 * 64; }
__host__ __device__ inline long long flat_long_size(long long n) { return 8 + flat_long_pad(n) + ((n + 31) / 32 + 1 + 63) / 64 * 64; }
__host__ __device__ inline long long aux_size(const DevTensor& d) { return aux_rfac(d) + d.rows - d.aux_off; }

struct Task {
  int tensor;
  int phase;
  long long e0;  // first element (flat index); multiple of the plan's alignment unit and a row start
  int n;         // elements (<= CAP); whole rows for >=2-D tensors
  int row0;      // first row (>=2-D tensors); FINAL items: first column of the strip
  int slot;      // STATS items: index of the column-partial slot; otherwise 0
  int pad;       // Lion items of a tensor cut into flat runs: column of the first element (e0 - row0 * cols)
};

// Mirrors of the weight buffer on other GPUs (ZeRO-1 publish fused into the step): every weight the
// kernels write at address a is also stored at a + delta[r], r < n.  delta[r] is the byte distance from
// this rank's weight buffer to the mapping of rank r's copy (peer memory, plain stores; multiples of 16).
struct Peers {
  int n;
  int pad;
  long long delta[KAON_MAX_PEERS];
};

// Device pointers handed to the kernels by value.
struct PlanView {
  const DevTensor* tensors;
  const void* const* grads;  // [n_tensors], refreshed by kaon_plan_set_grads
  const Task* tasks;
  int n_tasks;
  int n_tensors;
  unsigned* task_counter;  // claims
  unsigned* done;          // Lion: [n_tensors] MAIN items finished.  Adakaon: [4][n_tensors] =
                           //   STATS items done | FINAL strips arrived | FINAL complete | COUNT items done
  unsigned* kept;          // [n_tensors] cautious kept count
  float* aux;              // Adakaon scratch (see DevTensor::aux_off)
  const void* const* signal;  // AdaMuon: per-tensor orthogonalised momentum (bf16); null otherwise
  unsigned* status;        // 0 = ok; else the code of the first bounded wait that ran out
  unsigned char* codes;    // 2 bits per element
  Peers peers;             // n == 0: no mirrors
  unsigned spin_limit;     // polls a completion-counter wait makes before it gives up (0: the default)
  unsigned sm_reserve;     // multiprocessors (the highest ids) whose CTAs leave at once, so that a collective's
                           // CTAs find them empty beside the persistent step (0: none)
};

}  // namespace kaon

// Host-side plan object behind the opaque handle.
struct kaon_plan {
  int device = 0;
  int optimizer = 0, param_dtype = 0, momentum_kind = 0;
  int n_tensors = 0;
  int n_tasks_full = 0;   // MAIN + APPLY items interleaved
  int n_tasks_main = 0;   // MAIN items only (cautious off)
  int n_tasks_axpy = 0;
  kaon::PlanView view{};
  kaon::Task* d_tasks_full = nullptr;
  kaon::Task* d_tasks_main = nullptr;
  kaon::Task* d_tasks_axpy = nullptr;
  void* d_block = nullptr;      // one allocation holding tables and counters
  unsigned char* d_codes = nullptr;
  float* d_aux = nullptr;
  kaon::Task* d_tasks_nocount = nullptr;  // Adakaon work list without the COUNT items (cautious off)
  int n_tasks_nocount = 0;
  int threads = 0;
  bool double_buffer = false;  // Adakaon/AdaMuon: shared memory holds two staging buffer sets
  std::vector<kaon::DevTensor> h_tensors;   // host copy of the table
  std::vector<const void*> h_grads;         // host copy of the gradient-pointer column
  // AdaMuon only (built lazily by the first step)
  kaon::Task* d_tasks_ema = nullptr;         // row-chunk items of the factored tensors, tensor by tensor
  std::vector<int> ema_begin;                // [n_tensors + 1] ranges into d_tasks_ema
  const void** d_signal = nullptr;           // per-tensor pointer to O in the caller's workspace
  const void* signal_base = nullptr;         // workspace the pointers were computed for
  bool muon_lanes_ready = false;             // internal streams of the per-matrix Newton-Schulz chains
  cudaStream_t muon_stream[4] = {nullptr, nullptr, nullptr, nullptr};
  cudaEvent_t muon_join[4] = {nullptr, nullptr, nullptr, nullptr};
  cudaEvent_t muon_fork = nullptr;
  // Adakaon / AdaMuon (built lazily by the first step): COUNT and APPLY as launches of their own
  bool has_long_rows = false;                // a factored tensor's rows exceed a work item: streaming launches only
  int apply2 = 0;                            // 0 = not decided, 1 = in use, -1 = this plan is not eligible
  kaon::Task* d_tasks_apply2 = nullptr;      // flat items of the factored tensors
  int n_tasks_apply2 = 0;
  // the persistent kernel's lists beside those launches: [0] without COUNT items, [1] with them
  kaon::Task* d_tasks_na[2] = {nullptr, nullptr};
  int n_tasks_na[2] = {0, 0};
  bool long_rows_ok = false;                 // every tensor whose rows exceed a work item left the persistent kernel
  // STATS as a launch of its own: the STATS items that qualify
  kaon::Task* d_tasks_stats = nullptr;
  int n_tasks_stats = 0, stats_grid = 0;
  unsigned* d_counter2 = nullptr;            // claim counter of the COUNT / APPLY launches
  int apply_grid = 0;
  size_t apply_smem = 0;
  unsigned* d_counters = nullptr;  // task_counter, status, done[n], kept[n] (contiguous; memset per step)
  size_t counters_bytes = 0;
  int64_t device_bytes = 0;
  int64_t launches = 0;
  int grid = 0;          // persistent grid size
  int sm_count = 0;      // multiprocessors of the plan's device
  int* d_flat_tensors = nullptr;  // Lion: indices of the tensors cut into flat runs (row means by a pre-pass)
  int n_flat_tensors = 0;
  size_t smem_bytes = 0;
  int64_t total_elems = 0;
  // AdaPNM only: lists, partial sums and the second-momentum table (adapnm.cu), built by kaon_adapnm_attach
  void* pnm = nullptr;
  bool pnm_has_max_v = false;
  // KProdigy only: item lists, partial sums and the s / p0 table (kprodigy.cu), built by kaon_kprodigy_attach
  void* kp = nullptr;
};

namespace kaon {
void pnm_free(kaon_plan* pl);
void kp_free(kaon_plan* pl);
}
