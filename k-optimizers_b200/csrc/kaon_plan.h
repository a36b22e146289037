// Internal layout of a plan: the device-side descriptor table, the work list and the scratch.
// Shared by the host planner (plan.cu) and the kernels.
#pragma once

#include <stdint.h>

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
enum : int { PH_LION_MAIN = 0, PH_LION_APPLY = 1, PH_AXPY = 2 };

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
  int n_main;           // number of MAIN work items of this tensor (what `done` must reach)
};

struct Task {
  int tensor;
  int phase;
  long long e0;  // first element (flat index); multiple of the plan's alignment unit and a row start
  int n;         // elements (<= CAP); whole rows for >=2-D tensors
  int row0;      // first row (>=2-D tensors)
};

// Device pointers handed to the kernels by value.
struct PlanView {
  const DevTensor* tensors;
  const void* const* grads;  // [n_tensors], refreshed by kaon_plan_set_grads
  const Task* tasks;
  int n_tasks;
  int n_tensors;
  unsigned* task_counter;  // claims
  unsigned* done;          // [n_tensors] MAIN items finished
  unsigned* kept;          // [n_tensors] cautious kept count
  unsigned* status;        // 0 = ok; else the code of the first bounded wait that ran out
  unsigned char* codes;    // 2 bits per element
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
  unsigned* d_counters = nullptr;  // task_counter, status, done[n], kept[n] (contiguous; memset per step)
  size_t counters_bytes = 0;
  int64_t device_bytes = 0;
  int64_t launches = 0;
  int grid = 0;          // persistent grid size
  size_t smem_bytes = 0;
  int64_t total_elems = 0;
};
