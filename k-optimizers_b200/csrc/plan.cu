// Host side of libkaon_b200: plans (descriptor table + work list + scratch) and error plumbing.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <deque>
#include <string>
#include <vector>

#include "kaon_host.h"
#include "kaon_plan.h"

namespace kaon {

static thread_local std::string g_err;

int fail(int code, const char* fmt, ...) {
  char buf[512];
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(buf, sizeof buf, fmt, ap);
  va_end(ap);
  g_err = buf;
  return code;
}

int cuda_fail(cudaError_t e, const char* what) {
  return fail(KAON_E_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

static long long gcd_ll(long long a, long long b) { return b ? gcd_ll(b, a % b) : a; }

// Element alignment every work item must start on so that vector loads, the bulk copies of the
// momentum bytes and the 4-bit blocks line up.
static int align_unit(int momentum_kind, unsigned block) {
  if (momentum_kind != KAON_M_4BIT) return 8;
  return block == 256u ? 256 : 128;  // smaller power-of-two blocks divide 128
}

size_t momentum_bytes_per_cap(int mk) {
  switch (mk) {
    case KAON_M_F32: return (size_t)CAP * 4;
    case KAON_M_BF16: return (size_t)CAP * 2;
    case KAON_M_INT8: return (size_t)CAP;
    case KAON_M_4BIT: return (size_t)CAP / 2;
    default: return 0;
  }
}

// Split one tensor into work items: runs of whole rows (>=2-D) or flat runs (1-D), each at most CAP
// elements, each starting on the alignment unit.
static int split_tensor(const kaon_tensor_desc& d, int ti, int mk, bool lion, std::vector<Task>& out) {
  const long long n = d.numel;
  const int A = align_unit(mk, d.block);
  if (n == 0) return 0;
  if (d.rows > 0) {
    const long long C = n / d.rows;
    if (C * d.rows != n) return fail(KAON_E_INVALID, "tensor %d: numel %lld not divisible by rows %lld", ti, n, (long long)d.rows);
    if (n <= CAP && d.rows <= MAX_TASK_ROWS) {
      out.push_back(Task{ti, 0, 0, (int)n, 0});
      return 0;
    }
    const long long unit = A / gcd_ll(C, A);  // rows per aligned group
    long long rpt = (CAP / C) / unit * unit;   // rows per work item
    rpt = std::min<long long>(rpt, MAX_TASK_ROWS / unit * unit);
    if (rpt <= 0 && lion && mk != KAON_M_INT8 && C >= 8) {
      // Lion: flat runs instead of whole rows (only the row means tie a row together, and a pre-pass takes
      // those); int8 momentum keeps whole rows (one scale per row).  Returns 1: the caller marks the tensor.
      const long long chunk = CAP / A * A;
      for (long long e = 0; e < n; e += chunk) {
        const long long r0 = e / C;
        out.push_back(Task{ti, 0, e, (int)std::min<long long>(chunk, n - e), (int)r0, 0, (int)(e - r0 * C)});
      }
      return 1;
    }
    if (rpt <= 0 && !lion && C >= 256 && (C & 7) == 0 && (mk != KAON_M_INT8 || (C & 15) == 0)) {
      // Adakaon / Nekaon: the streaming launches (STATS, COUNT and APPLY as kernels of their own) never stage
      // whole rows, so a longer row is fine there.  Flat runs for the climb list; returns 2: the caller marks
      // the plan, and a step that cannot take the streaming form refuses.
      const long long chunk = CAP / A * A;
      for (long long e = 0; e < n; e += chunk)
        out.push_back(Task{ti, 0, e, (int)std::min<long long>(chunk, n - e), (int)(e / C), 0, (int)(e % C)});
      return 2;
    }
    if (rpt <= 0)
      return fail(KAON_E_UNSUPPORTED,
                  "tensor %d: %lld rows of %lld elements cannot be cut into row-aligned work items of <= %d "
                  "elements (row length x alignment group %lld too large)", ti, (long long)d.rows, C, CAP, unit);
    for (long long r = 0; r < d.rows; r += rpt) {
      long long nr = std::min<long long>(rpt, d.rows - r);
      out.push_back(Task{ti, 0, r * C, (int)(nr * C), (int)r});
    }
    return 0;
  }
  if (mk == KAON_M_INT8 && n > CAP && lion)
    return fail(KAON_E_UNSUPPORTED, "tensor %d: a 1-D tensor of %lld elements with int8 momentum (one scalar scale) exceeds %d", ti, n, CAP);
  const long long chunk = CAP / A * A;
  for (long long e = 0; e < n; e += chunk)
    out.push_back(Task{ti, 0, e, (int)std::min<long long>(chunk, n - e), 0});
  return 0;
}

}  // namespace kaon

namespace kaon {

int check_kahan(const kaon_plan* pl, int bf16_method) {
  if (bf16_method != KAON_W_KAHAN || pl->param_dtype != KAON_DT_BF16) return KAON_OK;
  for (int i = 0; i < pl->n_tensors; ++i)
    if (pl->h_tensors[i].numel > 0 && pl->h_tensors[i].shift == nullptr)
      return fail(KAON_E_INVALID, "bf16_method kahan: tensor %d has no shift buffer", i);
  return KAON_OK;
}

int check_device(const kaon_plan* pl) {
  int dev = -1;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaGetDevice");
  if (dev != pl->device)
    return fail(KAON_E_INVALID, "the plan lives on device %d but the current device is %d", pl->device, dev);
  return KAON_OK;
}

}  // namespace kaon

using namespace kaon;

extern "C" {

int kaon_abi_version(void) { return KAON_ABI_VERSION; }
const char* kaon_last_error(void) { return g_err.c_str(); }

int kaon_plan_create(kaon_plan** out, int optimizer, int param_dtype, int momentum_kind,
                     const kaon_tensor_desc* descs, int n) {
  if (!out || !descs || n <= 0) return fail(KAON_E_INVALID, "kaon_plan_create: null argument or n <= 0");
  if (param_dtype != KAON_DT_F32 && param_dtype != KAON_DT_BF16) return fail(KAON_E_INVALID, "param_dtype %d", param_dtype);
  if (momentum_kind < KAON_M_F32 || momentum_kind > KAON_M_NONE) return fail(KAON_E_INVALID, "momentum_kind %d", momentum_kind);
  if (optimizer < KAON_OPT_LION || optimizer > KAON_OPT_KPRODIGY) return fail(KAON_E_INVALID, "optimizer %d", optimizer);
  if (optimizer == KAON_OPT_LION && momentum_kind == KAON_M_NONE) return fail(KAON_E_INVALID, "Lion needs a momentum");
  if (optimizer == KAON_OPT_ADAPNM && momentum_kind == KAON_M_NONE) return fail(KAON_E_INVALID, "AdaPNM needs its two momenta");
  *out = nullptr;

  std::vector<DevTensor> tens(n);
  std::vector<std::vector<Task>> per(n);
  long long code_bytes = 0, total = 0, lion_aux_floats = 0;
  std::vector<int> flat_tensors;
  std::vector<char> long_rows(n, 0);
  for (int i = 0; i < n; ++i) {
    const kaon_tensor_desc& d = descs[i];
    if (!d.p || d.numel < 0) return fail(KAON_E_INVALID, "tensor %d: null weights or negative numel", i);
    if ((uintptr_t)d.p & 15) return fail(KAON_E_INVALID, "tensor %d: weights not 16-byte aligned", i);
    if (momentum_kind != KAON_M_NONE && !d.m && d.numel) return fail(KAON_E_INVALID, "tensor %d: momentum pointer missing", i);
    if ((uintptr_t)d.m & 15) return fail(KAON_E_INVALID, "tensor %d: momentum not 16-byte aligned", i);
    if ((momentum_kind == KAON_M_INT8 || momentum_kind == KAON_M_4BIT) && !d.m_scale && d.numel) return fail(KAON_E_INVALID, "tensor %d: m_scale missing", i);
    if (d.numel >= (1ll << 40)) return fail(KAON_E_UNSUPPORTED, "tensor %d: more than 2^40 elements", i);
    int bshift = 7;
    if (momentum_kind == KAON_M_4BIT && d.numel) {
      // reference src/kaon/_momentum_codec.py:192-200: the block in use is min(block, numel), or numel for
      // a non-positive setting; the caller passes that value
      const long long b = d.block;
      const bool pow2 = b >= 32 && b <= 256 && (b & (b - 1)) == 0;
      const bool whole = b == d.numel && (d.numel <= 128 || (d.rows <= 0 && optimizer != KAON_OPT_LION));
      if (pow2 && b < d.numel) { bshift = 0; while ((1ll << bshift) < b) ++bshift; }
      else if (whole || (pow2 && b == d.numel && d.numel <= 128)) bshift = 31;
      else return fail(KAON_E_UNSUPPORTED, "tensor %d: 4-bit block size %u (numel %lld): the library handles power-of-two blocks of 32..256 elements, one block covering a tensor of <= 128 elements, and one block covering a 1-D tensor of any length (not under Lion)", i, d.block, (long long)d.numel);
    }
    DevTensor& t = tens[i];
    t.p = d.p; t.m = d.m; t.m_scale = d.m_scale; t.stat_a = d.stat_a; t.stat_b = d.stat_b;
    t.shift = d.shift;
    if ((uintptr_t)d.shift & 15) return fail(KAON_E_INVALID, "tensor %d: shift buffer not 16-byte aligned", i);
    t.numel = d.numel;
    t.rows = (int)d.rows;
    t.cols = (int)(d.rows > 0 ? d.numel / d.rows : std::min<long long>(d.numel, 0x7fffffff));
    if (d.rows > 0x7fffffffll) return fail(KAON_E_UNSUPPORTED, "tensor %d: more than 2^31 rows", i);
    t.row_magic = t.cols > 1 ? (unsigned)((0x100000000ull + (unsigned)t.cols - 1) / (unsigned)t.cols) : 0u;
    t.tensor_id = d.tensor_id;
    t.block = d.block;
    t.bshift = bshift;
    t.code_off = code_bytes;
    code_bytes += ((d.numel + 3) / 4 + 63) / 64 * 64;  // 2 bits per element, 64-byte granules
    total += d.numel;
    int rc = split_tensor(d, i, momentum_kind, optimizer == KAON_OPT_LION, per[i]);
    if (rc < 0) return rc;
    if (rc == 1) {  // cut into flat runs: row means come from a pre-pass into the scratch
      t.chunk_rows = -1;
      t.aux_off = lion_aux_floats;
      lion_aux_floats += (d.rows + 63) / 64 * 64;
      flat_tensors.push_back(i);
    }
    if (rc == 2) {
      if (optimizer == KAON_OPT_ADAMUON)
        return fail(KAON_E_UNSUPPORTED, "tensor %d: rows of %d elements exceed a work item of %d (AdaMuon steps whole rows)", i, t.cols, CAP);
      long_rows[i] = 1;
    }
    t.n_main = (int)per[i].size();
  }

  int dev = 0;
  cudaError_t ce = cudaGetDevice(&dev);
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaGetDevice");
  cudaDeviceProp prop;
  ce = cudaGetDeviceProperties(&prop, dev);
  if (ce != cudaSuccess) return cuda_fail(ce, "cudaGetDeviceProperties");

  kaon_plan* pl = new kaon_plan();
  pl->device = dev;
  pl->sm_count = prop.multiProcessorCount;
  pl->optimizer = optimizer; pl->param_dtype = param_dtype; pl->momentum_kind = momentum_kind;
  pl->n_tensors = n;
  pl->total_elems = total;

  // Per-tensor stages.  Lion: MAIN, APPLY.  Adakaon (factored): STATS, FINAL, COUNT, APPLY; (1-D): FLAT.
  std::vector<std::vector<std::vector<Task>>> stages(n);
  long long aux_floats = 0;
  int max_cols = 1;
  if (optimizer == KAON_OPT_LION) {
    for (int i = 0; i < n; ++i) {
      stages[i].resize(2);
      for (const Task& t : per[i]) {
        Task m = t; m.phase = PH_LION_MAIN; stages[i][0].push_back(m);
        Task a = t; a.phase = PH_LION_APPLY; stages[i][1].push_back(a);
      }
    }
  } else {
    for (int i = 0; i < n; ++i) {
      DevTensor& t = tens[i];
      if (per[i].empty()) continue;
      if (t.rows <= 0) {
        if (t.numel > 0x7fffffffll) { delete pl; return fail(KAON_E_UNSUPPORTED, "tensor %d: a 1-D tensor of %lld elements (more than 2^31)", i, t.numel); }
        const bool lng = t.numel > CAP;  // one work item all the same, streamed from global memory
        stages[i].resize(1);
        if (!lng) max_cols = std::max<int>(max_cols, (int)t.numel);  // FLAT keeps the whole tensor as fp32 in shared memory
        stages[i][0].push_back(Task{i, PH_ADA_FLAT, 0, (int)t.numel, 0, lng ? 1 : 0, 0});
        t.aux_off = aux_floats; t.n_stats = 0; t.n_strips = 0; t.chunk_rows = 0;
        aux_floats += lng ? flat_long_size(t.numel) : 8;
        continue;
      }
      const long long C = t.cols;
      if (long_rows[i]) {  // streaming launches only: no row of it is ever staged by the persistent kernel
        pl->has_long_rows = true;
        t.chunk_rows = 1;
      } else {
        max_cols = std::max<int>(max_cols, (int)C);
        t.chunk_rows = (int)(per[i][0].n / C);
      }
      // rows per run: column partials (8 B per column per run) stay under ~10 % of the run's gradient
      // bytes, and a run is at least ~128 K elements
      long long run_rows = std::max<long long>(40, (131072 + C - 1) / C);
      run_rows = (run_rows + t.chunk_rows - 1) / t.chunk_rows * t.chunk_rows;
      stages[i].resize(4);
      int slot = 0;
      for (long long r = 0; r < t.rows; r += run_rows, ++slot) {
        long long nr = std::min<long long>(run_rows, t.rows - r);
        Task k{i, PH_ADA_STATS, r * C, (int)(nr * C), (int)r, slot, 0};
        stages[i][0].push_back(k);
        k.phase = PH_ADA_COUNT; stages[i][2].push_back(k);
        k.phase = PH_ADA_APPLY; stages[i][3].push_back(k);
      }
      t.n_stats = slot;
      t.n_count = slot;
      t.n_strips = (int)((C + FINAL_STRIP - 1) / FINAL_STRIP);
      for (int s = 0; s < t.n_strips; ++s)
        stages[i][1].push_back(Task{i, PH_ADA_FINAL, 0, (int)std::min<long long>(FINAL_STRIP, C - (long long)s * FINAL_STRIP), s * FINAL_STRIP, s, 0});
      t.aux_off = aux_floats;
      aux_floats += aux_size(t);
      aux_floats = (aux_floats + 63) / 64 * 64;
    }
  }
  int rc = optimizer == KAON_OPT_LION ? configure_launch(pl, prop) : configure_launch_adakaon(pl, prop, max_cols);
  if (rc) { delete pl; return rc; }

  // Work-list order: a tensor's next stage is released once at least `lag` other items have been
  // listed after its previous stage, so that an item's dependencies have normally finished when it is
  // claimed (claims are in list order, so a waiting item can never block the items it waits for),
  // while what the previous stage left in L2 is still there.
  const size_t lag = (size_t)pl->grid * 3;
  std::vector<Task> full_list, main_list, axpy_list;
  {
    std::deque<std::pair<size_t, std::pair<int, int>>> pending;  // (release position, (tensor, stage))
    auto emit = [&](int ti, int st) {
      for (const Task& t : stages[ti][st]) full_list.push_back(t);
      if (st + 1 < (int)stages[ti].size()) pending.push_back({full_list.size() + lag, {ti, st + 1}});
    };
    auto drain = [&](bool all) {
      while (!pending.empty() && (all || pending.front().first <= full_list.size())) {
        auto pr = pending.front().second; pending.pop_front(); emit(pr.first, pr.second);
      }
    };
    for (int i = 0; i < n; ++i) {
      if (stages[i].empty()) continue;
      // release what is due before each new item of this tensor's first stage
      std::vector<Task> first = stages[i][0];
      stages[i][0].clear();
      for (const Task& t : first) { drain(false); full_list.push_back(t); }
      if (stages[i].size() > 1) pending.push_back({full_list.size() + lag, {i, 1}});
    }
    drain(true);
  }
  for (const Task& t : full_list)
    if (t.phase != PH_LION_APPLY && t.phase != PH_ADA_COUNT) main_list.push_back(t);
  for (int i = 0; i < n; ++i)
    if (tens[i].m)
      for (const Task& t : per[i]) { Task a = t; a.phase = PH_AXPY; axpy_list.push_back(a); }

  // One device allocation: tensors | grads | tasks(full) | tasks(main) | tasks(axpy) | counters.
  auto up = [](size_t x) { return (x + 255) / 256 * 256; };
  size_t o_t = 0, o_g = o_t + up(sizeof(DevTensor) * n), o_f = o_g + up(sizeof(void*) * n);
  size_t o_m = o_f + up(sizeof(Task) * full_list.size()), o_a = o_m + up(sizeof(Task) * main_list.size());
  size_t o_c = o_a + up(sizeof(Task) * axpy_list.size());
  pl->counters_bytes = sizeof(unsigned) * (size_t)(2 + 5 * n);
  size_t tot = o_c + up(pl->counters_bytes);
  ce = cudaMalloc(&pl->d_block, tot);
  if (ce != cudaSuccess) { delete pl; return cuda_fail(ce, "cudaMalloc(plan tables)"); }
  if (optimizer != KAON_OPT_LION) code_bytes = 0;  // only Lion's MAIN/APPLY pair hands 2-bit codes over
  if (code_bytes > 0) {
    ce = cudaMalloc((void**)&pl->d_codes, (size_t)code_bytes);
    if (ce != cudaSuccess) { cudaFree(pl->d_block); delete pl; return cuda_fail(ce, "cudaMalloc(code scratch)"); }
  }
  if (optimizer == KAON_OPT_LION && !flat_tensors.empty()) {
    aux_floats = lion_aux_floats;
    ce = cudaMalloc((void**)&pl->d_flat_tensors, sizeof(int) * flat_tensors.size());
    if (ce == cudaSuccess) ce = cudaMemcpy(pl->d_flat_tensors, flat_tensors.data(), sizeof(int) * flat_tensors.size(), cudaMemcpyHostToDevice);
    if (ce != cudaSuccess) { cudaFree(pl->d_block); cudaFree(pl->d_codes); delete pl; return cuda_fail(ce, "cudaMalloc(flat-run tensor list)"); }
    pl->n_flat_tensors = (int)flat_tensors.size();
  }
  if (optimizer != KAON_OPT_LION || !flat_tensors.empty()) {
    ce = cudaMalloc((void**)&pl->d_aux, sizeof(float) * (size_t)std::max<long long>(aux_floats, 64));
    if (ce != cudaSuccess) { cudaFree(pl->d_block); cudaFree(pl->d_codes); delete pl; return cuda_fail(ce, "cudaMalloc(aux scratch)"); }
  }
  pl->device_bytes = (int64_t)tot + code_bytes + (pl->d_aux ? 4 * std::max<long long>(aux_floats, 64) : 0);
  char* base = (char*)pl->d_block;
  std::vector<const void*> grads(n);
  for (int i = 0; i < n; ++i) grads[i] = descs[i].g;
  cudaMemset(base + o_c, 0, up(pl->counters_bytes));
  cudaMemcpy(base + o_t, tens.data(), sizeof(DevTensor) * n, cudaMemcpyHostToDevice);
  cudaMemcpy(base + o_g, grads.data(), sizeof(void*) * n, cudaMemcpyHostToDevice);
  cudaMemcpy(base + o_f, full_list.data(), sizeof(Task) * full_list.size(), cudaMemcpyHostToDevice);
  cudaMemcpy(base + o_m, main_list.data(), sizeof(Task) * main_list.size(), cudaMemcpyHostToDevice);
  ce = cudaMemcpy(base + o_a, axpy_list.data(), sizeof(Task) * axpy_list.size(), cudaMemcpyHostToDevice);
  if (ce != cudaSuccess) { kaon_plan_destroy(pl); return cuda_fail(ce, "cudaMemcpy(plan tables)"); }
  pl->h_tensors = tens;
  pl->h_grads = grads;
  pl->d_tasks_full = (Task*)(base + o_f); pl->n_tasks_full = (int)full_list.size();
  pl->d_tasks_main = (Task*)(base + o_m); pl->n_tasks_main = (int)main_list.size();
  pl->d_tasks_axpy = (Task*)(base + o_a); pl->n_tasks_axpy = (int)axpy_list.size();
  pl->d_counters = (unsigned*)(base + o_c);
  PlanView& v = pl->view;
  v.tensors = (const DevTensor*)(base + o_t);
  v.grads = (const void* const*)(base + o_g);
  v.n_tensors = n;
  v.status = pl->d_counters;            // sticky: not cleared per step
  v.task_counter = pl->d_counters + 1;  // cleared per step from here on
  v.done = pl->d_counters + 2;
  v.kept = pl->d_counters + 2 + 4 * n;
  v.codes = pl->d_codes;
  v.aux = pl->d_aux;
  *out = pl;
  return KAON_OK;
}

int kaon_plan_set_grads(kaon_plan* pl, const void* const* grads, int n, void* stream) {
  if (!pl || !grads || n != pl->n_tensors) return fail(KAON_E_INVALID, "kaon_plan_set_grads: bad plan or n");
  if (int rc = check_device(pl)) return rc;
  for (int i = 0; i < n; ++i)
    if ((uintptr_t)grads[i] & 15) return fail(KAON_E_INVALID, "gradient %d not 16-byte aligned", i);
  // pageable source: the runtime stages it before returning, so the caller's array is free at once
  pl->h_grads.assign(grads, grads + n);
  cudaError_t ce = cudaMemcpyAsync((void*)pl->view.grads, grads, sizeof(void*) * (size_t)n,
                                   cudaMemcpyHostToDevice, (cudaStream_t)stream);
  return ce == cudaSuccess ? KAON_OK : cuda_fail(ce, "cudaMemcpyAsync(grad pointers)");
}

int kaon_plan_destroy(kaon_plan* pl) {
  if (!pl) return KAON_OK;
  cudaFree(pl->d_block);
  cudaFree(pl->d_codes);
  cudaFree(pl->d_aux);
  cudaFree(pl->d_flat_tensors);
  kaon::pnm_free(pl);
  kaon::kp_free(pl);
  cudaFree(pl->d_tasks_ema);
  cudaFree(pl->d_tasks_apply2);
  cudaFree(pl->d_tasks_na[0]);
  cudaFree(pl->d_tasks_na[1]);
  cudaFree(pl->d_tasks_stats);
  cudaFree(pl->d_counter2);
  cudaFree((void*)pl->d_signal);
  if (pl->muon_lanes_ready) {
    for (int l = 0; l < 4; ++l) {
      if (pl->muon_stream[l]) cudaStreamDestroy(pl->muon_stream[l]);
      if (pl->muon_join[l]) cudaEventDestroy(pl->muon_join[l]);
    }
    if (pl->muon_fork) cudaEventDestroy(pl->muon_fork);
  }
  delete pl;
  return KAON_OK;
}

int kaon_plan_status(kaon_plan* pl, void* stream) {
  if (!pl) return fail(KAON_E_INVALID, "null plan");
  unsigned st = 0;
  cudaError_t ce = cudaMemcpyAsync(&st, pl->view.status, 4, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize((cudaStream_t)stream);
  if (ce != cudaSuccess) return cuda_fail(ce, "kaon_plan_status");
  if (st) return fail(KAON_E_DEVICE, "device status %u: a bounded wait ran out (code = 1000*phase + kind)", st);
  return KAON_OK;
}

int kaon_plan_debug_stall(kaon_plan* pl, int tensor, uint32_t spin_limit) {
  if (!pl || tensor < 0 || tensor >= pl->n_tensors) return fail(KAON_E_INVALID, "kaon_plan_debug_stall: bad plan or tensor");
  if (pl->optimizer != KAON_OPT_LION) return fail(KAON_E_UNSUPPORTED, "kaon_plan_debug_stall: Lion plans only");
  if (int rc = check_device(pl)) return rc;
  pl->h_tensors[tensor].n_main += 1;  // one more MAIN item than the work list holds: APPLY's wait cannot be met
  pl->view.spin_limit = spin_limit;
  cudaError_t ce = cudaMemcpy((void*)(pl->view.tensors + tensor), &pl->h_tensors[tensor], sizeof(DevTensor), cudaMemcpyHostToDevice);
  return ce == cudaSuccess ? KAON_OK : cuda_fail(ce, "kaon_plan_debug_stall");
}

int64_t kaon_plan_device_bytes(const kaon_plan* pl) { return pl ? pl->device_bytes : 0; }
int64_t kaon_plan_launch_count(const kaon_plan* pl) { return pl ? pl->launches : 0; }

int kaon_plan_set_sm_limit(kaon_plan* pl, int sms) {
  if (!pl || sms < 1) return fail(KAON_E_INVALID, "kaon_plan_set_sm_limit: null plan or sms < 1");
  // Launches keep their size; the CTAs that land on the multiprocessors with the highest ids leave at once
  // (work is claimed from a counter, so the others do all of it) and those multiprocessors stay empty.
  pl->view.sm_reserve = sms < pl->sm_count ? (unsigned)(pl->sm_count - sms) : 0u;
  return KAON_OK;
}

int kaon_plan_set_peers(kaon_plan* pl, const int64_t* byte_delta, int n_peers) {
  if (!pl || n_peers < 0 || n_peers > KAON_MAX_PEERS || (n_peers > 0 && !byte_delta))
    return fail(KAON_E_INVALID, "kaon_plan_set_peers: bad arguments (at most 7 peers)");
  for (int r = 0; r < n_peers; ++r)
    if (byte_delta[r] == 0 || (byte_delta[r] & 15))
      return fail(KAON_E_INVALID, "kaon_plan_set_peers: a mirror offset must be a non-zero multiple of 16 bytes");
  pl->view.peers = kaon::Peers{};
  pl->view.peers.n = n_peers;
  for (int r = 0; r < n_peers; ++r) pl->view.peers.delta[r] = byte_delta[r];
  return KAON_OK;
}

int kaon_plan_kept_counts(kaon_plan* pl, uint32_t* host_out, int n, void* stream) {
  if (!pl || !host_out || n != pl->n_tensors) return fail(KAON_E_INVALID, "kaon_plan_kept_counts: bad arguments");
  cudaError_t ce = cudaMemcpyAsync(host_out, pl->view.kept, 4 * (size_t)n, cudaMemcpyDeviceToHost, (cudaStream_t)stream);
  if (ce == cudaSuccess) ce = cudaStreamSynchronize((cudaStream_t)stream);
  return ce == cudaSuccess ? KAON_OK : cuda_fail(ce, "kaon_plan_kept_counts");
}

}  // extern "C"
