// Device-side hyper-parameter block of the Adakaon / AdaMuon kernels and the launch helpers other
// translation units use.
#pragma once

#include <stddef.h>
#include <stdint.h>

#include "kaon_plan.h"

namespace kaon {

struct AdaDev {
  float w1, w1m1, w2, w2m1, eps1, clip, lrwd, upd_scale;
  int small_w1, small_w2, has_eps, has_wd, cautious, gc, sr, has_m;
  int remove, climb, kahan, int8;
  float a_remove, b_remove, a_climb, b_climb;
  uint32_t step, k0, k1;
};

typedef void (*AdaKernel)(PlanView, AdaDev, int);
AdaKernel pick_ada(int param_dtype, int momentum_kind, bool muon);
size_t x_offset_rows(const kaon_plan* pl);
// COUNT and APPLY as launches of their own (plans whose factored tensors all stream)
int ensure_apply2(kaon_plan* pl);
int launch_count_apply(kaon_plan* pl, const PlanView& base, const AdaDev& hp, cudaStream_t s);
int launch_stats(kaon_plan* pl, const PlanView& base, const AdaDev& hp, cudaStream_t s);
// the STATS launch over a caller's list of STATS items (all of which pass stats_item_ok); KAON_OK or an error
bool stats_item_ok(const kaon_plan* pl, const Task& t);
int launch_stats_tasks(kaon_plan* pl, const PlanView& base, const AdaDev& hp, const Task* tasks, int n, cudaStream_t s);

}  // namespace kaon
