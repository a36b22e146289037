// Adakaon step and the Nekaon climb: entry points (kernels under construction).
#include "kaon_host.h"
#include "kaon_plan.h"

using namespace kaon;

extern "C" int kaon_adakaon_step(kaon_plan* pl, const kaon_adakaon_hparams* h, uint64_t seed,
                                 uint32_t step, void* stream) {
  (void)pl; (void)h; (void)seed; (void)step; (void)stream;
  return fail(KAON_E_UNSUPPORTED, "kaon_adakaon_step: not built yet");
}

extern "C" int kaon_msam_apply(kaon_plan* pl, double alpha, double bound, uint32_t tag, uint64_t seed,
                               uint32_t step, void* stream) {
  (void)pl; (void)alpha; (void)bound; (void)tag; (void)seed; (void)step; (void)stream;
  return fail(KAON_E_UNSUPPORTED, "kaon_msam_apply: not built yet");
}
