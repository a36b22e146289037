// Host-only helpers shared by the translation units of libkaon_b200.
#pragma once

#include <cuda_runtime.h>
#include <stddef.h>

struct kaon_plan;

namespace kaon {

int fail(int code, const char* fmt, ...);           // records the message, returns code
int cuda_fail(cudaError_t e, const char* what);     // KAON_E_CUDA with the runtime's message
size_t momentum_bytes_per_cap(int momentum_kind);   // bytes of momentum storage per CAP elements
int configure_launch(kaon_plan* pl, const cudaDeviceProp& prop);  // Lion: grid + dynamic shared memory
int configure_launch_adakaon(kaon_plan* pl, const cudaDeviceProp& prop, int max_cols);
// bf16_method == KAHAN with bf16 weights needs every tensor's shift buffer: KAON_OK or an error
int check_kahan(const kaon_plan* pl, int bf16_method);
// the calling thread's current device must be the one the plan was built on: KAON_OK or KAON_E_INVALID
int check_device(const kaon_plan* pl);

#define KAON_CUDA(call)                                              \
  do {                                                               \
    cudaError_t e__ = (call);                                        \
    if (e__ != cudaSuccess) return ::kaon::cuda_fail(e__, #call);    \
  } while (0)

}  // namespace kaon
