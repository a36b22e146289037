/*
 * kaon_b200.h — C ABI of libkaon_b200.so: the fused optimizer step of kaon (Koronos/K-Optimizers)
 * for NVIDIA B200 (sm_100a).
 *
 * The reference is pure Python and has no FFI for this path; its boundary is the Python optimizer
 * classes.  Every entry point below names the reference function whose work it replaces (path within
 * the reference project).  Conventions: plain C types; raw DEVICE pointers unless a parameter says
 * "host"; every call returns 0 on success or a negative KAON_E_* code and records a message readable
 * with kaon_last_error(); nothing throws across the ABI; launches are asynchronous on the stream
 * passed in (a cudaStream_t cast to void*); the library creates no threads.
 */
#ifndef KAON_B200_H
#define KAON_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define KAON_ABI_VERSION 2

/* parameter / gradient element type (grads have the parameter's type) */
#define KAON_DT_F32 0
#define KAON_DT_BF16 1

/* momentum_dtype (reference src/kaon/_momentum_codec.py:42) */
#define KAON_M_F32 0
#define KAON_M_BF16 1
#define KAON_M_INT8 2 /* per-row absmax, one fp32 scale per dim-0 row, one scalar for 1-D */
#define KAON_M_4BIT 3 /* flat blocks of `block` elements, nibble-packed, even index in the low nibble */
#define KAON_M_NONE 4 /* betas[0] == 0: no first moment (Adakaon / AdaMuon only) */

/* bf16_method (reference src/kaon/_backend.py:82-122) */
#define KAON_W_NONE 0 /* p - bf16(delta), round to nearest even */
#define KAON_W_SR 1   /* stochastic rounding, Philox4x32-7 keyed on (seed, step, tensor id, element) */
#define KAON_W_KAHAN 2 /* compensated bf16 write with the per-tensor `shift` buffer (_backend.py:89-94) */

/* optimizer kinds a plan can be built for */
#define KAON_OPT_LION 0
#define KAON_OPT_ADAKAON 1
#define KAON_OPT_ADAMUON 2
#define KAON_OPT_ADAPNM 3
#define KAON_OPT_KPRODIGY 4

/* error codes */
#define KAON_OK 0
#define KAON_E_INVALID (-1)     /* bad argument (message says which) */
#define KAON_E_UNSUPPORTED (-2) /* a shape / option the library has no kernel for */
#define KAON_E_CUDA (-3)        /* a CUDA runtime call failed */
#define KAON_E_DEVICE (-4)      /* the device status word reported a bounded wait that ran out */

/* SR stream tags: which of a step's weight writes a draw belongs to */
#define KAON_TAG_UPDATE 0
#define KAON_TAG_REMOVE 1
#define KAON_TAG_CLIMB 2
#define KAON_TAG_EVAL 3
#define KAON_TAG_TRAIN 4

/* One tensor of a parameter group: a row of the descriptor table.  All pointers are device pointers
 * that stay valid for the life of the plan, except `g`, which kaon_plan_set_grads may replace before
 * every step.  Layout of the state tensors is the reference's state_dict layout
 * (src/kaon/_momentum_codec.py:295-301, 350-360; src/kaon/adakaon.py:318-335). */
typedef struct kaon_tensor_desc {
  void* p;         /* weights, numel elements of the plan's param dtype; 16-byte aligned */
  const void* g;   /* gradients, same dtype and shape; 16-byte aligned; may be NULL (tensor skipped) */
  void* m;         /* momentum: fp32/bf16 [numel] | int8 [numel] | uint8 [(numel+1)/2]; NULL if none */
  float* m_scale;  /* int8: [rows] (or [1] for 1-D); 4bit: [ceil(numel/block)]; else NULL */
  float* stat_a;   /* Adakaon/AdaMuon: row[rows] for ndim>=2, v[numel] for 1-D; Lion: NULL */
  float* stat_b;   /* Adakaon/AdaMuon: col[cols] for ndim>=2; else NULL */
  int64_t numel;
  int64_t rows;    /* shape[0] when ndim >= 2, else 0 (1-D tensor) */
  uint32_t tensor_id; /* position in the optimizer's flattened param list: keys the SR stream */
  uint32_t block;  /* 4-bit block size actually in use: min(momentum_4bit_block, numel), or numel for a
                    * non-positive setting (src/kaon/_momentum_codec.py:192-200).  Plans take a power of two
                    * from 32 to 256, one block over a tensor of <= 128 elements, and (not under Lion) one
                    * block over a 1-D tensor of any length; anything else is KAON_E_UNSUPPORTED. */
  void* shift;     /* bf16_method="kahan" with bf16 weights: compensation buffer state["shift"], bf16
                      [numel], 16-byte aligned; NULL otherwise */
} kaon_tensor_desc;

typedef struct kaon_plan kaon_plan; /* opaque: descriptor table, work list and scratch on one device */

/* Hyper-parameters travel as the Python doubles the reference holds in param_groups; the library casts
 * to fp32 where the reference's torch ops do (e.g. the lerp weight is (float)(1.0 - beta)). */
typedef struct kaon_lion_hparams {
  double lr, beta1, beta2, weight_decay;
  int32_t cautious, gradient_centralization, bf16_method, reserved;
} kaon_lion_hparams;

typedef struct kaon_adakaon_hparams {
  double lr, beta1, beta2, eps1, weight_decay, clip_threshold;
  int32_t cautious, gradient_centralization, bf16_method, reserved;
  /* Nekaon (MSAM with norm="none", reference src/kaon/msam.py:374-406) fused into the step: if
   * msam_remove, every weight first gets  p += clamp(nan_to_num(decode(m_old) * alpha_remove),
   * +-bound_remove)  (taking the previous climb back out); if msam_climb, after the update
   * p += clamp(nan_to_num(decode(m_new as stored) * alpha_climb), +-bound_climb).  bf16 weights are
   * stochastically rounded after each of the three writes (stream tags REMOVE / UPDATE / CLIMB). */
  int32_t msam_remove, msam_climb;
  double msam_alpha_remove, msam_bound_remove, msam_alpha_climb, msam_bound_climb;
} kaon_adakaon_hparams;

typedef struct kaon_adamuon_hparams {
  double lr, beta1, beta2, eps1, weight_decay, clip_threshold;
  int32_t ns_steps, cautious, gradient_centralization, bf16_method;
} kaon_adamuon_hparams;

/* AdaPNM (src/kaon/adapnm.py:344-366, 998-1017).  group_step is the parameter group's 1-based step count
 * ("step" in the reference's param_groups): it sets the bias corrections and which stored momentum is the
 * positive one (odd: "m_pos"). */
typedef struct kaon_adapnm_hparams {
  double lr, beta1, beta2, beta0, eps, weight_decay, clip_threshold;
  int32_t cautious, gradient_centralization, ams_bound, bf16_method;
  uint32_t group_step, reserved;
} kaon_adapnm_hparams;

/* KProdigy (src/kaon/kprodigy.py:329-404).  The distance estimate d is a host scalar of the caller (the
 * reference keeps it in param_groups); the two passes take the values the reference computes around it:
 * pass 1 the d of the top of the step, alpha_s = (d/d0)*d or (d/d0)*dlr, the coupled weight decay (0 when
 * decoupled); pass 2 the d as just updated, the dlr of the top of the step, decay_dlr = weight_decay*dlr
 * (0 unless decoupled). */
typedef struct kaon_kprodigy_pass1_hparams {
  double beta1, beta2, beta3, d, alpha_s, weight_decay_coupled, eps_factored;
  int32_t do_d, gradient_centralization, factored, reserved;
} kaon_kprodigy_pass1_hparams;

typedef struct kaon_kprodigy_pass2_hparams {
  double d, dlr, eps, decay_dlr;
  int32_t cautious, gradient_centralization, factored, bf16_method;
} kaon_kprodigy_pass2_hparams;

/* ---- library ---- */
int kaon_abi_version(void);
const char* kaon_last_error(void); /* message of the calling thread's last failed call */

/* ---- descriptor tables (replace the foreach batcher: src/kaon/adakaon.py:757-838,
 *      src/kaon/lion.py:366-414, src/kaon/_backend.py:59-77) ---- */

/* Build the device-side table, the work list and the scratch for `n` tensors (host array `descs`)
 * of one parameter group on the current device.  Blocks until the table is resident. */
int kaon_plan_create(kaon_plan** out, int optimizer, int param_dtype, int momentum_kind,
                     const kaon_tensor_desc* descs, int n);
/* Replace the gradient pointers (host array of n device pointers, NULL = skip that tensor this step).
 * Asynchronous on `stream`; the host array may be reused as soon as the call returns. */
int kaon_plan_set_grads(kaon_plan* plan, const void* const* grads, int n, void* stream);
int kaon_plan_destroy(kaon_plan* plan);
/* Synchronise `stream` and read the plan's device status word: 0, or KAON_E_DEVICE with a message. */
int kaon_plan_status(kaon_plan* plan, void* stream);
/* Test hook (no reference counterpart): makes the bounded waits of a Lion plan observable without
 * faulting or hanging anything.  Raises tensor `tensor`'s expected count of finished MAIN work items by
 * one - a count the work list can never reach - and sets the number of polls a completion-counter wait
 * makes before it gives up.  The next kaon_lion_step then returns normally with that tensor's weights
 * not updated, kaon_plan_status reports KAON_E_DEVICE, and the plan stays drained (every later step is a
 * no-op) until it is destroyed.  Only the completion-counter polls are shortened; waits on copies in
 * flight keep their limit. */
int kaon_plan_debug_stall(kaon_plan* plan, int tensor, uint32_t spin_limit);
/* Bytes of device memory the plan owns (tables + scratch), and how many kernels it has launched. */
int64_t kaon_plan_device_bytes(const kaon_plan* plan);
int64_t kaon_plan_launch_count(const kaon_plan* plan);
/* Per-tensor cautious kept counts of the last step, copied to a host array of n uint32 (synchronises
 * `stream`).  Diagnostic: lets a test compare the mask population with the oracle's. */
int kaon_plan_kept_counts(kaon_plan* plan, uint32_t* host_out, int n, void* stream);

/* Weight mirrors on other GPUs (no reference counterpart: the reference has no distributed code).
 * After this call every step kernel of the plan stores each weight it writes at address a also at
 * a + byte_delta[r] for r < n_peers: the ZeRO-1 publish of the owned weights is fused into the step
 * as plain peer stores over NVLink, tile by tile, instead of an all-gather afterwards.
 * byte_delta[r] = (address at which THIS process has rank r's weight buffer mapped) - (address of its
 * own weight buffer); every tensor of the plan must lie in that buffer, the buffers must have the same
 * layout on every rank, and each delta must be a multiple of 16.  The caller maps the peer memory (CUDA
 * IPC, symmetric memory) and orders the ranks: no peer may read the weights, or start its next step,
 * before a barrier that follows this step on every rank's stream.  n_peers = 0 switches mirroring off. */
#define KAON_MAX_PEERS 7
int kaon_plan_set_peers(kaon_plan* plan, const int64_t* byte_delta, int n_peers);
/* Keep the step kernels of the plan off all but `sms` multiprocessors (at least half of the device's; the Lion
 * and Adakaon step kernels honour it).  They are persistent - their CTAs hold every register of a
 * multiprocessor until the launch ends - so a collective that should run beside a step (the next wave's
 * gradient reduce-scatter) finds no room unless some multiprocessors are left empty: CTAs that land on the
 * others leave before claiming work. */
int kaon_plan_set_sm_limit(kaon_plan* plan, int sms);

/* ---- optimizer steps ---- */

/* One Lion step over every tensor of the plan whose gradient is set.
 * Replaces Lion._step_impl / _bucket / _step_one_param (src/kaon/lion.py:322-352, 416-485) together
 * with centralize_grads_ (src/kaon/_backend.py:147-177), the codec store (src/kaon/lion.py:244-317),
 * cautious_batched_ (src/kaon/_backend.py:127-142) and subtract_batched_ (src/kaon/_backend.py:102-122).
 * `step` is the 1-based step index; (seed, step, tensor_id, element) key the SR noise. */
int kaon_lion_step(kaon_plan* plan, const kaon_lion_hparams* hp, uint64_t seed, uint32_t step,
                   void* stream);

/* One Lion step over ONE tensor that allocates nothing (no counterpart in the reference: it exists for
 * callers that may not call cudaMalloc where they step the optimizer - code under a memory pool it must
 * not disturb, launch-only real-time paths, hosts that own every allocation).  Same arithmetic and the
 * same kernel as kaon_lion_step, but the table, work list, counters and code scratch that
 * kaon_plan_create would allocate live in a device array built into the library (about 1.3 MiB on every
 * GPU that loads it).  `tensor` is a HOST struct; weights, gradient, momentum (4-bit, block 128 or one
 * block for <= 128 elements) and m_scale must be set; numel <= KAON_NOALLOC_MAX_NUMEL, else
 * KAON_E_UNSUPPORTED.  Calls no cudaMalloc/cudaFree.  The first call on a device resolves the array's
 * address and configures the kernel: make it before any stream capture.  All calls on a device share
 * the array: calls whose kernels overlap on the GPU race; calls ordered on one stream do not.
 * bf16_method is KAON_W_NONE or KAON_W_SR (the Kahan write needs a plan: KAON_E_UNSUPPORTED).  Two host
 * threads may make the first call on a device at the same time (the set-up is behind a mutex). */
#define KAON_NOALLOC_MAX_NUMEL (1 << 22)
int kaon_lion_step_noalloc(const kaon_tensor_desc* tensor, int param_dtype, const kaon_lion_hparams* hp,
                           uint64_t seed, uint32_t step, void* stream);
/* Device status of the kaon_lion_step_noalloc calls made so far on the current device (no counterpart
 * in the reference; allocates nothing).  Synchronises `stream`, returns KAON_OK, or KAON_E_DEVICE if a
 * bounded wait ran out inside one of those calls (that call stopped early and left its tensor partly
 * stepped; later calls ran normally), and clears the record. */
int kaon_lion_noalloc_status(void* stream);

/* One Adakaon step.  Replaces Adakaon._step_impl / _factored_bucket / _nonfactored_bucket /
 * _step_one_param (src/kaon/adakaon.py:339-383, 840-1014), update_factored_state and
 * factored_inv_sqrt_factors (src/kaon/_factored.py:26-83), the codec EMA
 * (src/kaon/_momentum_codec.py:303-340, 357-389), cautious and the weight write as for Lion;
 * optionally the Nekaon removal and climb (the msam_* fields of kaon_adakaon_hparams). */
int kaon_adakaon_step(kaon_plan* plan, const kaon_adakaon_hparams* hp, uint64_t seed, uint32_t step,
                      void* stream);

/* AdaPNM.  Replaces AdaPNM._step_impl / _native_dispatch / _step_foreach / _factored_bucket /
 * _nonfactored_bucket / _pn_stacked / _step_one_param / _pn_one (src/kaon/adapnm.py:599-645, 1039-1273)
 * with the same second-moment, codec, cautious and weight-write pieces as kaon_adakaon_step.  The plan is
 * created with optimizer KAON_OPT_ADAPNM; each descriptor's m / m_scale name the state's "m_pos" buffers,
 * stat_a / stat_b its row / col (or v) statistics.  kaon_adapnm_attach then names, per tensor, the
 * "m_neg" buffer, its scales (int8 / 4-bit; else null) and, for ams_bound, the 1-D tensors' max_v (null
 * array or null entries otherwise); it must be called once before the first step.  weight_decay is
 * applied to the weights before the update (p *= 1 - lr*wd, rounded to the weights' dtype), as the
 * reference does. */
int kaon_adapnm_attach(kaon_plan* plan, const void* const* m_neg, float* const* m_neg_scale,
                       float* const* max_v, int n);
int kaon_adapnm_step(kaon_plan* plan, const kaon_adapnm_hparams* hp, uint64_t seed, uint32_t step,
                     void* stream);

/* KProdigy.  Replaces KProdigy._pass1_per_param / _pass1_foreach / _pass1_momentum_foreach /
 * _pass1_second_moment_foreach / _update_momentum (src/kaon/kprodigy.py:417-703, 762-782) and _apply_updates /
 * _update_one_param / _update_foreach / _factored_bucket / _full_bucket (:706-949); the D update between
 * them (:371-391) stays with the caller.  The plan is created with optimizer KAON_OPT_KPRODIGY (momentum kind
 * KAON_M_NONE for betas[0] == 0); stat_a / stat_b name "row" / "col" of a factored tensor, stat_a alone the
 * full "v".  kaon_kprodigy_attach names each tensor's "s" buffer and "p0" reference point (a null entry for
 * the reference's zero-dimensional zero) with the slice_p they were built for.
 * kaon_kprodigy_pass1: statistics and moments; with do_d it synchronises `stream` and leaves, per tensor i,
 * sums_host[2i] = sum over the sliced elements of g*(p0 - p) and sums_host[2i+1] = sum |s| (zeros for a
 * tensor without a gradient); the caller folds them in tensor order.  kaon_kprodigy_pass2: the weights. */
int kaon_kprodigy_attach(kaon_plan* plan, float* const* s, const float* const* p0, int n, int64_t slice_p);
int kaon_kprodigy_pass1(kaon_plan* plan, const kaon_kprodigy_pass1_hparams* hp, float* sums_host, void* stream);
int kaon_kprodigy_pass2(kaon_plan* plan, const kaon_kprodigy_pass2_hparams* hp, uint64_t seed, uint32_t step,
                        void* stream);

/* One AdaMuon step.  Replaces AdaMuon._run_step / _factored_bucket / _nonfactored_bucket /
 * _step_one_param (src/kaon/adamuon.py:327-352, 434-615): per >=2-D tensor the EMA of the raw gradient
 * (less its row means when gradient_centralization is set, :334-335; the mask then compares with that
 * centralised gradient) through the codec, Newton-Schulz of the fp32 momentum (tcgen05 GEMMs), factored second moment of the
 * orthogonalised signal, clip, 0.2*lr scale, weight decay, cautious mask against the raw gradient,
 * weight write; 1-D tensors take the Adam-style branch.  `workspace` (device, 256-byte aligned, at least
 * kaon_adamuon_workspace_bytes(plan)) holds the orthogonalised matrices between the kernels; the caller
 * owns it and may reuse it between steps and plans. */
int64_t kaon_adamuon_workspace_bytes(const kaon_plan* plan);
/* Byte offset, inside the workspace, of tensor `tensor`'s orthogonalised matrix (bf16 [rows, cols]) as
 * the last step left it; -1 for 1-D tensors.  Diagnostic: lets a test feed the same matrix to the oracle. */
int64_t kaon_adamuon_signal_offset(const kaon_plan* plan, int tensor);
int kaon_adamuon_step(kaon_plan* plan, const kaon_adamuon_hparams* hp, void* workspace,
                      int64_t workspace_bytes, uint64_t seed, uint32_t step, void* stream);

/* Nekaon climb / removal / eval / train swap over every tensor of the plan that has a momentum:
 * p += clamp(nan_to_num(decode(m_stored) * (float)alpha), +-(float)bound), stochastic rounding for
 * bf16 weights (stream tag `tag`), plain add for fp32.  Replaces MSAM._apply with norm="none"
 * (src/kaon/msam.py:201-235) and _axpy_4bit_batched (src/kaon/_fused_triton.py:1145-1179). */
int kaon_msam_apply(kaon_plan* plan, double alpha, double bound, uint32_t tag, uint64_t seed,
                    uint32_t step, void* stream);

/* ---- Newton-Schulz orthogonalisation (zeropower_via_newtonschulz5, src/kaon/adamuon.py:97-149) ----
 * x_bf16 [rows, cols] (bf16, row-major, unnormalised) -> out_bf16 [rows, cols]: X = x/(||x||_F + 1e-7),
 * steps x { A = X X^T; B = b A + c A A; X = a X + B X } as tcgen05 bf16 GEMMs with fp32 accumulation.
 * The workspace (256-byte aligned, kaon_newton_schulz_workspace_bytes) holds the iterates; its first
 * word is the call's device status (non-zero: a bounded wait ran out).  out may not alias x. */
int64_t kaon_newton_schulz_workspace_bytes(int64_t rows, int64_t cols);
int kaon_newton_schulz(const void* x_bf16, int64_t rows, int64_t cols, int steps, void* out_bf16,
                       void* workspace, int64_t workspace_bytes, void* stream);

/* ---- standalone codec (src/kaon/_momentum_codec.py:72-189; CodecBuffer.read/write,
 *      src/kaon/_wrappers.py:56-168) ---- */
int kaon_codec_encode_int8(const float* m, int64_t numel, int64_t rows, int8_t* codes, float* scale,
                           void* stream);
int kaon_codec_decode_int8(const int8_t* codes, const float* scale, int64_t numel, int64_t rows,
                           float* m, void* stream);
int kaon_codec_encode_4bit(const float* m, int64_t numel, int64_t block, uint8_t* packed,
                           float* scale, void* stream);
int kaon_codec_decode_4bit(const uint8_t* packed, const float* scale, int64_t numel, int64_t block,
                           float* m, void* stream);

/* ---- weight write on its own (src/kaon/_stochastic_rounding.py:39-103): p += alpha * delta ---- */
int kaon_sr_add(void* p, int param_dtype, const float* delta, int64_t numel, float alpha,
                int bf16_method, uint64_t seed, uint32_t step, uint32_t tensor_id, uint32_t tag,
                void* stream);

#ifdef __cplusplus
}
#endif
#endif /* KAON_B200_H */
