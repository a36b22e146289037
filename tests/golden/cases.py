"""The optimizer cases behind the golden vectors: one table read by the generator
(make_golden.py, which runs the reference) and by the tests (which run the oracle and the CUDA path).

name -> (optimizer, constructor kwargs, shapes, param dtype, steps, seed, options)
options: correlated (a steady gradient direction under the noise), lr_sched ("cosine5": 1e-4 -> 1e-5 over 5 steps, the C4 schedule shortened), outlier (1 % of
the grads x100, the C3 grad distribution), sample (stride for big tensors), store_inputs, nekaon_eval.
"""
import math

SMALL = [(48, 64), (16, 20, 3, 3), (96,), (5, 7), (130,)]
MUON = [(48, 32), (32, 64), (40,), (8, 4, 3, 3)]
C1 = [(1024, 1024), (320, 320, 3, 3), (1024,)]
# rows of 16 640 elements (longer than a work item's 16 384) and a 1-D tensor above a work item
LONG = [(2, 2080, 2, 4), (50000,), (24, 16)]


def cosine5(t):
    return 1e-5 + 0.5 * (1e-4 - 1e-5) * (1 + math.cos(math.pi * t / 5))


SCHEDULES = {"cosine5": cosine5}

CASES = {
    # Lion, the C2 settings on small shapes; "none" makes weights comparable bit for bit
    "lion_4bit_none": ("Lion", dict(lr=2e-4, betas=(0.95, 0.98), momentum_dtype="4bit", cautious=True, bf16_method="none"), SMALL, "bf16", 6, 0, {}),
    "lion_4bit_nogc_wd": ("Lion", dict(lr=2e-4, betas=(0.95, 0.98), weight_decay=0.1, momentum_dtype="4bit", gradient_centralization=False, bf16_method="none"), SMALL, "bf16", 6, 1, {}),
    "lion_int8_none": ("Lion", dict(lr=2e-4, betas=(0.9, 0.99), momentum_dtype="int8", bf16_method="none"), SMALL, "bf16", 5, 2, {}),
    "lion_bf16_nocautious": ("Lion", dict(lr=2e-4, momentum_dtype="bfloat16", cautious=False, bf16_method="none"), SMALL, "bf16", 4, 3, {}),
    "lion_4bit_f32params": ("Lion", dict(lr=2e-4, betas=(0.95, 0.98), momentum_dtype="4bit"), SMALL, "f32", 5, 4, {}),
    "lion_4bit_sr": ("Lion", dict(lr=2e-4, betas=(0.95, 0.98), momentum_dtype="4bit"), SMALL, "bf16", 4, 5, {}),
    "lion_4bit_kahan": ("Lion", dict(lr=2e-4, betas=(0.95, 0.98), momentum_dtype="4bit", bf16_method="kahan"), SMALL, "bf16", 6, 6, {}),
    "lion_int8_kahan_wd_nocautious": ("Lion", dict(lr=2e-4, momentum_dtype="int8", weight_decay=0.1, cautious=False, bf16_method="kahan"), SMALL, "bf16", 4, 7, {}),
    "lion_4bit_block64": ("Lion", dict(lr=2e-4, betas=(0.95, 0.98), momentum_dtype="4bit", momentum_4bit_block=64, bf16_method="none"), SMALL, "bf16", 5, 8, {}),
    "lion_4bit_long": ("Lion", dict(lr=2e-4, betas=(0.95, 0.98), momentum_dtype="4bit", cautious=True, bf16_method="none"), LONG, "bf16", 3, 9, {}),
    # Adakaon, the C1 settings on small shapes
    "adakaon_int8_none": ("Adakaon", dict(lr=1e-4, betas=(0.9, 0.999), momentum_dtype="int8", bf16_method="none"), SMALL, "bf16", 6, 10, {}),
    "adakaon_int8_sr": ("Adakaon", dict(lr=1e-4, betas=(0.9, 0.999), momentum_dtype="int8"), SMALL, "bf16", 6, 11, {}),
    "adakaon_int8_outlier": ("Adakaon", dict(lr=1e-4, betas=(0.9, 0.999), momentum_dtype="int8", bf16_method="none"), SMALL, "bf16", 5, 12, {"outlier": True}),
    "adakaon_4bit_wd_f32": ("Adakaon", dict(lr=1e-4, betas=(0.2, 0.999), weight_decay=0.1, momentum_dtype="4bit"), SMALL, "f32", 5, 13, {}),
    "adakaon_bf16m_none": ("Adakaon", dict(lr=1e-4, momentum_dtype="bfloat16", bf16_method="none"), SMALL, "bf16", 4, 14, {}),
    "adakaon_int8_kahan": ("Adakaon", dict(lr=1e-4, betas=(0.9, 0.999), momentum_dtype="int8", bf16_method="kahan"), SMALL, "bf16", 6, 15, {}),
    "adakaon_4bit_block256_wd": ("Adakaon", dict(lr=1e-4, betas=(0.9, 0.999), weight_decay=0.05, momentum_dtype="4bit", momentum_4bit_block=256, bf16_method="none"), SMALL, "bf16", 5, 16, {}),
    "adakaon_4bit_block32_f32": ("Adakaon", dict(lr=1e-4, betas=(0.9, 0.999), momentum_dtype="4bit", momentum_4bit_block=32), SMALL, "f32", 4, 17, {}),
    "adakaon_int8_long": ("Adakaon", dict(lr=1e-4, betas=(0.9, 0.999), momentum_dtype="int8", bf16_method="none"), LONG, "bf16", 3, 18, {}),
    # Nekaon (C4 settings; fp32 params make the three writes deterministic) under a cosine LR
    "nekaon_f32": ("Nekaon", dict(lr=1e-4, betas=(0.2, 0.999)), SMALL, "f32", 5, 20, {"lr_sched": "cosine5", "nekaon_eval": True}),
    "nekaon_bf16": ("Nekaon", dict(lr=1e-4, betas=(0.2, 0.999)), SMALL, "bf16", 5, 21, {"lr_sched": "cosine5"}),
    # AdaMuon (C5 settings)
    "adamuon_int8_none": ("AdaMuon", dict(lr=1e-3, ns_steps=2, cautious=True, momentum_dtype="int8", bf16_method="none"), MUON, "bf16", 4, 30, {}),
    "adamuon_int8_kahan": ("AdaMuon", dict(lr=1e-3, ns_steps=2, cautious=True, momentum_dtype="int8", bf16_method="kahan"), MUON, "bf16", 3, 31, {}),
    "adamuon_int8_gc": ("AdaMuon", dict(lr=1e-3, ns_steps=2, cautious=True, momentum_dtype="int8", gradient_centralization=True, bf16_method="none"), MUON, "bf16", 4, 32, {}),
    # AdaPNM (two momenta through the same codecs; the second-moment EMA and the clip as Adakaon's)
    "adapnm_int8_none": ("AdaPNM", dict(lr=1e-4, momentum_dtype="int8", bf16_method="none"), SMALL, "bf16", 6, 40, {}),
    "adapnm_4bit_wd_f32": ("AdaPNM", dict(lr=1e-4, betas=(0.9, 0.999), beta0=1.0, weight_decay=0.1, momentum_dtype="4bit"), SMALL, "f32", 5, 41, {}),
    "adapnm_bf16m_sr": ("AdaPNM", dict(lr=1e-4), SMALL, "bf16", 4, 42, {}),
    "adapnm_f32m_ams_nocautious": ("AdaPNM", dict(lr=1e-4, eps=1e-6, momentum_dtype="float32", ams_bound=True, cautious=False, gradient_centralization=False, weight_decay=0.05, bf16_method="none"), SMALL, "bf16", 5, 43, {}),
    "adapnm_int8_kahan": ("AdaPNM", dict(lr=1e-4, momentum_dtype="int8", bf16_method="kahan", clip_threshold=0.5), SMALL, "bf16", 5, 44, {}),
    "adapnm_4bit_outlier": ("AdaPNM", dict(lr=1e-4, momentum_dtype="4bit", bf16_method="none"), SMALL, "bf16", 5, 45, {"outlier": True}),
    # KProdigy (two passes around one cross-tensor scalar, the distance estimate d)
    "kprodigy_default": ("KProdigy", dict(), SMALL, "bf16", 10, 50, {"correlated": True}),
    "kprodigy_4bit_factored_slice_cautious": ("KProdigy", dict(momentum_dtype="4bit", second_moment="factored", slice_p=3, cautious=True, weight_decay=0.01, bf16_method="none"), SMALL, "bf16", 10, 51, {"correlated": True}),
    "kprodigy_int8_wd_f32": ("KProdigy", dict(momentum_dtype="int8", weight_decay=0.05, d_coef=2.0), SMALL, "f32", 10, 52, {"correlated": True}),
    "kprodigy_f32m_nogc_bias_safeguard": ("KProdigy", dict(momentum_dtype="float32", gradient_centralization=False, use_bias_correction=True, safeguard_warmup=True, growth_rate=1.5, d0=1e-5, bf16_method="none"), SMALL, "bf16", 10, 53, {"correlated": True}),
    "kprodigy_nomomentum_coupled_wd": ("KProdigy", dict(betas=(0.0, 0.99), weight_decay=0.02, decouple=False, d_update_freq=2, bf16_method="none"), SMALL, "bf16", 10, 54, {"correlated": True}),
    "kprodigy_int8_kahan": ("KProdigy", dict(momentum_dtype="int8", bf16_method="kahan", cautious=True), SMALL, "bf16", 10, 55, {"correlated": True}),
    # C1 at full size (the CPU-runnable correctness workload); big tensors stored strided
    "c1_full": ("Adakaon", dict(lr=1e-4, betas=(0.9, 0.999), momentum_dtype="int8", bf16_method="stochastic_rounding"), C1, "bf16", 10, 0, {"store_inputs": False, "sample": 257}),
}
