"""ctypes binding of libkaon_b200.so (the C ABI declared in include/kaon_b200.h).

There is no CPU fallback: if the library is missing or a call fails, this raises.
"""
from __future__ import annotations

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "libkaon_b200.so")

DT_F32, DT_BF16 = 0, 1
M_F32, M_BF16, M_INT8, M_4BIT, M_NONE = 0, 1, 2, 3, 4
W_NONE, W_SR, W_KAHAN = 0, 1, 2
OPT_LION, OPT_ADAKAON, OPT_ADAMUON, OPT_ADAPNM, OPT_KPRODIGY = 0, 1, 2, 3, 4
TAG_UPDATE, TAG_REMOVE, TAG_CLIMB, TAG_EVAL, TAG_TRAIN = 0, 1, 2, 3, 4
MOMENTUM_KIND = {"float32": M_F32, "bfloat16": M_BF16, "int8": M_INT8, "4bit": M_4BIT}
BF16_METHOD = {"none": W_NONE, "stochastic_rounding": W_SR, "kahan": W_KAHAN}


class TensorDesc(C.Structure):
    _fields_ = [("p", C.c_void_p), ("g", C.c_void_p), ("m", C.c_void_p), ("m_scale", C.c_void_p),
                ("stat_a", C.c_void_p), ("stat_b", C.c_void_p), ("numel", C.c_int64),
                ("rows", C.c_int64), ("tensor_id", C.c_uint32), ("block", C.c_uint32),
                ("shift", C.c_void_p)]


class LionHParams(C.Structure):
    _fields_ = [("lr", C.c_double), ("beta1", C.c_double), ("beta2", C.c_double),
                ("weight_decay", C.c_double), ("cautious", C.c_int32),
                ("gradient_centralization", C.c_int32), ("bf16_method", C.c_int32),
                ("reserved", C.c_int32)]


class AdakaonHParams(C.Structure):
    _fields_ = [("lr", C.c_double), ("beta1", C.c_double), ("beta2", C.c_double),
                ("eps1", C.c_double), ("weight_decay", C.c_double), ("clip_threshold", C.c_double),
                ("cautious", C.c_int32), ("gradient_centralization", C.c_int32),
                ("bf16_method", C.c_int32), ("reserved", C.c_int32),
                ("msam_remove", C.c_int32), ("msam_climb", C.c_int32),
                ("msam_alpha_remove", C.c_double), ("msam_bound_remove", C.c_double),
                ("msam_alpha_climb", C.c_double), ("msam_bound_climb", C.c_double)]


class AdaMuonHParams(C.Structure):
    _fields_ = [("lr", C.c_double), ("beta1", C.c_double), ("beta2", C.c_double),
                ("eps1", C.c_double), ("weight_decay", C.c_double), ("clip_threshold", C.c_double),
                ("ns_steps", C.c_int32), ("cautious", C.c_int32),
                ("gradient_centralization", C.c_int32), ("bf16_method", C.c_int32)]


class AdaPNMHParams(C.Structure):
    _fields_ = [("lr", C.c_double), ("beta1", C.c_double), ("beta2", C.c_double), ("beta0", C.c_double),
                ("eps", C.c_double), ("weight_decay", C.c_double), ("clip_threshold", C.c_double),
                ("cautious", C.c_int32), ("gradient_centralization", C.c_int32), ("ams_bound", C.c_int32),
                ("bf16_method", C.c_int32), ("group_step", C.c_uint32), ("reserved", C.c_uint32)]


class KProdigyPass1(C.Structure):
    _fields_ = [("beta1", C.c_double), ("beta2", C.c_double), ("beta3", C.c_double), ("d", C.c_double),
                ("alpha_s", C.c_double), ("weight_decay_coupled", C.c_double), ("eps_factored", C.c_double),
                ("do_d", C.c_int32), ("gradient_centralization", C.c_int32), ("factored", C.c_int32),
                ("reserved", C.c_int32)]


class KProdigyPass2(C.Structure):
    _fields_ = [("d", C.c_double), ("dlr", C.c_double), ("eps", C.c_double), ("decay_dlr", C.c_double),
                ("cautious", C.c_int32), ("gradient_centralization", C.c_int32), ("factored", C.c_int32),
                ("bf16_method", C.c_int32)]


class KaonError(RuntimeError):
    pass


_lib = None


def lib() -> C.CDLL:
    """Load the CUDA library; fail loudly if it has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise KaonError(
                f"{LIB_PATH} is missing: build it with `python -m kaon_b200._build` (nvcc, sm_100a). "
                "kaon_b200 has no CPU or eager fallback.")
        _lib = C.CDLL(LIB_PATH)
        _lib.kaon_last_error.restype = C.c_char_p
        _lib.kaon_plan_device_bytes.restype = C.c_int64
        _lib.kaon_plan_launch_count.restype = C.c_int64
        _lib.kaon_adamuon_workspace_bytes.restype = C.c_int64
        _lib.kaon_adamuon_workspace_bytes.argtypes = [C.c_void_p]
        _lib.kaon_adamuon_signal_offset.restype = C.c_int64
        _lib.kaon_adamuon_signal_offset.argtypes = [C.c_void_p, C.c_int]
        _lib.kaon_newton_schulz_workspace_bytes.restype = C.c_int64
        _lib.kaon_plan_device_bytes.argtypes = [C.c_void_p]
        _lib.kaon_plan_launch_count.argtypes = [C.c_void_p]
        _lib.kaon_plan_set_peers.argtypes = [C.c_void_p, C.POINTER(C.c_int64), C.c_int]
        if _lib.kaon_abi_version() != 2:
            raise KaonError("libkaon_b200.so ABI version mismatch")
    return _lib


def check(rc: int) -> None:
    if rc != 0:
        msg = lib().kaon_last_error().decode("utf-8", "replace")
        if rc == -2:
            raise NotImplementedError(msg)
        raise KaonError(f"libkaon_b200 error {rc}: {msg}")
