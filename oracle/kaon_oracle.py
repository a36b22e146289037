"""ctypes front end of the CPU oracle (oracle/kaon_oracle.c).

TEST INFRASTRUCTURE ONLY: imported by tests/, by ``__graft_entry__.smoke()`` as the checker and by
``bench.py``'s CPU-baseline legs.  The shipped package never imports this module.

Arrays are numpy.  bf16 tensors travel as ``np.uint16`` bit patterns; fp32 as ``np.float32``.
``OracleOptimizer`` subclasses keep per-tensor state in the reference's ``state_dict`` layout
(``m``, ``m_scale``, ``row``, ``col``, ``v``; reference src/kaon/_momentum_codec.py:293-360,
src/kaon/adakaon.py:318-335) so tests can compare state key by key.
"""
from __future__ import annotations

import ctypes as C
import math
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libkaon_oracle.so")

F32, BF16 = 0, 1
M_F32, M_BF16, M_INT8, M_4BIT = 0, 1, 2, 3
W_NONE, W_SR, W_SR_NOISE, W_KAHAN = 0, 1, 2, 3
MKIND = {"float32": M_F32, "bfloat16": M_BF16, "int8": M_INT8, "4bit": M_4BIT}
METHOD = {"none": W_NONE, "stochastic_rounding": W_SR}

_lib = None


def build(force: bool = False) -> str:
    """Compile the C oracle with the committed Makefile (gcc, OpenMP)."""
    src = os.path.join(_HERE, "kaon_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-B", "libkaon_oracle.so"],
                              stdout=subprocess.DEVNULL)
    return _SO


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_SO)
        _lib.ko_lion_step.restype = C.c_int
        _lib.ko_adakaon_step.restype = C.c_int
        _lib.ko_adamuon_step.restype = C.c_int
        _lib.ko_msam_apply.restype = C.c_int
        _lib.ko_newton_schulz.restype = C.c_int
        _lib.ko_cautious.restype = C.c_int64
    return _lib


def _p(a):
    if a is None:
        return C.c_void_p(0)
    assert a.flags["C_CONTIGUOUS"]
    return C.c_void_p(a.ctypes.data)


def _dt(a) -> int:
    if a.dtype == np.uint16:
        return BF16
    if a.dtype == np.float32:
        return F32
    raise TypeError(f"oracle arrays are uint16 (bf16 bits) or float32, got {a.dtype}")


# ----------------------------------------------------------------------------- bf16 helpers

def bf16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    return (a.astype(np.uint32) << 16).view(np.float32)


def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even fp32 -> bf16 bit patterns (finite inputs)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    u = u + 0x7FFF + ((u >> 16) & 1)
    return (u >> 16).astype(np.uint16)


def as_f32(a: np.ndarray) -> np.ndarray:
    return bf16_bits_to_f32(a) if a.dtype == np.uint16 else a.astype(np.float32)


# ----------------------------------------------------------------------------- primitives

def philox4x32(ctr, key) -> np.ndarray:
    c = (C.c_uint32 * 4)(*ctr)
    k = (C.c_uint32 * 2)(*key)
    o = (C.c_uint32 * 4)()
    lib().ko_philox4x32(c, k, o)
    return np.array(list(o), dtype=np.uint32)


def sr_noise(seed: int, step: int, tensor_id: int, tag: int, n: int) -> np.ndarray:
    out = np.empty(n, np.uint16)
    lib().ko_sr_noise_fill(C.c_uint64(seed), C.c_uint32(step), C.c_uint32(tensor_id),
                           C.c_uint32(tag), C.c_int64(n), _p(out))
    return out


def centralize(g: np.ndarray, rows: int) -> np.ndarray:
    n = g.size
    out = np.empty(n, np.float32)
    lib().ko_centralize(_p(g), _dt(g), C.c_int64(rows), C.c_int64(n // rows), _p(out))
    return out


def encode_int8(m: np.ndarray, rows: int):
    m = np.ascontiguousarray(m, np.float32).reshape(-1)
    codes = np.empty(m.size, np.int8)
    scale = np.empty(max(rows, 1), np.float32)
    lib().ko_encode_int8(_p(m), C.c_int64(m.size), C.c_int64(rows), _p(codes), _p(scale))
    return codes, scale


def decode_int8(codes: np.ndarray, scale: np.ndarray, rows: int) -> np.ndarray:
    out = np.empty(codes.size, np.float32)
    lib().ko_decode_int8(_p(codes), _p(scale), C.c_int64(codes.size), C.c_int64(rows), _p(out))
    return out


def encode_4bit(m: np.ndarray, block: int = 128):
    m = np.ascontiguousarray(m, np.float32).reshape(-1)
    n = m.size
    bs = fourbit_block(n, block)
    packed = np.empty((n + 1) // 2, np.uint8)
    scale = np.empty((n + bs - 1) // bs, np.float32)
    lib().ko_encode_4bit(_p(m), C.c_int64(n), C.c_int64(bs), _p(packed), _p(scale))
    return packed, scale


def decode_4bit(packed: np.ndarray, scale: np.ndarray, n: int, block: int = 128) -> np.ndarray:
    out = np.empty(n, np.float32)
    lib().ko_decode_4bit(_p(packed), _p(scale), C.c_int64(n), C.c_int64(fourbit_block(n, block)),
                         _p(out))
    return out


def fourbit_block(numel: int, block: int) -> int:
    """reference src/kaon/_momentum_codec.py:192-200"""
    if block <= 0:
        return numel
    return min(block, numel) if numel > 0 else 1


def newton_schulz(m: np.ndarray, steps: int) -> np.ndarray:
    m = np.ascontiguousarray(m, np.float32)
    R, Cc = m.shape
    out = np.empty_like(m)
    rc = lib().ko_newton_schulz(_p(m), C.c_int64(R), C.c_int64(Cc), C.c_int(steps), _p(out))
    assert rc == 0
    return out


def write(p: np.ndarray, delta: np.ndarray, alpha: float, method: int, seed=0, step=0, tensor_id=0,
          tag=0, noise=None) -> None:
    delta = np.ascontiguousarray(delta, np.float32).reshape(-1)
    lib().ko_write(_p(p), _dt(p), _p(delta), C.c_int64(p.size), C.c_float(alpha), C.c_int(method),
                   C.c_uint64(seed), C.c_uint32(step), C.c_uint32(tensor_id), C.c_uint32(tag),
                   _p(noise))


# ----------------------------------------------------------------------------- per-tensor state

class OracleTensor:
    """One parameter tensor with its optimizer state, in the reference's state layout."""

    def __init__(self, p: np.ndarray, shape):
        self.shape = tuple(int(s) for s in shape)
        self.p = np.ascontiguousarray(p).reshape(-1).copy()
        self.n = self.p.size
        self.rows = self.shape[0] if len(self.shape) >= 2 else 0
        self.cols = self.n // self.rows if self.rows else self.n
        self.state: dict = {}

    def init_momentum(self, md: str, block: int, key: str = "m") -> None:
        """reference src/kaon/_momentum_codec.py:263-264, 295-301, 350-360 (AdaPNM's two buffers,
        keys "m_pos" / "m_neg": src/kaon/adapnm.py:451-480)"""
        st = self.state
        if md == "int8":
            st[key] = np.zeros(self.n, np.int8)
            st[f"{key}_scale"] = np.ones(max(self.rows, 1), np.float32)
        elif md == "4bit":
            bs = fourbit_block(self.n, block)
            st[key] = np.full((self.n + 1) // 2, 0x88, np.uint8)
            st[f"{key}_scale"] = np.ones((self.n + bs - 1) // bs, np.float32)
            st[f"{key}_numel"], st[f"{key}_block"] = self.n, bs
        elif md == "bfloat16":
            st[key] = np.zeros(self.n, np.uint16)
        else:
            st[key] = np.zeros(self.n, np.float32)

    def init_second_moment(self) -> None:
        """reference src/kaon/adakaon.py:318-331"""
        if self.rows:
            self.state["row"] = np.zeros(self.rows, np.float32)
            self.state["col"] = np.zeros(self.cols, np.float32)
        else:
            self.state["v"] = np.zeros(self.n, np.float32)

    def block(self) -> int:
        return int(self.state.get("m_block", self.state.get("m_pos_block", 128)))

    def decoded_m(self, md: str) -> np.ndarray:
        st = self.state
        if md == "int8":
            return decode_int8(st["m"], st["m_scale"], self.rows)
        if md == "4bit":
            return decode_4bit(st["m"], st["m_scale"], self.n, st["m_block"])
        return as_f32(st["m"]).copy()


class OracleOptimizer:
    def __init__(self, params, shapes, *, seed: int = 0, **hp):
        self.hp = dict(self.DEFAULTS)
        unknown = set(hp) - set(self.hp)
        if unknown:
            raise TypeError(f"unknown hyper-parameters {sorted(unknown)}")
        self.hp.update(hp)
        self.tensors = [OracleTensor(p, s) for p, s in zip(params, shapes)]
        self.seed = seed
        self.t = 0  # number of completed steps; the SR stream uses the 1-based step index
        self.kept: list[int] = []

    def _lazy_init(self, t: OracleTensor) -> None:
        raise NotImplementedError

    def _method(self, t: OracleTensor, noise=None) -> int:
        """Weight-write mode of this step call; for the Kahan write also hands the tensor's shift buffer
        (state["shift"], bf16 bits; reference src/kaon/lion.py:240-241) to the C side."""
        if noise is not None:
            return W_SR_NOISE
        m = self.hp["bf16_method"]
        if m != "kahan":
            return METHOD[m]
        if t.p.dtype != np.uint16:
            return W_NONE  # fp32 weights: plain subtract
        if "shift" not in t.state:
            t.state["shift"] = np.zeros(t.n, np.uint16)
        lib().ko_set_kahan_shift(_p(t.state["shift"]))
        return W_KAHAN

    def _args_common(self, t: OracleTensor, g: np.ndarray):
        hp = self.hp
        st = t.state
        return (_p(t.p), _p(np.ascontiguousarray(g).reshape(-1)), _dt(t.p), C.c_int64(t.n),
                C.c_int64(t.rows), C.c_int(MKIND[hp["momentum_dtype"]]), _p(st.get("m")),
                _p(st.get("m_scale")), C.c_int64(t.block()))


class OracleLion(OracleOptimizer):
    """reference src/kaon/lion.py:152-171 (defaults), :322-352 (step)"""
    DEFAULTS = dict(lr=1e-4, betas=(0.9, 0.99), weight_decay=0.0, momentum_dtype="bfloat16",
                    momentum_4bit_block=128, cautious=True, gradient_centralization=True,
                    bf16_method="stochastic_rounding")

    def _lazy_init(self, t):
        if not t.state:
            t.init_momentum(self.hp["momentum_dtype"], self.hp["momentum_4bit_block"])

    def step(self, grads, noises=None):
        hp = self.hp
        self.t += 1
        self.kept = []
        for tid, (t, g) in enumerate(zip(self.tensors, grads)):
            if g is None:
                self.kept.append(-1)
                continue
            self._lazy_init(t)
            kept = C.c_int64(-1)
            noise = None if noises is None else noises[tid]
            method = self._method(t, noise)
            rc = lib().ko_lion_step(
                *self._args_common(t, g), C.c_double(hp["lr"]), C.c_double(hp["betas"][0]),
                C.c_double(hp["betas"][1]), C.c_double(hp["weight_decay"]),
                C.c_int(bool(hp["cautious"])), C.c_int(bool(hp["gradient_centralization"])),
                C.c_int(method), C.c_uint64(self.seed), C.c_uint32(self.t), C.c_uint32(tid),
                _p(noise), C.byref(kept))
            assert rc == 0
            self.kept.append(kept.value)


class OracleAdakaon(OracleOptimizer):
    """reference src/kaon/adakaon.py:195-218 (defaults), :339-383 (step)"""
    DEFAULTS = dict(lr=1e-3, betas=(0.9, 0.999), eps=(1e-30, 1e-3), weight_decay=0.0,
                    clip_threshold=1.0, momentum_dtype="bfloat16", momentum_4bit_block=128,
                    cautious=True, gradient_centralization=True,
                    bf16_method="stochastic_rounding")

    def _lazy_init(self, t):
        if not t.state:
            t.init_second_moment()
            if self.hp["betas"][0] > 0:
                t.init_momentum(self.hp["momentum_dtype"], self.hp["momentum_4bit_block"])

    def step(self, grads, noises=None, _advance=True):
        hp = self.hp
        if _advance:
            self.t += 1
        self.kept, self.rms = [], []
        for tid, (t, g) in enumerate(zip(self.tensors, grads)):
            if g is None:
                self.kept.append(-1)
                self.rms.append(float("nan"))
                continue
            self._lazy_init(t)
            st = t.state
            kept, rms = C.c_int64(-1), C.c_float(0)
            noise = None if noises is None else noises[tid]
            method = self._method(t, noise)
            rc = lib().ko_adakaon_step(
                *self._args_common(t, g), _p(st["row"] if t.rows else st["v"]),
                _p(st["col"] if t.rows else None), C.c_double(hp["lr"]),
                C.c_double(hp["betas"][0]), C.c_double(hp["betas"][1]), C.c_double(hp["eps"][0]),
                C.c_double(hp["weight_decay"]), C.c_double(hp["clip_threshold"]),
                C.c_int(bool(hp["cautious"])), C.c_int(bool(hp["gradient_centralization"])),
                C.c_int(method), C.c_uint64(self.seed), C.c_uint32(self.t), C.c_uint32(tid),
                _p(noise), C.byref(kept), C.byref(rms))
            assert rc == 0
            self.kept.append(kept.value)
            self.rms.append(rms.value)


class OracleAdaPNM(OracleOptimizer):
    """reference src/kaon/adapnm.py:344-366 (defaults), :599-620 (step), :1209-1273 (one tensor)"""
    DEFAULTS = dict(lr=1e-3, betas=(0.8, 0.999), beta0=0.5, eps=1e-8, weight_decay=0.0,
                    clip_threshold=1.0, cautious=True, gradient_centralization=True, ams_bound=False,
                    momentum_dtype="bfloat16", momentum_4bit_block=128,
                    bf16_method="stochastic_rounding")

    def _lazy_init(self, t):
        if not t.state:
            t.init_second_moment()
            if not t.rows and self.hp["ams_bound"]:
                t.state["max_v"] = np.zeros(t.n, np.float32)
            t.init_momentum(self.hp["momentum_dtype"], self.hp["momentum_4bit_block"], "m_pos")
            t.init_momentum(self.hp["momentum_dtype"], self.hp["momentum_4bit_block"], "m_neg")

    def step(self, grads, noises=None):
        hp = self.hp
        self.t += 1
        pos, neg = ("m_pos", "m_neg") if self.t % 2 == 1 else ("m_neg", "m_pos")  # adapnm.py:588-596
        self.kept, self.rms = [], []
        for tid, (t, g) in enumerate(zip(self.tensors, grads)):
            if g is None:
                self.kept.append(-1)
                self.rms.append(float("nan"))
                continue
            self._lazy_init(t)
            st = t.state
            kept, rms = C.c_int64(-1), C.c_float(0)
            noise = None if noises is None else noises[tid]
            method = self._method(t, noise)
            rc = lib().ko_adapnm_step(
                _p(t.p), _p(np.ascontiguousarray(g).reshape(-1)), _dt(t.p), C.c_int64(t.n), C.c_int64(t.rows),
                C.c_int(MKIND[hp["momentum_dtype"]]), _p(st[pos]), _p(st.get(f"{pos}_scale")), _p(st[neg]),
                _p(st.get(f"{neg}_scale")), C.c_int64(t.block()),
                _p(st["row"] if t.rows else st["v"]), _p(st["col"] if t.rows else None), _p(st.get("max_v")),
                C.c_double(hp["lr"]), C.c_double(hp["betas"][0]), C.c_double(hp["betas"][1]),
                C.c_double(hp["beta0"]), C.c_double(hp["eps"]), C.c_double(hp["weight_decay"]),
                C.c_double(hp["clip_threshold"]), C.c_int(bool(hp["cautious"])),
                C.c_int(bool(hp["gradient_centralization"])), C.c_int(bool(hp["ams_bound"])), C.c_int(method),
                C.c_uint32(self.t), C.c_uint64(self.seed), C.c_uint32(self.t), C.c_uint32(tid), _p(noise),
                C.byref(kept), C.byref(rms))
            assert rc == 0
            self.kept.append(kept.value)
            self.rms.append(rms.value)


class OracleKProdigy(OracleOptimizer):
    """reference src/kaon/kprodigy.py:151-236 (defaults), :299-404 (step: the distance estimate d between two
    passes over the tensors), :417-478 (pass 1), :800-840 (pass 2).  One parameter group."""
    DEFAULTS = dict(lr=1.0, betas=(0.9, 0.999), beta3=None, eps=1e-8, weight_decay=0.0, decouple=True,
                    use_bias_correction=False, safeguard_warmup=False, d0=1e-6, d_coef=1.0,
                    growth_rate=float("inf"), d_update_freq=1, slice_p=1, momentum_dtype="bfloat16",
                    momentum_4bit_block=128, second_moment="full", eps_factored=1e-30, cautious=False,
                    gradient_centralization=True, bf16_method="stochastic_rounding")

    def __init__(self, params, shapes, *, seed: int = 0, **hp):
        super().__init__(params, shapes, seed=seed, **hp)
        d0 = self.hp["d0"]
        self.group = {"d": d0, "d0": d0, "d_max": d0, "d_numerator": 0.0, "k": 0, "d_hat": None}

    def _lazy_init(self, t):
        if t.state:
            return
        hp = self.hp
        sp = hp["slice_p"]
        sliced = as_f32(t.p)[::sp].astype(np.float32)
        t.state["step"] = 0
        t.state["s"] = np.zeros(sliced.size, np.float32)
        # the reference keeps a 0-dim zero when the sliced weights are all zero (kprodigy.py:277-280)
        t.state["p0"] = sliced.copy() if float(np.linalg.norm(sliced.astype(np.float64))) > 0 else np.zeros((), np.float32)
        if hp["betas"][0] > 0:
            t.init_momentum(hp["momentum_dtype"], hp["momentum_4bit_block"])
        if hp["second_moment"] == "factored" and t.rows:
            t.state["row"] = np.zeros(t.rows, np.float32)
            t.state["col"] = np.zeros(t.cols, np.float32)
        else:
            t.state["v"] = np.zeros(t.n, np.float32)

    def step(self, grads, noises=None):
        hp, grp = self.hp, self.group
        self.t += 1
        beta1, beta2 = hp["betas"]
        beta3 = hp["beta3"] if hp["beta3"] is not None else math.sqrt(beta2)
        k, d, d0, lr = grp["k"], grp["d"], grp["d0"], hp["lr"]
        bc = ((1 - beta2 ** (k + 1)) ** 0.5) / (1 - beta1 ** (k + 1)) if hp["use_bias_correction"] else 1.0
        dlr = d * lr * bc
        should = (k % hp["d_update_freq"]) == 0
        d_over_d0 = d / d0
        d_numerator = grp["d_numerator"] * beta3
        alpha_s = (d_over_d0 * d) if hp["safeguard_warmup"] else (d_over_d0 * dlr)
        factored = hp["second_moment"] == "factored"
        wd = hp["weight_decay"]
        mk = MKIND[hp["momentum_dtype"]] if beta1 > 0 else MKIND["float32"]
        do_d = bool(lr > 0.0 and should)
        delta_num = np.float32(0.0)
        d_den = np.float32(0.0)
        const = d_over_d0 * dlr
        active = []
        for tid, (t, g) in enumerate(zip(self.tensors, grads)):
            if g is None:
                continue
            self._lazy_init(t)
            st = t.state
            active.append((tid, t, g))
            num, den = C.c_float(0), C.c_float(0)
            fac = factored and bool(t.rows)
            p0 = st["p0"] if st["p0"].ndim else None
            rc = lib().ko_kprodigy_pass1(
                _p(t.p), _p(np.ascontiguousarray(g).reshape(-1)), _dt(t.p), C.c_int64(t.n), C.c_int64(t.rows),
                C.c_int(mk), _p(st.get("m")), _p(st.get("m_scale")), C.c_int64(t.block()),
                _p(st["row"] if fac else st["v"]), _p(st["col"] if fac else None), C.c_int(fac), _p(st["s"]), _p(p0),
                C.c_int64(hp["slice_p"]), C.c_int(do_d), C.c_double(beta1), C.c_double(beta2), C.c_double(beta3),
                C.c_double(d), C.c_double(alpha_s), C.c_double(wd if (wd != 0 and not hp["decouple"]) else 0.0),
                C.c_double(hp["eps_factored"]), C.c_int(bool(hp["gradient_centralization"])),
                C.byref(num), C.byref(den))
            assert rc == 0
            if do_d:   # the fp32 left fold of the reference (kprodigy.py:451, 455, 580-588)
                delta_num = np.float32(delta_num + np.float32(np.float32(num.value) * np.float32(const)))
                d_den = np.float32(d_den + np.float32(den.value))
        if should and lr > 0.0 and active and float(d_den) > 0.0:
            global_num = d_numerator + float(delta_num)
            d_hat = hp["d_coef"] * global_num / float(d_den)
            d_new, d_max = d, grp["d_max"]
            if d_new == d0:
                d_new = max(d_new, d_hat)
            d_max = max(d_max, d_hat)
            d_new = min(d_max, d_new * hp["growth_rate"])
            grp.update(d_numerator=global_num, d=d_new, d_max=d_max, d_hat=d_hat)
            d = d_new   # pass 2 takes the NEW d for its denominator with the OLD dlr (kprodigy.py:379-403)
        self.kept = [-1] * len(self.tensors)
        for tid, t, g in active:
            st = t.state
            st["step"] += 1
            fac = factored and bool(t.rows)
            kept = C.c_int64(-1)
            noise = None if noises is None else noises[tid]
            method = self._method(t, noise)
            rc = lib().ko_kprodigy_pass2(
                _p(t.p), _p(np.ascontiguousarray(g).reshape(-1)), _dt(t.p), C.c_int64(t.n), C.c_int64(t.rows),
                C.c_int(mk), _p(st.get("m")), _p(st.get("m_scale")), C.c_int64(t.block()),
                _p(st["row"] if fac else st["v"]), _p(st["col"] if fac else None), C.c_int(fac), C.c_int(beta1 > 0),
                C.c_double(d), C.c_double(dlr), C.c_double(hp["eps"]),
                C.c_double(wd * dlr if (wd != 0 and hp["decouple"]) else 0.0), C.c_int(bool(hp["cautious"])),
                C.c_int(bool(hp["gradient_centralization"])), C.c_int(method), C.c_uint64(self.seed),
                C.c_uint32(self.t), C.c_uint32(tid), _p(noise), C.byref(kept))
            assert rc == 0
            self.kept[tid] = kept.value
        grp["k"] += 1


class OracleNekaon(OracleAdakaon):
    """reference src/kaon/nekaon.py:122-185 over src/kaon/msam.py:374-406 with norm="none".

    SR stream tags: 0 = the inner update, 1 = removal of the previous climb, 2 = the new climb,
    3 = eval() removal, 4 = train() restore.
    """
    DEFAULTS = dict(OracleAdakaon.DEFAULTS, lr=1e-3, betas=(0.5, 0.999), weight_decay=0.1,
                    momentum_dtype="4bit", k=1.5)

    def __init__(self, params, shapes, **hp):
        super().__init__(params, shapes, **hp)
        self.has_e = False
        self.train_mode = True
        self.bound = None

    def _apply(self, sign: float, tag: int):
        hp = self.hp
        rho = -float(hp["k"])
        if sign > 0 and self.bound is None:
            self.bound = abs(rho) * hp["clip_threshold"] * hp["lr"]  # msam.py:169-188
        for tid, t in enumerate(self.tensors):
            st = t.state
            if "m" not in st:
                continue
            rc = lib().ko_msam_apply(
                _p(t.p), _dt(t.p), C.c_int64(t.n), C.c_int64(t.rows),
                C.c_int(MKIND[hp["momentum_dtype"]]), _p(st["m"]), _p(st.get("m_scale")),
                C.c_int64(t.block()), C.c_double(sign * rho), C.c_double(self.bound),
                C.c_int(W_SR), C.c_uint64(self.seed), C.c_uint32(self.t), C.c_uint32(tid),
                C.c_uint32(tag), _p(None))
            assert rc == 0

    def step(self, grads, noises=None):
        if not self.train_mode:
            raise RuntimeError("step() outside train mode")
        self.t += 1  # removal, update and climb of one step() share its step index in the SR stream
        if self.has_e:
            self._apply(-1.0, 1)
            self.has_e = False
        self.bound = None
        super().step(grads, noises, _advance=False)
        if self.hp["k"] != 0.0 and any("m" in t.state for t in self.tensors):
            self._apply(+1.0, 2)
            self.has_e = True

    def eval(self):
        if self.train_mode and self.has_e:
            self._apply(-1.0, 3)
        self.train_mode = False

    def train(self):
        if not self.train_mode and self.has_e:
            self._apply(+1.0, 4)
        self.train_mode = True


class OracleAdaMuon(OracleOptimizer):
    """reference src/kaon/adamuon.py:216-239 (defaults), :327-352 (step)"""
    DEFAULTS = dict(lr=2e-2, betas=(0.95, 0.999), eps=(1e-30, 1e-3), weight_decay=0.0, ns_steps=2,
                    clip_threshold=1.0, momentum_dtype="bfloat16", momentum_4bit_block=128,
                    cautious=True, gradient_centralization=False,
                    bf16_method="stochastic_rounding")

    _lazy_init = OracleAdakaon._lazy_init

    def step(self, grads, ns_override=None, capture_ns_in=False):
        hp = self.hp
        self.t += 1
        self.ns_in = []
        for tid, (t, g) in enumerate(zip(self.tensors, grads)):
            if g is None:
                self.ns_in.append(None)
                continue
            self._lazy_init(t)
            st = t.state
            ns_in = np.empty(t.n, np.float32) if (capture_ns_in and t.rows) else None
            ov = None
            if ns_override is not None and ns_override[tid] is not None:
                ov = np.ascontiguousarray(ns_override[tid], np.float32).reshape(-1)
            rc = lib().ko_adamuon_step(
                *self._args_common(t, g), _p(st["row"] if t.rows else st["v"]),
                _p(st["col"] if t.rows else None), C.c_double(hp["lr"]),
                C.c_double(hp["betas"][0]), C.c_double(hp["betas"][1]), C.c_double(hp["eps"][0]),
                C.c_double(hp["weight_decay"]), C.c_double(hp["clip_threshold"]),
                C.c_int(hp["ns_steps"]), C.c_int(bool(hp["cautious"])),
                C.c_int(bool(hp["gradient_centralization"])), C.c_int(self._method(t)),
                C.c_uint64(self.seed), C.c_uint32(self.t), C.c_uint32(tid), _p(None), _p(ns_in),
                _p(ov))
            assert rc == 0
            self.ns_in.append(ns_in)


def cosine_lr(t: int, total: int, hi: float, lo: float) -> float:
    return lo + 0.5 * (hi - lo) * (1.0 + math.cos(math.pi * t / total))
