"""Helpers shared by the tests: golden-fixture access and oracle drivers."""
from __future__ import annotations

import ast
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


class Fixture:
    """One ``tests/golden/<name>.npz`` written by tests/golden/make_golden.py."""

    def __init__(self, name: str):
        self.name = name
        self.z = np.load(os.path.join(GOLDEN, f"{name}.npz"))
        if "meta_shapes" in self.z:
            self.shapes = [ast.literal_eval(str(s)) for s in self.z["meta_shapes"]]
            self.steps = int(self.z["meta_steps"])
            self.seed = int(self.z["meta_seed"])
            self.bf16 = "bfloat16" in str(self.z["meta_dtype"])
            self.outlier = bool(self.z["meta_outlier"])

    def __getitem__(self, k):
        return self.z[k]

    def __contains__(self, k):
        return k in self.z

    def params(self):
        return [self.z[f"p_in_t{i}"] for i in range(len(self.shapes))]

    def grads(self, step):
        return [self.z[f"g_s{step}_t{i}"] for i in range(len(self.shapes))]

    def weights(self, step, i):
        return self.z[f"p_s{step}_t{i}"]

    def state(self, step, i, key):
        k = f"st_s{step}_t{i}_{key}"
        return self.z[k] if k in self.z else None


def ulp_diff_bf16(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    """Distance in bf16 ulps between two uint16 bit-pattern arrays (sign-magnitude aware)."""
    def key(x):
        x = x.astype(np.int32)
        return np.where(x & 0x8000, -(x & 0x7FFF), x & 0x7FFF)
    return np.abs(key(a) - key(b))


def rel_err(a, b):
    a = np.asarray(a, np.float64)
    b = np.asarray(b, np.float64)
    return float(np.max(np.abs(a - b) / np.maximum(np.abs(b), 1e-30))) if a.size else 0.0


def sr_close(a_bits, b_bits, writes, step_mag):
    """Two bf16 weight arrays that went through ``writes`` independent stochastic roundings of the
    same exact updates differ by at most one bf16 ulp per write; the ulp is taken at the larger of
    the weight and the per-step displacement ``step_mag`` (a weight may cross zero)."""
    a = (a_bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    b = (b_bits.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    mag = np.maximum(np.maximum(np.abs(a), np.abs(b)), step_mag)
    return bool(np.all(np.abs(a - b) <= writes * mag * 2.0 ** -7))
