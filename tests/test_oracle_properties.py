"""Size-independent properties of the CPU oracle's building blocks, at sizes far above the golden vectors':
what a codec, the centralization and the stochastic-rounding write must satisfy whatever the input."""
import numpy as np
import pytest

import kaon_oracle as ko


def _heavy_tailed(rng, n, scale=1e-3):
    x = rng.standard_normal(n).astype(np.float32) * scale
    x[rng.random(n) < 0.01] *= 100.0          # the 1 % outliers of the benchmark's gradient distribution
    return x


@pytest.mark.parametrize("rows,cols", [(1, 1), (3, 5), (640, 1280), (4000, 1), (0, 300001)])
def test_int8_codec_round_trip_and_idempotence(rows, cols):
    rng = np.random.default_rng(rows * 7919 + cols)
    n = max(rows, 1) * cols
    x = _heavy_tailed(rng, n)
    if rows >= 3:
        x[cols:2 * cols] = 0.0                # an all-zero row: the absmax floor
    codes, scale = ko.encode_int8(x, rows)
    dec = ko.decode_int8(codes, scale, rows)
    per_elem = np.repeat(scale, cols) if rows else np.full(n, scale[0], np.float32)
    # every element within half a level of its row's scale (and one fp32 ulp of the product)
    assert np.all(np.abs(dec - x) <= per_elem * 0.5 * (1 + 1e-6) + 1e-30)
    assert np.all(np.abs(codes.astype(np.int32)) <= 127)
    # the row's largest element takes the last level
    if rows:
        amax_rows = np.abs(x.reshape(rows, cols)).max(axis=1)
        top = np.abs(codes.reshape(rows, cols).astype(np.int32)).max(axis=1)
        assert np.all(top[amax_rows > 1e-12] == 127)
    # encoding what was decoded gives the same codes and scales
    codes2, scale2 = ko.encode_int8(dec, rows)
    live = np.repeat(np.abs(codes.reshape(max(rows, 1), cols).astype(np.int32)).max(axis=1) == 127, cols)
    assert np.array_equal(codes2[live], codes[live])
    assert np.allclose(scale2, scale, rtol=1e-6, atol=1e-20)


@pytest.mark.parametrize("n,block", [(1, 128), (77, 128), (129, 128), (1 << 20, 128), (300001, 64), (50000, 256),
                                     (4096, 32), (999, 0)])
def test_4bit_codec_round_trip_and_idempotence(n, block):
    rng = np.random.default_rng(n + block)
    x = _heavy_tailed(rng, n)
    bs = ko.fourbit_block(n, block)
    if n > 2 * bs:
        x[bs:2 * bs] = 0.0                    # an all-zero block
    packed, scale = ko.encode_4bit(x, block)
    assert packed.size == (n + 1) // 2 and scale.size == (n + bs - 1) // bs
    dec = ko.decode_4bit(packed, scale, n, block)
    per_elem = np.repeat(scale, bs)[:n]
    assert np.all(np.abs(dec - x) <= per_elem * 0.5 * (1 + 1e-6) + 1e-30)
    nib = np.stack([packed & 15, packed >> 4], -1).reshape(-1)[:n].astype(np.int32) - 8
    assert nib.min() >= -7 and nib.max() <= 7
    packed2, scale2 = ko.encode_4bit(dec, block)
    live = np.repeat(np.array([np.abs(nib[b * bs:(b + 1) * bs]).max() == 7 for b in range(scale.size)]), bs)[:n]
    nib2 = np.stack([packed2 & 15, packed2 >> 4], -1).reshape(-1)[:n].astype(np.int32) - 8
    assert np.array_equal(nib2[live], nib[live])
    assert np.allclose(scale2, scale, rtol=1e-6, atol=1e-20)


@pytest.mark.parametrize("rows,cols,bf16", [(640, 1280, True), (333, 77, True), (48, 4100, False)])
def test_centralization_is_idempotent_up_to_rounding_and_kills_the_row_mean(rows, cols, bf16):
    rng = np.random.default_rng(rows + cols)
    x = (rng.standard_normal(rows * cols) * 1e-3 + 2e-4).astype(np.float32)
    g = ko.f32_to_bf16_bits(x) if bf16 else x
    out = ko.centralize(g, rows)                       # fp32 values (bf16-representable for bf16 input)
    means = out.reshape(rows, cols).astype(np.float64).mean(axis=1)
    tol = 2.0 ** -8 * 4e-3 if bf16 else 1e-9           # half a bf16 level of the largest entries
    assert np.abs(means).max() <= tol
    again = ko.centralize(ko.f32_to_bf16_bits(out) if bf16 else out, rows)
    assert np.abs(again - out).max() <= 2 * tol


def test_stochastic_rounding_write_is_unbiased_and_one_level_wide():
    n = 1 << 16
    rng = np.random.default_rng(5)
    p = ko.f32_to_bf16_bits((rng.standard_normal(n) * 0.02).astype(np.float32))
    d = (rng.standard_normal(n) * 1e-5).astype(np.float32)     # far below a bf16 level of p
    exact = ko.as_f32(p).astype(np.float64) - d
    acc = np.zeros(n, np.float64)
    steps = 64
    for step in range(1, steps + 1):
        q = p.copy()
        ko.write(q, d, -1.0, 1, seed=9, step=step, tensor_id=3)    # in place
        got = ko.as_f32(q).astype(np.float64)
        level = np.maximum(np.abs(ko.as_f32(p)), np.abs(exact)) * 2.0 ** -7 + 1e-30
        assert np.all(np.abs(got - exact) <= level)               # one of the two bf16 neighbours of the exact value
        acc += got
    # the mean over steps approaches the exact difference: error of the mean well below one level
    big = np.abs(ko.as_f32(p)) > 1e-3                             # the step is far below a level there
    level = np.abs(ko.as_f32(p)).astype(np.float64) * 2.0 ** -8
    z = ((acc / steps - exact) / (level / np.sqrt(steps)))[big]
    assert abs(z.mean()) < 0.05 and z.std() < 1.5
