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


# ---- whole steps: properties the reference's tests hold its optimizers to, asked of the oracle ----

SHAPES = [(64, 96), (16, 8, 3, 3), (300,), (5, 7)]


def _f32(rng, shapes, scale):
    return [(rng.standard_normal(int(np.prod(s))) * scale).astype(np.float32) for s in shapes]


def test_lion_moves_every_weight_by_exactly_lr_against_the_sign():
    """reference tests/test_lion.py: without mask, decay and centralization the first update is
    -lr * sign(g) on every element with a non-zero gradient."""
    rng = np.random.default_rng(1)
    p0 = _f32(rng, SHAPES, 0.02)
    g = _f32(rng, SHAPES, 1e-3)
    opt = ko.OracleLion([p.copy() for p in p0], SHAPES, lr=1e-3, betas=(0.9, 0.99), momentum_dtype="float32",
                        cautious=False, gradient_centralization=False, bf16_method="none")
    opt.step(g)
    for t, a, gi in zip(opt.tensors, p0, g):
        want = a - np.float32(1e-3) * np.sign(gi)
        assert np.array_equal(t.p, want.astype(np.float32))
        assert np.allclose(t.state["m"], np.float32(0.01) * gi, rtol=1e-6, atol=0)      # (1 - beta2) * g


def test_lion_cautious_mask_rescales_by_the_kept_fraction():
    """With the mask on, weights whose update sign disagrees with the gradient stay, the others move by
    lr * numel / kept (reference src/kaon/lion.py:344-348)."""
    rng = np.random.default_rng(2)
    shapes = [(128, 64)]
    p0 = _f32(rng, shapes, 0.02)
    opt = ko.OracleLion([p.copy() for p in p0], shapes, lr=1e-3, betas=(0.9, 0.5), momentum_dtype="float32",
                        cautious=True, gradient_centralization=False, bf16_method="none")
    opt.step(_f32(rng, shapes, 1e-3))              # momentum = half the first gradient: it decides the next sign
    before = opt.tensors[0].p.copy()
    g2 = _f32(rng, shapes, 1e-3)                   # an independent gradient: about half the signs disagree
    opt.step(g2)
    moved = opt.tensors[0].p != before
    frac = moved.mean()
    assert 0.3 < frac < 0.9
    step = np.abs(opt.tensors[0].p - before)[moved]
    assert np.allclose(step, 1e-3 / frac, rtol=2e-3)


@pytest.mark.parametrize("md", ["float32", "int8", "4bit"])
def test_adakaon_first_step_does_not_depend_on_the_gradients_scale(md):
    """The factored second moment normalises the gradient: scaling every gradient by 64 leaves the first
    update unchanged (up to eps1 = 1e-30 and rounding)."""
    rng = np.random.default_rng(3)
    p0 = _f32(rng, SHAPES, 0.02)
    g = _f32(rng, SHAPES, 1e-3)
    outs = []
    for k in (1.0, 64.0):
        opt = ko.OracleAdakaon([p.copy() for p in p0], SHAPES, lr=1e-3, betas=(0.9, 0.999), momentum_dtype=md,
                               cautious=True, gradient_centralization=True, bf16_method="none")
        opt.step([gi * np.float32(k) for gi in g])
        outs.append([t.p.copy() for t in opt.tensors])
    for a, b, base in zip(outs[0], outs[1], p0):
        assert np.abs(a - base).max() > 0
        assert np.allclose(a - base, b - base, rtol=2e-2, atol=2e-6)


def test_zero_gradient_changes_nothing_but_decay():
    rng = np.random.default_rng(4)
    p0 = _f32(rng, SHAPES, 0.02)
    z = [np.zeros_like(p) for p in p0]
    for cls, kw in ((ko.OracleLion, dict(lr=1e-3, momentum_dtype="4bit")),
                    (ko.OracleAdakaon, dict(lr=1e-3, momentum_dtype="int8")),
                    (ko.OracleAdaPNM, dict(lr=1e-3, momentum_dtype="int8"))):
        opt = cls([p.copy() for p in p0], SHAPES, bf16_method="none", **kw)
        opt.step(z)
        opt.step(z)
        for t, a in zip(opt.tensors, p0):
            assert np.array_equal(t.p, a), cls.__name__


def test_nekaon_eval_removes_the_climb_exactly_for_fp32_weights():
    """reference tests/test_nekaon.py: after eval() the weights are the ones an Adakaon without the climb
    would hold; train() puts the climb back."""
    rng = np.random.default_rng(6)
    p0 = _f32(rng, SHAPES, 0.02)
    opt = ko.OracleNekaon([p.copy() for p in p0], SHAPES, lr=1e-3, betas=(0.2, 0.999))
    for _ in range(3):
        opt.step(_f32(rng, SHAPES, 1e-3))
    climbed = [t.p.copy() for t in opt.tensors]
    opt.eval()
    flat = [t.p.copy() for t in opt.tensors]
    assert any(np.abs(a - b).max() > 0 for a, b in zip(climbed, flat))
    opt.train()
    for t, a in zip(opt.tensors, climbed):
        assert np.allclose(t.p, a, rtol=0, atol=1e-9)


def test_kprodigy_distance_estimate_never_shrinks_and_grows_on_a_steady_direction():
    rng = np.random.default_rng(7)
    p0 = _f32(rng, SHAPES, 0.02)
    base = _f32(rng, SHAPES, 1e-3)
    opt = ko.OracleKProdigy([p.copy() for p in p0], SHAPES, bf16_method="none")
    ds = []
    for _ in range(12):
        opt.step([b + n for b, n in zip(base, _f32(rng, SHAPES, 3e-4))])
        ds.append(float(opt.group["d"]))
    assert all(b >= a for a, b in zip(ds, ds[1:]))
    assert ds[-1] > ds[0]
