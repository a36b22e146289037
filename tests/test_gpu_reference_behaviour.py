"""The behaviours the reference's own hot-path tests hold it to, asked of this package on a GPU.

Each test names the reference test it restates (tests/test_adakaon.py, tests/test_lion.py,
tests/test_msam.py, tests/test_nekaon.py of the reference).  They go through the public classes only:
state sizes and dtypes, training sanity, an independent numpy Lion, the Nekaon climb's bound and its exact
removal, checkpoints through ``torch.save``."""
import io
import math

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


def _mlp(dtype=torch.float32):
    torch.manual_seed(0xC0DE)
    return torch.nn.Sequential(torch.nn.Linear(32, 64), torch.nn.GELU(), torch.nn.Linear(64, 8)).to(DEV, dtype)


def _train(model, opt, x, y, steps):
    loss = None
    for _ in range(steps):
        opt.zero_grad()
        loss = (model(x) - y).pow(2).mean()
        loss.backward()
        opt.step()
    torch.cuda.synchronize()
    return loss


# ---- reference tests/test_adakaon.py:16-41: what the state costs ----

def test_conv_kernel_keeps_row_plus_column_statistics_only():
    import kaon_b200
    p = torch.nn.Parameter(torch.randn(64, 32, 3, 3, device=DEV))
    opt = kaon_b200.Adakaon([p], lr=1e-3, betas=(0.0, 0.999))
    p.grad = torch.randn_like(p)
    opt.step()
    st = opt.state[p]
    floats = sum(v.numel() for v in st.values() if torch.is_tensor(v))
    assert st["row"].numel() == 64 and st["col"].numel() == 32 * 9
    assert floats < p.numel() / 50


def test_bf16_momentum_takes_half_the_bytes_of_fp32_momentum():
    import kaon_b200

    def mom_bytes(md):
        p = torch.nn.Parameter(torch.randn(128, 128, device=DEV))
        opt = kaon_b200.Adakaon([p], lr=1e-3, momentum_dtype=md)
        p.grad = torch.randn_like(p)
        opt.step()
        m = opt.state[p]["m"]
        return m.numel() * m.element_size()

    assert mom_bytes("bfloat16") * 2 == mom_bytes("float32")


def test_4bit_momentum_is_half_a_byte_per_parameter_plus_block_scales():
    """reference tests/test_adakaon.py:231-243"""
    import kaon_b200
    p = torch.nn.Parameter(torch.randn(256, 384, device=DEV))
    opt = kaon_b200.Adakaon([p], lr=1e-3, momentum_dtype="4bit")
    p.grad = torch.randn_like(p)
    opt.step()
    st = opt.state[p]
    assert st["m"].dtype == torch.uint8 and st["m"].numel() == p.numel() // 2
    assert st["m_scale"].numel() == p.numel() // 128 and st["m_block"] == 128 and st["m_numel"] == p.numel()


# ---- reference tests/test_adakaon.py:43-92, 246-262, 327-345: it trains ----

@pytest.mark.parametrize("cls_name,kw", [("Adakaon", dict(lr=3e-3)), ("Adakaon", dict(lr=3e-3, momentum_dtype="4bit")),
                                         ("Adakaon", dict(lr=3e-3, momentum_dtype="int8")), ("Lion", dict(lr=3e-3)),
                                         ("AdaPNM", dict(lr=3e-3)), ("Nekaon", dict(lr=3e-3))])
def test_regression_loss_drops(cls_name, kw):
    import kaon_b200
    model = _mlp()
    opt = getattr(kaon_b200, cls_name)(model.parameters(), **kw)
    gen = torch.Generator().manual_seed(1)
    x, y = torch.randn(64, 32, generator=gen).to(DEV), torch.randn(64, 8, generator=gen).to(DEV)
    first = (model(x) - y).pow(2).mean().item()
    _train(model, opt, x, y, 80)
    if hasattr(opt, "eval"):
        opt.eval()
    last = (model(x) - y).pow(2).mean().item()
    assert last < 0.5 * first, (first, last)


def test_conv_net_trains_without_nan():
    import kaon_b200
    torch.manual_seed(0)
    net = torch.nn.Sequential(torch.nn.Conv2d(4, 16, 3, padding=1), torch.nn.GELU(),
                              torch.nn.Conv2d(16, 4, 3, padding=1)).to(DEV)
    opt = kaon_b200.Adakaon(net.parameters(), lr=3e-3)
    x, y = torch.randn(8, 4, 16, 16, device=DEV), torch.randn(8, 4, 16, 16, device=DEV)
    assert math.isfinite(_train(net, opt, x, y, 30).item())


@pytest.mark.parametrize("cls_name", ["Adakaon", "Lion", "AdaPNM", "AdaMuon"])
def test_bf16_weights_train_without_nan(cls_name):
    import kaon_b200
    model = _mlp(torch.bfloat16)
    opt = getattr(kaon_b200, cls_name)(model.parameters(), lr=3e-3 if cls_name != "Lion" else 3e-4,
                                      bf16_method="stochastic_rounding")
    x = torch.randn(64, 32, device=DEV, dtype=torch.bfloat16)
    y = torch.randn(64, 8, device=DEV, dtype=torch.bfloat16)
    assert torch.isfinite(_train(model, opt, x, y, 30))
    assert all(torch.isfinite(p).all() for p in model.parameters())


# ---- reference tests/test_lion.py:17-105: the sign-momentum arithmetic against an independent numpy ----

def _numpy_lion(p, g, m, lr, b1, b2, wd, cautious):
    c = b1 * m + (1.0 - b1) * g
    m2 = b2 * m + (1.0 - b2) * g
    delta = np.sign(c) + wd * p
    if cautious:
        mask = (delta * g > 0).astype(delta.dtype)
        delta = delta * mask / max(mask.mean(), 1e-8)
    return p - lr * delta, m2


@pytest.mark.parametrize("cautious", [False, True])
@pytest.mark.parametrize("wd", [0.0, 0.1])
def test_lion_matches_an_independent_numpy_step(cautious, wd):
    import kaon_b200
    torch.manual_seed(0)
    lr, b1, b2 = 0.01, 0.9, 0.99
    p = torch.nn.Parameter(torch.randn(16, 7).to(DEV))
    opt = kaon_b200.Lion([p], lr=lr, betas=(b1, b2), weight_decay=wd, momentum_dtype="float32",
                         cautious=cautious, gradient_centralization=False)
    pr = p.detach().cpu().numpy().astype(np.float64)
    mr = np.zeros_like(pr)
    gen = torch.Generator().manual_seed(3)
    for _ in range(12):
        g = torch.randn(16, 7, generator=gen)
        p.grad = g.to(DEV)
        opt.step()
        pr, mr = _numpy_lion(pr, g.numpy().astype(np.float64), mr, lr, b1, b2, wd, cautious)
    torch.testing.assert_close(p.detach().cpu().double(), torch.from_numpy(pr), rtol=1e-5, atol=1e-6)
    torch.testing.assert_close(opt.state[p]["m"].cpu().double(), torch.from_numpy(mr), rtol=1e-5, atol=1e-6)


def test_lion_first_step_moves_every_weight_by_lr_against_the_gradient_sign():
    import kaon_b200
    p = torch.nn.Parameter(torch.randn(12, 9, device=DEV))
    before = p.detach().clone()
    opt = kaon_b200.Lion([p], lr=1e-2, momentum_dtype="float32", cautious=False, gradient_centralization=False)
    p.grad = torch.randn_like(p)
    opt.step()
    torch.testing.assert_close(before - p.detach(), 1e-2 * torch.sign(p.grad), rtol=0, atol=1e-7)


# ---- reference tests/test_msam.py:152-246 through the Nekaon preset (rho = -k, norm "none", weight decay 0.1) ----

def _nekaon_params(seed=0):
    gen = torch.Generator().manual_seed(seed)
    return [torch.nn.Parameter(torch.randn(s, generator=gen).to(DEV)) for s in ((24, 16), (40,), (6, 4, 3, 3))]


def _attach(params, seed):
    gen = torch.Generator().manual_seed(100 + seed)
    for p in params:
        p.grad = torch.randn(p.shape, generator=gen).to(DEV)


def test_nekaon_climb_is_k_times_the_stored_momentum_capped_per_element():
    import kaon_b200
    k, lr = 1.5, 1e-3
    pa = _nekaon_params()
    opt = kaon_b200.Nekaon(pa, lr=lr, k=k, betas=(0.2, 0.999), momentum_dtype="float32")
    _attach(pa, 1)
    opt.step()
    live = [p.detach().clone() for p in pa]
    mom = [opt.base_optimizer.state[p]["m"].detach().clone() for p in pa]
    opt.eval()
    bound = k * 1.0 * lr
    for w, p, m in zip(live, pa, mom):
        expected = (-k * m.reshape(p.shape)).clamp(-bound, bound)
        assert torch.allclose(w - p.detach(), expected, atol=1e-6, rtol=1e-6)
    opt.train()
    for p, w in zip(pa, live):
        assert torch.equal(p.detach(), w)


def test_nekaon_momentum_spike_cannot_move_a_weight_beyond_the_bound():
    import kaon_b200
    k, lr = 1.5, 1e-3
    pa = _nekaon_params()
    opt = kaon_b200.Nekaon(pa, lr=lr, k=k, betas=(0.2, 0.999), momentum_dtype="float32")
    _attach(pa, 1)
    opt.step()
    opt.base_optimizer.state[pa[0]]["m"][0, 0] = 1.0     # a thousand times any sane update
    _attach(pa, 2)
    opt.step()
    live = [p.detach().clone() for p in pa]
    opt.eval()
    worst = max((w - p.detach()).abs().max().item() for w, p in zip(live, pa))
    assert worst <= k * lr * (1 + 1e-5), worst
    opt.train()
    for p, w in zip(pa, live):
        assert torch.equal(p.detach(), w)


def test_nekaon_non_finite_momentum_contributes_no_climb():
    import kaon_b200
    pa = _nekaon_params()
    opt = kaon_b200.Nekaon(pa, lr=1e-3, k=1.5, betas=(0.2, 0.999), momentum_dtype="float32")
    _attach(pa, 1)
    opt.step()
    opt.eval()
    m = opt.base_optimizer.state[pa[0]]["m"]
    m[0, 0] = float("nan")
    m[0, 1] = float("inf")
    opt.train()
    torch.cuda.synchronize()
    assert all(torch.isfinite(p).all() for p in pa)


def test_nekaon_bound_is_frozen_when_the_lr_changes_between_steps():
    import kaon_b200
    pa = _nekaon_params()
    opt = kaon_b200.Nekaon(pa, lr=1e-3, k=1.5, betas=(0.2, 0.999), momentum_dtype="float32")
    _attach(pa, 1)
    opt.step()
    for g in opt.param_groups:
        g["lr"] = 1e-4
    live = [p.detach().clone() for p in pa]
    opt.eval()
    opt.train()
    for p, w in zip(pa, live):
        assert torch.equal(p.detach(), w)


def test_nekaon_step_outside_train_mode_is_an_error():
    import kaon_b200
    pa = _nekaon_params()
    opt = kaon_b200.Nekaon(pa, lr=1e-3)
    _attach(pa, 1)
    opt.step()
    opt.eval()
    _attach(pa, 2)
    with pytest.raises(RuntimeError, match="outside train mode"):
        opt.step()


# ---- reference tests/test_adakaon.py:347-385: checkpoints through torch.save keep every dtype and resume exactly ----

@pytest.mark.parametrize("cls_name", ["Adakaon", "Lion", "AdaPNM"])
@pytest.mark.parametrize("md", ["bfloat16", "float32", "int8", "4bit"])
def test_checkpoint_through_torch_save_keeps_dtypes_and_resumes_exactly(cls_name, md):
    import kaon_b200
    cls = getattr(kaon_b200, cls_name)
    shapes = [(32, 48), (8, 4, 3, 3), (40,)]

    def build():
        gen = torch.Generator().manual_seed(5)
        ps = [torch.nn.Parameter(torch.randn(s, generator=gen).to(DEV)) for s in shapes]
        o = cls(ps, lr=1e-3 if cls_name != "Lion" else 1e-4, momentum_dtype=md)
        o.sr_seed = 9
        return ps, o

    gen = torch.Generator().manual_seed(6)
    grads = [[torch.randn(s, generator=gen).to(DEV) for s in shapes] for _ in range(5)]

    def run(ps, o, ks):
        for k in ks:
            for p, g in zip(ps, grads[k]):
                p.grad = g
            o.step()
        torch.cuda.synchronize()

    pa, oa = build()
    run(pa, oa, range(5))
    pb, ob = build()
    run(pb, ob, range(3))
    buf = io.BytesIO()
    torch.save({"opt": ob.state_dict(), "w": [p.detach().cpu() for p in pb]}, buf)
    buf.seek(0)
    ck = torch.load(buf, weights_only=False)
    pc, oc = build()
    with torch.no_grad():
        for q, w in zip(pc, ck["w"]):
            q.copy_(w)
    oc.load_state_dict(ck["opt"])
    for b, c in zip(pb, pc):
        for key, vb in ob.state[b].items():
            vc = oc.state[c][key]
            if torch.is_tensor(vb):
                assert vc.dtype == vb.dtype and vc.shape == vb.shape and vc.device == vb.device, key
    run(pc, oc, range(3, 5))
    for a, c in zip(pa, pc):
        assert torch.equal(a.detach(), c.detach())


# ---- this package's own: the per-group hooks a pipelined caller hangs its events on ----

def test_group_hooks_run_around_each_groups_launches_and_change_no_result():
    """`before_group(i)` / `after_group(i)` are called once per parameter group and step, in order, around
    that group's launches; a step cut into groups writes the same weights as the same list in one group
    (the stochastic-rounding stream is keyed by the tensor's position in the whole list)."""
    import kaon_b200
    gen = torch.Generator().manual_seed(77)
    host = [(torch.randn(s, generator=gen) * 0.02).bfloat16() for s in [(96, 128), (64,), (48, 16, 3, 3), (200, 40)]]
    grads = [(torch.randn(h.shape, generator=gen) * 1e-3).bfloat16() for h in host]
    out = []
    for grouped in (False, True):
        ps = [torch.nn.Parameter(h.clone().to(DEV)) for h in host]
        arg = [{"params": ps[:1]}, {"params": ps[1:3]}, {"params": ps[3:]}] if grouped else ps
        opt = kaon_b200.Lion(arg, lr=1e-3, momentum_dtype="4bit")
        opt.sr_seed = 5
        calls = []
        opt.before_group = lambda gi: calls.append(("before", gi))
        opt.after_group = lambda gi: calls.append(("after", gi))
        for _ in range(2):
            for p, g in zip(ps, grads):
                p.grad = g.clone().to(DEV)
            opt.step()
        torch.cuda.synchronize()
        opt.check_device_status()
        n = 3 if grouped else 1
        assert calls == [(w, gi) for gi in range(n) for w in ("before", "after")] * 2
        out.append([p.detach().cpu() for p in ps])
    for a, b in zip(*out):
        assert torch.equal(a, b)
