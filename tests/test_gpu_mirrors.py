"""Weight mirrors (the ZeRO-1 publish fused into the step as peer stores).

On one GPU the "peer" is a second region of the same buffer: the kernels' mirror stores are the same
instructions whatever memory the address maps to.  With two or more GPUs the real thing runs as one
process per GPU over symmetric memory and must give, on every rank, the weights of a single-GPU run."""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

SHAPES = [(96, 128), (16, 12, 3, 3), (200,), (40, 72), (7,), (33, 77), (256, 512)]
# every row a multiple of 16 elements: the plan takes the streaming stages and the separate COUNT/APPLY launches
SHAPES_STREAM = [(96, 128), (16, 16, 4, 4), (200,), (40, 272), (7,), (48, 4096), (256, 512)]


def _numel(s):
    n = 1
    for d in s:
        n *= d
    return n


def _layout(dtype, shapes=None):
    offs, cur = [], 0
    for s in (shapes or SHAPES):
        offs.append(cur)
        cur += (_numel(s) + 127) // 128 * 128
    return offs, cur


@pytest.mark.parametrize("cls_name,kw", [
    ("Lion", dict(lr=2e-4, momentum_dtype="4bit")),
    ("Lion", dict(lr=2e-4, momentum_dtype="int8", weight_decay=0.1, bf16_method="none")),
    ("Lion", dict(lr=2e-4, momentum_dtype="bfloat16", cautious=False)),
    ("Adakaon", dict(lr=1e-4, momentum_dtype="int8")),
    ("Adakaon", dict(lr=1e-4, momentum_dtype="4bit", weight_decay=0.1, bf16_method="none")),
    ("Nekaon", dict(lr=1e-4, betas=(0.2, 0.999))),
    ("AdaMuon", dict(lr=1e-3, momentum_dtype="int8")),
])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("shapes", [SHAPES, SHAPES_STREAM], ids=["ragged", "stream"])
def test_mirror_region_tracks_the_weights(cls_name, kw, dtype, shapes):
    import kaon_b200
    SHAPES = shapes  # noqa: N806 - the body below reads the list under this name
    offs, n = _layout(dtype, shapes)
    flat = torch.zeros(3 * n, dtype=dtype, device="cuda")  # [weights | mirror 1 | mirror 2]
    gen = torch.Generator().manual_seed(11)
    params = []
    for s, o in zip(SHAPES, offs):
        flat[o:o + _numel(s)].copy_((torch.randn(s, generator=gen) * 0.02).to(dtype).reshape(-1))
        params.append(torch.nn.Parameter(flat[o:o + _numel(s)].view(s)))
    flat[n:2 * n].copy_(flat[:n])
    flat[2 * n:].copy_(flat[:n])
    opt = getattr(kaon_b200, cls_name)(params, **kw)
    opt.sr_seed = 2
    esz = flat.element_size()
    opt.set_weight_mirrors(flat.data_ptr(), n * esz, [n * esz, 2 * n * esz])
    for step in range(3):
        for p, s in zip(params, SHAPES):
            p.grad = (torch.randn(s, generator=gen) * 1e-3).to(dtype).cuda()
        opt.step()
    if cls_name == "Nekaon":
        opt.eval()
        opt.train()
    torch.cuda.synchronize()
    opt.check_device_status()
    assert torch.equal(flat[:n], flat[n:2 * n]) and torch.equal(flat[:n], flat[2 * n:])
    assert flat[:n].abs().sum().item() > 0


def test_parameter_outside_the_mirrored_buffer_is_refused():
    import kaon_b200
    from kaon_b200._lib import KaonError
    buf = torch.zeros(4096, dtype=torch.bfloat16, device="cuda")
    p = torch.nn.Parameter(torch.zeros(64, 64, dtype=torch.bfloat16, device="cuda"))
    opt = kaon_b200.Lion([p], momentum_dtype="4bit")
    opt.set_weight_mirrors(buf.data_ptr(), 2048, [2048])
    p.grad = torch.ones_like(p)
    with pytest.raises(KaonError, match="outside the mirrored"):
        opt.step()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("opt_name", ["Lion", "Adakaon", "Adakaon-stream", "Lion-waves", "Adakaon-waves"])
def test_two_ranks_fused_publish_equals_single_gpu(opt_name, tmp_path):
    """One process per GPU; every rank ends with the same full weight buffer as a 1-GPU run."""
    script = os.path.join(os.path.dirname(__file__), "_zero1_rank.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = str(tmp_path / "w")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29533", script, opt_name, out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    ref = subprocess.run([sys.executable, script, opt_name, out], env=dict(env, WORLD_SIZE="1", RANK="0", LOCAL_RANK="0"),
                         capture_output=True, text=True, timeout=600)
    assert ref.returncode == 0, ref.stdout[-3000:] + ref.stderr[-3000:]
    single = torch.load(out + ".w1.r0.pt")
    for r_ in range(2):
        got = torch.load(out + f".w2.r{r_}.pt")
        for i, (a, b) in enumerate(zip(single, got)):
            assert torch.equal(a.view(torch.int16), b.view(torch.int16)), (r_, i)
    # the gathered optimizer state is the single-process checkpoint, entry for entry
    s1, s2 = torch.load(out + ".w1.state.pt"), torch.load(out + ".w2.state.pt")
    if opt_name.endswith("-waves"):   # one group per wave, and a rank's waves depend on what it owns: same union, same settings
        flat = lambda sd: sorted(i for g in sd["param_groups"] for i in g["params"])  # noqa: E731
        assert flat(s1) == flat(s2)
        strip = lambda g: {k: v for k, v in g.items() if k != "params"}  # noqa: E731
        assert all(strip(g) == strip(s1["param_groups"][0]) for g in s1["param_groups"] + s2["param_groups"])
    else:
        assert s1["param_groups"] == s2["param_groups"]
    assert s1["_kaon_b200"] == s2["_kaon_b200"]
    assert s1["state"].keys() == s2["state"].keys()
    for k in s1["state"]:
        assert s1["state"][k].keys() == s2["state"][k].keys()
        for key, v in s1["state"][k].items():
            w = s2["state"][k][key]
            assert torch.equal(v, w) if torch.is_tensor(v) else v == w, (k, key)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_kprodigy_share_one_distance_estimate(tmp_path):
    """KProdigy under ZeRO-1: each rank steps its own tensors, the two sums behind d are all-reduced, so both
    ranks hold the same d as a single-GPU run (to the order of the fp32 additions) and the same weights."""
    script = os.path.join(os.path.dirname(__file__), "_zero1_rank.py")
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = str(tmp_path / "k")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
           "--master-addr", "127.0.0.1", "--master-port", "29534", script, "KProdigy", out]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    ref = subprocess.run([sys.executable, script, "KProdigy", out], env=dict(env, WORLD_SIZE="1", RANK="0", LOCAL_RANK="0"),
                         capture_output=True, text=True, timeout=600)
    assert ref.returncode == 0, ref.stdout[-3000:] + ref.stderr[-3000:]
    s1, s2 = torch.load(out + ".w1.state.pt"), torch.load(out + ".w2.state.pt")
    g1, g2 = s1["param_groups"][0], s2["param_groups"][0]
    assert g1["k"] == g2["k"] == 8 and g1["d"] > g1["d0"]
    for key in ("d", "d_max", "d_numerator"):
        assert abs(g1[key] - g2[key]) <= 1e-5 * abs(g1[key]), (key, g1[key], g2[key])
    single = torch.load(out + ".w1.r0.pt")
    for r_ in range(2):
        got = torch.load(out + f".w2.r{r_}.pt")
        for i, (a, b) in enumerate(zip(single, got)):
            assert (a.view(torch.int16) != b.view(torch.int16)).float().mean() < 2e-3, (r_, i)
