"""The JSON line bench.py prints: the reference arm runs without a GPU (it times the reference package
when it is installed beside the benchmark, else the CPU oracle port, on a bounded sample), so its
contract can be checked here; the GPU arm's keys are checked on a GPU."""
import json
import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(args, timeout=600):
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                       timeout=timeout, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, r.stdout[-2000:]
    return json.loads(lines[0])


def test_reference_arm_line():
    d = _run(["--impl", "reference", "--steps", "1", "--warmup", "0"])
    assert d["impl"] == "reference" and d["metric"] == "optimizer_step_params_per_sec" and d["unit"] == "params/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["value"] > 0
    assert d["config"]["workload"] == "lion4bit_unet2p6b"
    cb = d["cpu_baseline"]
    assert cb["kind"] in ("port", "reference") and cb["cores"] >= 1 and cb["value"] == d["value"] and cb["sample"]
    if cb["kind"] == "reference":
        assert cb["port"]["value"] > 0
    assert d["e2e"] == {"value": d["value"], "unit": "params/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


@pytest.mark.gpu
def test_gpu_arm_line_has_the_contract_keys():
    d = _run(["--workload", "lion4bit_sample", "--steps", "3", "--warmup", "3"])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "roofline", "cpu_baseline", "e2e", "gpu_launches", "clocks"):
        assert key in d, key
    assert d["vs_baseline"] is None and d["data"] == "synthetic" and d["config"]["workload"] == "lion4bit_sample"
    ro = d["roofline"]
    assert ro["bound"] == "hbm" and ro["unit"] == "GB/s" and 0 < ro["frac"] < 1.5 and ro["peak"] > 1000
    assert abs(ro["frac"] - ro["achieved"] / ro["peak"]) < 1e-9
    assert d["gpu_launches"] == d["steps"]           # one Lion kernel per step
    e = d["e2e"]
    assert e["h2d_bytes_per_step"] > 0 and e["d2h_bytes_per_step"] > 0 and e["value"] < d["value"]
    assert d["cpu_baseline"]["kind"] in ("port", "reference") and d["cpu_baseline"]["cores"] >= 1
    assert d["compute_only_ms"] == d["incl_publish_ms"] == d["ms_per_step"]   # one GPU: nothing to publish


def test_reference_arm_uses_the_host_cores_under_a_launcher():
    """torch.distributed.run exports OMP_NUM_THREADS=1; the CPU arm must still use every host core."""
    env = dict(os.environ, OMP_NUM_THREADS="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1",
                        "--warmup", "0"], capture_output=True, text=True, timeout=600, cwd=ROOT, env=env)
    assert r.returncode == 0, r.stderr[-2000:]
    d = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][0])
    assert d["cpu_baseline"]["cores"] == len(os.sched_getaffinity(0))


def test_end_to_end_groups_tile_the_shard():
    """The end-to-end loop copies a rank's shard slice by slice, one slice per parameter group: the slices
    must cover every element exactly once, in order, whatever the padding between tensors, and hold the
    tensors of their group."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    sizes = [1000, 24, 5000, 8, 8, 3000, 700, 64, 12000, 16]
    offsets, cur = [], 0
    for s in sizes:
        offsets.append(cur)
        cur += (s + 127) // 128 * 128        # every tensor starts on an aligned boundary: padding between them
    shard_len = cur + 256
    for ng in (1, 3, 4, 16, 100):
        chunks, bounds = bench.e2e_groups(sizes, offsets, shard_len, ng)
        assert 1 <= len(chunks) <= min(ng, len(sizes)) and len(chunks) == len(bounds)
        assert [k for ch in chunks for k in ch] == list(range(len(sizes)))       # every tensor once, in order
        assert bounds[0][0] == 0 and bounds[-1][1] == shard_len
        assert all(bounds[j][1] == bounds[j + 1][0] for j in range(len(bounds) - 1))
        for ch, (lo, hi) in zip(chunks, bounds):
            assert all(lo <= offsets[k] and offsets[k] + sizes[k] <= hi for k in ch)
    with pytest.raises(ValueError):
        bench.e2e_groups([10, 10, 10, 10], [0, 256, 128, 384], 512, 4)           # not in list order
