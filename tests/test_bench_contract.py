"""bench.py on a machine without a GPU: the reference arm (the CPU oracle port) prints the contract's
JSON line; the product arm refuses to run instead of falling back to anything on the CPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _run(*args):
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    return subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), *args], capture_output=True, text=True,
                          env=env, timeout=600)


def test_reference_arm_prints_one_contract_line():
    r = _run("--impl", "reference", "--workload", "cfg1", "--steps", "3", "--warmup", "3")
    assert r.returncode == 0, r.stderr
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and d["metric"] == "tree_attn_calls_per_s" and d["unit"] == "calls/s"
    assert d["higher_is_better"] is True and d["n_gpus"] == 1 and d["steps"] == 3 and d["value"] > 0
    assert d["config"]["workload"].startswith("cfg1")
    assert d["cpu_baseline"]["kind"] == "port" and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["value"] == d["value"]
    assert d["e2e"] == {"value": d["value"], "unit": "calls/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}


def test_product_arm_has_no_cpu_path():
    r = _run("--steps", "1", "--warmup", "3", "--no-cpu-baseline")
    assert not [ln for ln in r.stdout.splitlines() if ln.startswith("{")], "no number may be printed without a GPU"
    assert "no CPU path" in (r.stdout + r.stderr)


import pytest  # noqa: E402


@pytest.mark.gpu
def test_product_arm_line_carries_the_contract_keys():
    """One short run of the GPU arm on a small batch of the headline workload: one JSON line with the
    contract's keys, a roofline fraction that is a fraction, an end-to-end figure with its copies
    declared, the oracle check of what was timed, and a clean kernel status."""
    env = dict(os.environ)
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--workload", "cfg3", "--batch", "4", "--only",
                        "--steps", "3", "--warmup", "3", "--no-cpu-baseline", "--no-triton"],
                       capture_output=True, text=True, env=env, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    d = json.loads(lines[0])
    for k in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
              "vs_baseline", "dtype", "data", "config", "roofline", "e2e", "gpu_launches", "clocks"):
        assert k in d, k
    assert d["metric"] == "tree_attn_calls_per_s" and d["unit"] == "calls/s" and d["n_gpus"] == 1 and d["value"] > 0
    assert d["config"]["workload"].startswith("cfg3") and d["dtype"] == "bf16" and d["vs_baseline"] is None
    roof = d["roofline"]
    assert roof["bound"] == "hbm" and roof["unit"] == "GB/s" and 0 < roof["frac"] < 1.3
    assert abs(roof["frac"] - roof["achieved"] / roof["peak"]) < 1e-9
    e2e = d["e2e"]
    assert e2e["value"] > 0 and e2e["h2d_bytes_per_step"] > 0 and e2e["d2h_bytes_per_step"] > 0
    assert e2e["value"] <= d["value"] * 1.05  # copies can only cost
    assert d["gpu_launches"] == 2 * 3 * 5  # stage 1 + stage 2, 3 steps, 5 timed regions
    assert d["within_tolerance"] is True and d["kernel_status"] == 0
    assert d["max_abs_out"] <= 2e-3 + 2.0 ** -8 and d["max_abs_lse"] <= 1e-3


def test_reference_arm_under_a_multi_rank_launch():
    """Launched as one of several ranks (torch.distributed.run exports OMP_NUM_THREADS=1): rank 0 alone
    runs the arm, on all host cores, and says that the job is partitioned over the ranks; the other
    ranks print nothing and exit 0."""
    base = dict(os.environ, CUDA_VISIBLE_DEVICES="", WORLD_SIZE="4", OMP_NUM_THREADS="1")
    cmd = [sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--workload", "cfg1", "--gpus", "4",
           "--steps", "3", "--warmup", "3"]
    r1 = subprocess.run(cmd, capture_output=True, text=True, env=dict(base, RANK="1"), timeout=600)
    assert r1.returncode == 0 and not [ln for ln in r1.stdout.splitlines() if ln.startswith("{")]
    r0 = subprocess.run(cmd, capture_output=True, text=True, env=dict(base, RANK="0"), timeout=600)
    assert r0.returncode == 0, r0.stderr
    d = json.loads([ln for ln in r0.stdout.splitlines() if ln.startswith("{")][-1])
    assert d["impl"] == "reference" and d["n_gpus"] == 4 and d["scaling"] == "strong"
    assert d["cpu_baseline"]["cores"] == (os.cpu_count() or 1)
    assert "4 GPUs" in d["config"]["parallelism"]
