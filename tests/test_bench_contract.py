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
