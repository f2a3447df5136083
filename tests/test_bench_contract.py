"""bench.py keeps its contract: one JSON line with the agreed keys at one GPU, a refusal for more,
and an `unavailable` line for the reference arm."""
import json
import os
import subprocess
import sys

import pytest

from helpers import ROOT

BENCH = os.path.join(ROOT, "bench.py")


def _run(*args, timeout=600):
    return subprocess.run([sys.executable, BENCH, *args], capture_output=True, text=True, timeout=timeout, cwd=ROOT)


def test_more_than_one_gpu_is_refused_with_one_line():
    p = _run("--gpus", "2", "--steps", "2", "--warmup", "1")
    assert p.returncode == 2
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1 and "ONE GPU" in lines[0]


def test_reference_arm_says_why_it_is_unavailable():
    p = _run("--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "1")
    assert p.returncode == 0
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    d = json.loads(lines[0])
    assert d["impl"] == "reference" and isinstance(d["unavailable"], str) and d["unavailable"]


@pytest.mark.gpu
def test_the_line_of_a_short_run_has_every_agreed_key():
    """Two layers of the headline sizes, a few steps: the keys, their types and the simple relations between them."""
    p = _run("--layers", "2", "--steps", "6", "--warmup", "3")
    assert p.returncode == 0, p.stderr[-2000:]
    lines = [l for l in p.stdout.splitlines() if l.strip()]
    assert len(lines) == 1, "exactly one line on standard output"
    d = json.loads(lines[0])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
                "vs_baseline", "dtype", "data", "config", "e2e", "gpu_launches", "clocks", "roofline", "points", "prefill"):
        assert key in d, key
    assert d["n_gpus"] == 1 and d["steps"] == 6 and d["warmup"] == 3 and d["higher_is_better"] is True
    assert d["dtype"] == "bf16" and d["impl"] == "ours" and d["gpu_launches"] > 0
    batch = d["config"]["global_batch"]
    assert abs(d["value"] - batch * 1000.0 / d["ms_per_step"]) <= 0.01 * d["value"]
    cfg = d["config"]
    assert len(cfg) <= 20 and all(not isinstance(v, (dict, list)) for v in cfg.values()), "flat, at most 20 keys"
    assert cfg["layers"] == 2 and cfg["layers_full"] == 36 and cfg["seq_len"] == 2048
    e2e = d["e2e"]
    assert e2e["value"] > 0 and e2e["h2d_bytes_per_step"] > 0 and e2e["d2h_bytes_per_step"] == 4 * batch
    assert e2e["value"] != d["value"], "the end-to-end number is measured, not copied"
    r = d["roofline"]
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-3
    pf = d["prefill"]
    assert pf["tokens"] == 2048 and pf["ms"] > 0 and 0 < pf["frac"] < 1.5
    assert abs(pf["value"] - 2048 * 1000.0 / pf["ms"]) <= 0.01 * pf["value"]
    assert set(d["points"]) == {"decode_b1", "decode_b64"} and all(v > 0 for v in d["points"].values())
    c = d["clocks"]
    assert "sm_mhz" in c and "sm_max_mhz" in c and isinstance(c["reasons"], list)
