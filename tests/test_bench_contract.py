"""The one-line JSON contract of bench.py: the CPU reference arm here, the GPU arm on a B200."""

from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
COMMON = {"metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling",
          "vs_baseline", "dtype", "data", "config", "e2e", "cpu_baseline", "gpu_launches"}


def _run(args, env=None, timeout=600):
    proc = subprocess.run([sys.executable, str(ROOT / "bench.py"), *args], capture_output=True, text=True, cwd=ROOT,
                          env={**os.environ, **(env or {})}, timeout=timeout)
    assert proc.returncode == 0, proc.stderr[-2000:]
    return [ln for ln in proc.stdout.splitlines() if ln.startswith("{")]


def test_reference_arm_prints_one_line_and_other_ranks_stay_silent():
    (line,) = _run(["--impl", "reference", "--steps", "2", "--warmup", "1", "--cpu-seconds", "3"])
    d = json.loads(line)
    assert COMMON <= set(d) and d["impl"] == "reference" and d["gpu_launches"] == 0
    assert d["metric"] == "BEVFormer-base SCA MSDA Gsamples/s" and d["unit"] == "Gsamples/s" and d["value"] > 0
    assert d["config"]["workload"] == "base_sca" and d["steps"] == 2 and d["higher_is_better"] is True
    # the reference's own evaluator when oracle/_ref was made from a checkout, else the restatement
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["cores"] >= 1 and d["cpu_baseline"]["sample"]
    assert d["cpu_baseline"]["single_thread_cli_loop"]["cores"] == 1 and d["scaling"] == "strong"
    assert d["cpu_baseline"]["value"] == d["value"] == d["e2e"]["value"]
    assert d["e2e"]["h2d_bytes_per_step"] == 0 and d["e2e"]["d2h_bytes_per_step"] == 0
    # under a multi-rank launcher only rank 0 works
    assert _run(["--impl", "reference", "--gpus", "2", "--steps", "1", "--warmup", "0", "--cpu-seconds", "1"],
                env={"RANK": "1", "LOCAL_RANK": "1", "WORLD_SIZE": "2"}) == []


@pytest.mark.gpu
def test_gpu_arm_line_carries_the_roofline_the_baseline_and_the_clocks():
    (line,) = _run(["--steps", "5", "--warmup", "3", "--kernel-only"])
    d = json.loads(line)
    assert d["kernel_only"] is True and d["parity"]["fp32_max_abs"] <= 1e-4
    (line,) = _run(["--steps", "10", "--warmup", "3", "--e2e-steps", "2"], timeout=900)
    d = json.loads(line)
    assert COMMON | {"roofline", "clocks"} <= set(d)
    assert d["n_gpus"] == 1 and d["gpu_launches"] == 10 and d["dtype"] == "f32" and d["vs_baseline"] is None
    r = d["roofline"]
    assert r["bound"] == "hbm" and r["unit"] == "GB/s" and abs(r["frac"] - r["achieved"] / r["peak"]) < 1e-9
    assert r["traffic"] and 0.05 < r["frac"] < 1.2
    assert d["e2e"]["h2d_bytes_per_step"] == 373708800 and d["e2e"]["d2h_bytes_per_step"] == 61440000
    assert 0 < d["e2e"]["value"] < d["value"]
    assert d["cpu_baseline"]["kind"] in ("reference", "port") and d["cpu_baseline"]["value"] > 0
    assert d["scaling"] == "strong" and d["config"]["global_queries_per_camera"] == 10000
    assert d["e2e"]["default_session"]["value"] > 0 and d["e2e"]["checked_max_abs"] <= 1e-4
    assert d["clocks"]["sm_max_mhz"] >= d["clocks"]["sm_mhz"] > 0
    assert d["parity"]["fp32_max_abs"] <= 1e-4
