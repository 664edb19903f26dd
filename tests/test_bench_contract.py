"""The benchmark's reference arm on the CPU: one JSON line with the keys the contract names, and
the flop accounting of the workloads."""
from __future__ import annotations

import json
import subprocess
import sys

from conftest import ROOT

sys.path.insert(0, str(ROOT))
import bench  # noqa: E402


def test_flop_accounting_of_the_configurations():
    # F_alg = 24 * heads * pairs * D (12 contractions); causal counts N(N+1)/2 pairs
    w = bench.WORKLOADS
    assert bench.f_alg(w["cfg1"]) == 24.0 * 2 * 256 * 256 * 64 == 201326592.0
    assert round(bench.f_alg(w["cfg2"]) / 1e11, 3) == 4.123
    assert round(bench.f_alg(w["cfg3"]) / 1e12, 3) == 3.299
    assert round(bench.f_alg(w["cfg4"]) / 1e13, 3) == 5.278
    assert round(bench.f_alg(w["cfg5"]) / 1e13, 3) == 5.278
    assert bench.pairs(w["cfg3"]) == 4096 * 4097 // 2
    assert abs(bench.EXEC_OVER_ALG - 22 / 12) < 1e-12
    assert w["cfg5"]["bh"] == 16 * 32 and w["cfg4"]["bh"] == 32


def test_reference_arm_prints_one_contract_line():
    out = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--workload", "cfg1",
                          "--steps", "2", "--warmup", "1"], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [l for l in out.stdout.splitlines() if l.strip()]
    assert len(lines) == 1
    j = json.loads(lines[0])
    for key in ("metric", "value", "unit", "impl", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better",
                "scaling", "vs_baseline", "dtype", "data", "config", "cpu_baseline", "e2e"):
        assert key in j, key
    assert j["impl"] == "reference" and j["unit"] == "TFLOP/s" and j["higher_is_better"] is True
    assert j["config"]["workload"] == "cfg1" and j["vs_baseline"] is None and j["data"] == "synthetic"
    assert j["cpu_baseline"]["kind"] == "port" and j["cpu_baseline"]["cores"] >= 1 and j["cpu_baseline"]["sample"]
    assert j["cpu_baseline"]["value"] == j["value"] == j["e2e"]["value"] > 0
    assert j["e2e"]["h2d_bytes_per_step"] == 0 and j["e2e"]["d2h_bytes_per_step"] == 0

