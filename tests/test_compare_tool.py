"""The compare tool: run as a subprocess and parse its JSON, like upstream's tool tests
(tests/test_backend_benchmark_tools.py:714-744)."""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
SAMPLES = str(ROOT / "tests" / "compare_samples.py")


def _run(*extra: str) -> object:
    done = subprocess.run([sys.executable, "-m", "baybridge_b200.compare", SAMPLES, "indexed_add_f32_kernel", *extra],
                          capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    return json.loads(done.stdout)


def test_compile_only_summary(tmp_path):
    payload = _run("--sample-factory", "shape_only_args", "--backends", "b200,portable,ptx_exec", "--include-env",
                   "--cache-dir", str(tmp_path))
    results = {entry["backend"]: entry for entry in payload["results"]}
    assert results["b200"]["status"] == "ok" and results["b200"]["dialect"] == "b200.plan" and results["b200"]["target"] == "sm_100a"
    assert results["portable"]["status"] == "ok" and results["portable"]["lowered_path"] is None
    assert results["ptx_exec"]["status"] == "error" and results["ptx_exec"]["error_type"] == "CompilationError"
    assert "python" in payload["environment"]


def test_timing_summary_matches_upstream_definition():
    from baybridge_b200.compare import summarize_timings_ms

    summary = summarize_timings_ms([9.0, 1.0, 3.0, 2.0])
    assert summary == {"cold_ms": 9.0, "warm_timings_ms": [1.0, 3.0, 2.0], "warm_median_ms": 2.0}


@pytest.mark.gpu
def test_execute_on_device(tmp_path):
    payload = _run("--sample-factory", "device_args", "--backends", "b200,portable", "--execute", "--repeat", "5",
                   "--cache-dir", str(tmp_path))
    results = {entry["backend"]: entry for entry in payload}
    b200 = results["b200"]
    assert b200["execute_status"] == "ok" and len(b200["timings_ms"]) == 5 and b200["warm_median_ms"] > 0
    n = 65536
    assert b200["result_summaries"]["2"]["sum"] == pytest.approx(n * (n - 1) / 2 + 2.0 * n, rel=1e-6)
    assert results["portable"]["execute_status"] == "skipped_non_exec_backend"
