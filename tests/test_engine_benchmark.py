"""The native engine benchmark (benchmark/engine/engine_bench.cpp, C API only) on a tiny CPU model: every scenario runs to its
JSON report and its gates (reference: benchmark/engine/docs/benchmark-requirements.md:46-47), and the replica launcher adds up
the throughput of independent engine processes."""
import json
import os
import shutil
import subprocess
import sys

import pytest

from helpers import tiny_model_dir

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
RUN = os.path.join(ROOT, "benchmark", "engine", "run.py")

pytestmark = pytest.mark.skipif(shutil.which("g++") is None, reason="no C++ compiler")


@pytest.fixture(scope="module")
def model_dir(tmp_path_factory):
    d, _ = tiny_model_dir(str(tmp_path_factory.mktemp("bench_model")), std=0.3)
    return d


def _run(model_dir, tmp_path, *extra):
    out = str(tmp_path / "r.json")
    r = subprocess.run([sys.executable, RUN, "--model", model_dir, "--build_dir", str(tmp_path), "--out", out, "--concurrency", "3",
                        "--prompt_len", "24", "--long_prompt_len", "200", "--new_tokens", "10", "--trials", "3", "--turns", "2", *extra],
                       capture_output=True, text=True, timeout=900)
    assert os.path.exists(out), r.stdout[-2000:] + r.stderr[-2000:]
    return json.load(open(out)), r.returncode


def test_all_scenarios_report_and_gate(model_dir, tmp_path):
    res, rc = _run(model_dir, tmp_path, "--all", "--itl_gate_ratio", "1000")
    runs = {r["scenario"]: r for r in res["runs"]}
    assert set(runs) == {"decode_baseline", "mixed", "cancellation", "continuation"}
    assert rc == 0 and res["gates_passed"], res
    base = runs["decode_baseline"]
    assert base["tokens"] == 3 * 10 and base["all_complete"] and base["itl_ms_n"] == 3 * 9 and base["tokens_per_s"] > 0
    assert runs["mixed"]["starved"] is False and runs["mixed"]["itl_during_prefill_ms_n"] >= 3
    assert runs["cancellation"]["cancel_latency_ms_n"] == 3 and runs["cancellation"]["cancel_latency_ms_p95"] <= 500.0
    cont = runs["continuation"]
    assert cont["turn1_ttft_ms_n"] == 3      # every request went through a second turn on its resident cache
    assert "commit" in res["environment"] or "python" in res["environment"]


def test_a_failed_gate_fails_the_run(model_dir, tmp_path):
    res, rc = _run(model_dir, tmp_path, "--scenario", "cancellation", "--cancel_gate_ms", "0.000001")
    assert rc == 1 and res["gates_passed"] is False


def test_replica_launcher_sums_independent_engines(model_dir, tmp_path):
    res, rc = _run(model_dir, tmp_path, "--scenario", "decode_baseline", "--replicas", "2")
    run = res["runs"][0]
    assert rc == 0 and run["replica_count"] == 2 and len(run["replicas"]) == 2
    assert abs(run["tokens_per_s_total"] - sum(r["tokens_per_s"] for r in run["replicas"])) < 1e-6
