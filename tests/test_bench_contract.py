"""The reference arm of bench.py on the CPU (no GPU involved): one JSON line with the keys the measurement contract
names, alone and under torch.distributed.run with two ranks (rank 0 alone measures and prints; the other rank leaves
without work)."""
from __future__ import annotations

import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]


def _check(line: dict, n_gpus: int):
    assert line["impl"] == "reference"
    assert line["metric"] == "bf16_gemm_tflops" and line["unit"] == "TFLOP/s"
    assert line["n_gpus"] == n_gpus and line["steps"] == 1
    assert line["value"] > 0 and line["ms_per_step"] > 0
    assert line["higher_is_better"] is True and line["vs_baseline"] is None
    assert line["data"] == "synthetic" and "workload" in line["config"]
    cb = line["cpu_baseline"]
    assert cb["kind"] in ("reference", "port") and cb["cores"] >= 1 and cb["sample"] and cb["value"] == line["value"]
    e2e = line["e2e"]
    assert e2e["value"] == line["value"] and e2e["h2d_bytes_per_step"] == 0 and e2e["d2h_bytes_per_step"] == 0


@pytest.fixture(scope="module")
def _oracle_built(port):  # (the session fixture builds / loads the CPU oracle the arm times)
    return port


def test_reference_arm_prints_one_contract_line(_oracle_built):
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "0",
                        "--no-secondary"], capture_output=True, text=True, timeout=600, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1
    _check(json.loads(lines[0]), 1)


def test_reference_arm_under_two_ranks(_oracle_built):
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29717", str(ROOT / "bench.py"), "--impl",
                        "reference", "--gpus", "2", "--steps", "1", "--warmup", "0", "--no-secondary"],
                       capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [ln for ln in r.stdout.splitlines() if ln.startswith("{")]
    assert len(lines) == 1, r.stdout[-2000:]
    _check(json.loads(lines[0]), 2)
