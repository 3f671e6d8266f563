"""GPU: the C++ side of the boundary. tests/cpp/test_backend.cpp builds yt::YTensor operands with the reference's own
headers, runs the reference CPU implementation and yt::cuda::* (ytensor_b200/cpp/ytensor_cuda.hpp over the C ABI) on
the same data and compares them; this test runs that binary. It is built where the reference sources are
(`make -C tests/cpp`) and travels as a built artefact; without it the test is skipped."""
import subprocess
from pathlib import Path

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
BIN = Path(__file__).resolve().parent / "cpp" / "_build" / "test_backend"


def test_ytensor_api_through_the_device_backend():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    if not BIN.exists():
        pytest.skip("tests/cpp/_build/test_backend is not built (needs the reference sources)")
    r = subprocess.run([str(BIN)], capture_output=True, text=True, timeout=600)
    print(r.stdout)
    assert r.returncode == 0, r.stdout + r.stderr
    assert "ALL CASES PASSED" in r.stdout
    assert r.stdout.count("PASS") >= 20
