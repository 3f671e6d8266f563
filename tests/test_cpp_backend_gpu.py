"""GPU: the C++ side of the boundary, through the reference's own tensor type.

tests/cpp/test_backend.cpp builds yt::YTensor operands with the reference's headers, runs the reference CPU
implementation and yt::cuda::* (ytensor_b200/cpp/ytensor_cuda.hpp over the C ABI) on the same data and compares them.
tests/cpp/test_seam.cpp is compiled with -DYT_USE_CUDA=1 against a copy of the reference tree to which
integration/apply_seam.py has added the backend branches, and calls YTensor's OWN entry points:
a.matmul(b, MatmulBackend::CUDA), scaledDotProductAttention(..., sdpaBackend::FLASH_CUDA), and rmsNorm / += /
softmax_ / copy_ on device-resident tensors. Both binaries are built where the reference sources are
(`make -C tests/cpp`) and travel as built artefacts; without them the tests are skipped."""
import subprocess
from pathlib import Path

import pytest

torch = pytest.importorskip("torch")
pytestmark = pytest.mark.gpu
BUILD = Path(__file__).resolve().parent / "cpp" / "_build"


def _run(name, marker, at_least):
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    exe = BUILD / name
    if not exe.exists():
        pytest.skip(f"tests/cpp/_build/{name} is not built (needs the reference sources)")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    print(r.stdout)
    assert r.returncode == 0, r.stdout + r.stderr
    assert marker in r.stdout
    assert r.stdout.count("PASS") >= at_least


def test_ytensor_api_through_the_device_backend():
    _run("test_backend", "ALL CASES PASSED", 20)


def test_backend_switches_inside_ytensor_itself():
    _run("test_seam", "ALL SEAM CASES PASSED", 20)
