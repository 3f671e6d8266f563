"""The seam script on a copy of the YTensor tree (CPU only; skipped where the tree is not present): every anchor is
found, the patched copy still compiles without the backend (-DYT_USE_CUDA=0) and with it (-DYT_USE_CUDA=1, syntax
only: nothing is linked or run here)."""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
REF = Path(os.environ.get("YT_REFERENCE", "/root/reference"))

pytestmark = pytest.mark.skipif(not (REF / "ytensor.hpp").exists() or shutil.which("g++") is None,
                                reason="needs the YTensor source tree and g++")

PROGRAM = """
#include "ytensor.hpp"
int main() {
  yt::YTensor<float, 2> a(4, 8), b(8, 4);
  auto c = a.matmul(b);
  auto s = yt::function::softmax(c, -1);
  return static_cast<int>(s.size()) == 16 ? 0 : 1;
}
"""


@pytest.fixture(scope="module")
def patched(tmp_path_factory):
    out = tmp_path_factory.mktemp("seam") / "tree"
    r = subprocess.run([sys.executable, str(ROOT / "integration" / "apply_seam.py"), str(REF), str(out)],
                       capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    return out


def test_every_branch_is_inserted(patched):
    infos = (patched / "include" / "ytensor_infos.hpp").read_text(encoding="utf-8")
    assert "YT_USE_CUDA" in infos and "CUDA" in infos.split("enum class MatmulBackend")[1].split("}")[0]
    assert "FLASH_CUDA" in (patched / "include" / "function" / "ops.hpp").read_text(encoding="utf-8")
    assert "ytensor_cuda.hpp" in (patched / "ytensor.hpp").read_text(encoding="utf-8")
    math = (patched / "src" / "ytensor_math.inl").read_text(encoding="utf-8")
    assert "MatmulBackend::CUDA" in math and "yt::cuda::seam" in math
    assert "FLASH_CUDA" in (patched / "src" / "function" / "ops.inl").read_text(encoding="utf-8")
    # nothing of the reference was removed: every original line is still there, in order
    for rel in ("src/ytensor_math.inl", "src/function/ops.inl", "include/ytensor_infos.hpp"):
        # (the one edit that is not an insertion: the last enumerator of MatmulBackend gains a comma)
        new = (patched / rel).read_text(encoding="utf-8").replace("AVX2 = 2,", "AVX2 = 2 ").split("\n")
        it = iter(new)
        for line in (REF / rel).read_text(encoding="utf-8").split("\n"):
            assert any(line == cand for cand in it), f"{rel}: a line of the reference is missing or out of order"


@pytest.mark.parametrize("use_cuda", [0, 1])
def test_patched_tree_compiles(patched, tmp_path, use_cuda):
    src = tmp_path / "prog.cpp"
    src.write_text(PROGRAM)
    cmd = ["g++", "-std=c++20", "-fsyntax-only", "-include", "algorithm", "-w", "-mavx2", "-mfma", "-mf16c", "-fopenmp",
           f"-DYT_USE_CUDA={use_cuda}", f"-I{patched}", f"-I{ROOT / 'include'}", f"-I{ROOT / 'ytensor_b200' / 'cpp'}",
           str(src)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
