"""CPU: the C-ABI library loads without a GPU and exports every symbol include/ytcuda.h declares."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def declared_functions():
    text = (ROOT / "include" / "ytcuda.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ytcuda_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_functions():
    names = declared_functions()
    assert "ytcuda_gemm" in names and len(names) >= 10


def test_library_exports_every_declared_symbol():
    import __graft_entry__
    __graft_entry__.build()
    lib = ctypes.CDLL(str(ROOT / "ytensor_b200" / "libytensor_cuda.so"))
    missing = [n for n in declared_functions() if not hasattr(lib, n)]
    assert not missing, f"declared in include/ytcuda.h but not exported: {missing}"


def test_python_binding_covers_the_header():
    from ytensor_b200 import _lib
    assert sorted(_lib.SIGNATURES) == declared_functions()
    _lib.lib()  # binds every signature; raises if a symbol is missing


def test_argument_validation_needs_no_gpu():
    from ytensor_b200 import _lib
    L = _lib.lib()
    # bad dtype and negative extents are rejected before any CUDA call
    assert L.ytcuda_gemm(7, 0, None, None, None, 1, 1, 1, 1.0, 0.0, 1, 1, 1, 1, 1, 1, 1, 0, 0, 0, None) == _lib.INVALID_ARG
    assert L.ytcuda_gemm(0, 0, None, None, None, -1, 1, 1, 1.0, 0.0, 1, 1, 1, 1, 1, 1, 1, 0, 0, 0, None) == _lib.INVALID_ARG
    assert b"negative" in L.ytcuda_last_error_string()
    # empty problems succeed without a launch (reference kernels return silently on empty dims)
    assert L.ytcuda_gemm(0, 0, None, None, None, 0, 5, 5, 1.0, 0.0, 1, 1, 1, 1, 1, 1, 1, 0, 0, 0, None) == _lib.OK
    assert L.ytcuda_launch_count() == 0
