"""Writes tests/golden/ref_sample.yt and ref_sample_zlib.yt with the UNMODIFIED reference's yt::io::YTensorIO
(behind oracle/ref_shim.cpp), the expected contents next to them (golden_yt.npz), and checks that files written by
ytensor_b200.ytfile.write_yt are read back correctly by the reference.

Run from the repository root, where the reference sources are available:
    make -C oracle ref REF=<YTensor source tree> && python tests/golden/make_golden_yt.py
"""
from __future__ import annotations

import ctypes as C
import sys
import tempfile
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle as O  # noqa: E402
from ytensor_b200 import ytfile  # noqa: E402
from ytensor_b200.qwen3 import bf16_bits_to_f32, f32_to_bf16_bits  # noqa: E402

HERE = Path(__file__).resolve().parent


def main() -> None:
    lib = O.ref(threads=1).lib
    lib.ytref_yt_load_f32.restype = C.c_longlong
    rng = np.random.default_rng(31)
    f32 = rng.standard_normal((5, 7)).astype(np.float32)
    bf16 = f32_to_bf16_bits(rng.standard_normal((4, 6)).astype(np.float32))
    i32 = rng.integers(-1000, 1000, (2, 3)).astype(np.int32)
    big = np.tile(rng.standard_normal((1, 64)).astype(np.float32), (48, 1))  # compresses well
    tensors = [("weights.f32", 0, f32), ("weights.bf16", 1, bf16), ("ids", 3, i32), ("tiled.f32", 0, big)]
    for fname, method in (("ref_sample.yt", b""), ("ref_sample_zlib.yt", b"zlib")):
        path = str(HERE / fname).encode()
        for n, (name, dt, arr) in enumerate(tensors):
            rc = lib.ytref_yt_save(path, int(n > 0), name.encode(), dt, arr.ctypes.data_as(C.c_void_p), arr.shape[0],
                                   arr.shape[1], method)
            assert rc == 0, (fname, name, rc)
        print(fname, (HERE / fname).stat().st_size, "bytes")
    np.savez_compressed(HERE / "golden_yt.npz", **{"weights.f32": f32, "weights.bf16": bf16, "ids": i32,
                                                    "tiled.f32": big})
    # the other direction: the reference reads what write_yt writes
    with tempfile.TemporaryDirectory() as d:
        for method in ("", "zlib"):
            p = Path(d) / f"ours_{method or 'raw'}.yt"
            ytfile.write_yt(p, {"weights.f32": f32, "weights.bf16": bf16, "tiled.f32": big}, compress=method,
                            bfloat16=("weights.bf16",))
            for name, want in (("weights.f32", f32), ("weights.bf16", bf16_bits_to_f32(bf16)), ("tiled.f32", big)):
                out = np.empty(want.size, np.float32)
                shape = (C.c_int * 2)()
                n = lib.ytref_yt_load_f32(str(p).encode(), name.encode(), out.ctypes.data_as(C.c_void_p),
                                          C.c_longlong(out.size), shape)
                assert n == want.size and tuple(shape) == want.shape, (method, name, n, tuple(shape))
                assert np.array_equal(out.reshape(want.shape), want), (method, name)
    print("the reference reads files written by write_yt (raw and zlib): ok")


if __name__ == "__main__":
    main()
