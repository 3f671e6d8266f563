"""Generates tests/golden/golden_ext.npz by running the UNMODIFIED reference (oracle/_ref/libyt_ref.so) on seeded
inputs, for the operators beyond the first golden file:

    make -C oracle ref REF=<YTensor source tree> && python tests/golden/make_golden_ext.py

  norm_*    yt::function::normalize (p = 2 and 1.5, one and two axes, affine), instanceNorm, batchNorm, groupNorm
            (channel axis 1 and 2, plain and affine)                     src/function/normalization.inl:278-577
  fp8_*     float -> yt::float8_e5m2 / e4m3 / e8m0 bits for a sweep that covers zero, subnormal results, ties,
            overflow, infinities and NaN; and all 256 encodings of each type back to float
                                                                          include/types/float_spec.hpp:299-371, 435-491
  mmc_*     YTensor::masked_matmul with the causal predicate (tile-pruning form) at two offsets
                                                                          src/ytensor_math.inl:368-412
"""
from __future__ import annotations

import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))
from oracle import oracle as O  # noqa: E402

OUT = Path(__file__).resolve().parent / "golden_ext.npz"


def main():
    R = O.ref(threads=1)
    rng = np.random.default_rng(77)
    N = lambda *s, scale=1.0: (rng.standard_normal(s) * scale).astype(np.float32)  # noqa: E731
    g = {}
    X = N(3, 6, 5, 8) + 0.3
    g["norm_x"] = X
    gam, bia = rng.uniform(0.5, 1.5, 6).astype(np.float32), N(6)
    g["norm_gamma6"], g["norm_bias6"] = gam, bia
    g["norm_l2_m1"] = R.norm("normalize", X, [-1], p=2.0, eps=1e-12)
    g["norm_l15_a13"] = R.norm("normalize", X, [1, 3], p=1.5, eps=1e-6)
    g["norm_l2_a1_affine"] = R.norm("normalize", X, [1], gam, bia, p=2.0, eps=1e-12)
    g["norm_inst_c1"] = R.norm("instanceNorm", X, [1], eps=1e-5)
    g["norm_inst_c1_affine"] = R.norm("instanceNorm", X, [1], gam, bia, eps=1e-5)
    gam5, bia5 = rng.uniform(0.5, 1.5, 5).astype(np.float32), N(5)
    g["norm_gamma5"], g["norm_bias5"] = gam5, bia5
    g["norm_inst_c2_affine"] = R.norm("instanceNorm", X, [2], gam5, bia5, eps=1e-5)
    g["norm_batch_c1"] = R.norm("batchNorm", X, [1], eps=1e-5)
    g["norm_batch_c1_affine"] = R.norm("batchNorm", X, [1], gam, bia, eps=1e-5)
    g["norm_batch_cm1"] = R.norm("batchNorm", X, [-1], eps=1e-5)
    g["norm_group2_c1"] = R.norm("groupNorm", X, [1], groups=2, eps=1e-5)
    g["norm_group3_c1_affine"] = R.norm("groupNorm", X, [1], gam, bia, groups=3, eps=1e-5)
    Xg = N(2, 5, 4, 7)
    g["norm_xg"] = Xg
    gam4, bia4 = rng.uniform(0.5, 1.5, 4).astype(np.float32), N(4)
    g["norm_gamma4"], g["norm_bias4"] = gam4, bia4
    g["norm_group2_c2_affine"] = R.norm("groupNorm", Xg, [2], gam4, bia4, groups=2, eps=1e-5)

    # fp8: magnitudes from below the smallest normal of every format to above its largest, exact ties, specials
    mags = np.concatenate([np.exp2(rng.uniform(-20, 18, 4000)), np.exp2(np.arange(-20, 18)) * 1.25,
                           np.exp2(np.arange(-20, 18)) * 1.125, np.exp2(np.arange(-20, 18)) * 1.0625,
                           np.exp2(rng.uniform(-140, 130, 500))]).astype(np.float32)
    sweep = np.concatenate([mags, -mags, np.array([0.0, -0.0, np.inf, -np.inf, np.nan, 1e-45, 3.4e38, 448.0, 57344.0,
                                                   65504.0, 240.0, 0.0078125], np.float32)])
    g["fp8_in"] = sweep
    for kind in ("float8_e5m2", "float8_e4m3", "float8_e8m0"):
        g[f"fp8_{kind}_bits"] = R.fp8(kind, sweep)
        g[f"fp8_{kind}_table"] = R.fp8_to_f32(kind, np.arange(256, dtype=np.uint8))

    a, b = N(2, 150, 40), N(40, 170)
    g["mmc_a"], g["mmc_b"] = a, b
    g["mmc_off0"] = R.masked_matmul_causal(a, b, 0, -1e9)
    g["mmc_off20"] = R.masked_matmul_causal(a, b, 20, 0.5)
    np.savez_compressed(OUT, **g)
    print(f"wrote {OUT} ({OUT.stat().st_size / 1024:.0f} KiB, {len(g)} arrays)")


if __name__ == "__main__":
    main()
