#!/usr/bin/env python
"""Applies the device-backend seam to a COPY of the YTensor source tree.

    python integration/apply_seam.py <reference tree> <output dir>

The reference tree is never edited: `ytensor.hpp`, `include/` and `src/` are copied to the output directory and
the copy gets the branches a maintainer of YTensor would add for the device backend. Every edit is an insertion next
to an anchor line (a signature or a `case` label of the reference, quoted below only as far as needed to find the
place); nothing is deleted (one enumerator gains the comma that lets another follow it). Compile the result with `-DYT_USE_CUDA=1 -I<repo>/include -I<repo>/ytensor_b200/cpp`
and link `-lytensor_cuda`. With `-DYT_USE_CUDA=0` (the default of the patched tree) it builds as before.

What is added:
  * include/ytensor_infos.hpp   the YT_USE_CUDA macro, MatmulBackend::CUDA, and CUDA first in the priority of
                                defaultMatmulBackend (CUDA > AVX2 > Eigen > Naive)
  * include/function/ops.hpp    sdpaBackend::FLASH_CUDA
  * ytensor.hpp                 #include "ytensor_cuda.hpp" between the class definitions and the implementations
  * src/ytensor_math.inl        `case MatmulBackend::CUDA` in YTensor::matmul; the in-place operators += -= *= /= go
                                to the device when their left operand is device-resident
  * src/function/ops.inl        `backend == sdpaBackend::FLASH_CUDA` in both scaledDotProductAttention overloads
                                (bool mask, predicate)
  * src/function/activation.inl, normalization.inl
                                softmax / softmax_ / rmsNorm / rmsNorm_ go to the device when x is device-resident
  * src/ytensor_core.inl        YTensor::copy_ between device-resident tensors (dtype conversion included), and
                                host -> device / device -> host when only one side is device-resident
"""
from __future__ import annotations

import re
import shutil
import sys
from pathlib import Path


class Patch:
    def __init__(self, root: Path):
        self.root = root
        self.count = 0

    def edit(self, rel: str, anchor: str, text: str, *, where: str = "after", nth: int = 0, regex: bool = False):
        """Inserts `text` before / after the nth line containing `anchor` (or matching it as a regex); with
        where='after_brace' after the first line at or below the anchor that ends in '{'."""
        p = self.root / rel
        lines = p.read_text(encoding="utf-8").split("\n")
        hits = [i for i, ln in enumerate(lines) if (re.search(anchor, ln) if regex else anchor in ln)]
        if len(hits) <= nth:
            raise SystemExit(f"{rel}: anchor not found ({nth + 1} x): {anchor!r}")
        i = hits[nth]
        if where == "after_brace":
            while not lines[i].rstrip().endswith("{"):
                i += 1
            where = "after"
        if where == "after_endif":
            while lines[i].strip() != "#endif":
                i += 1
            where = "after"
        at = i + 1 if where == "after" else i
        lines[at:at] = text.rstrip("\n").split("\n")
        p.write_text("\n".join(lines), encoding="utf-8")
        self.count += 1

    def replace(self, rel: str, old: str, new: str):
        p = self.root / rel
        s = p.read_text(encoding="utf-8")
        if s.count(old) != 1:
            raise SystemExit(f"{rel}: expected exactly one {old!r}, found {s.count(old)}")
        p.write_text(s.replace(old, new), encoding="utf-8")
        self.count += 1


def apply(ref: Path, out: Path) -> int:
    if out.exists():
        shutil.rmtree(out)
    out.mkdir(parents=True)
    shutil.copy2(ref / "ytensor.hpp", out / "ytensor.hpp")
    for d in ("include", "src"):
        shutil.copytree(ref / d, out / d)
    P = Patch(out)

    # ---- build switch and backend enums
    P.edit("include/ytensor_infos.hpp", "#ifndef YT_IMPL_INLINE", """\
/// Device backend (libytensor_cuda.so): off unless the build asks for it.
#ifndef YT_USE_CUDA
    #define YT_USE_CUDA 0
#endif
""", where="before")
    P.replace("include/ytensor_infos.hpp", "AVX2 = 2 ", "AVX2 = 2,")
    P.edit("include/ytensor_infos.hpp", "AVX2 = 2,", "        CUDA = 3    // sm_100a device backend (libytensor_cuda.so)")
    # CUDA first in the default's priority: the existing #if chain becomes the #else branch of a new one
    P.edit("include/ytensor_infos.hpp", "#if YT_USE_AVX2", """\
    #if YT_USE_CUDA
        MatmulBackend::CUDA
    #else""", where="before", nth=0)
    P.edit("include/ytensor_infos.hpp", "#if YT_USE_AVX2", "    #endif", where="after_endif", nth=0)
    P.replace("include/function/ops.hpp", "        FLASH_AVX2\n", "        FLASH_AVX2,\n        FLASH_CUDA  // sm_100a device backend\n")

    # ---- the backend's C++ header, after the class definitions, before the implementations that call into it
    P.edit("ytensor.hpp", '#include "src/ytensor_base_templates.inl"', """\
#if YT_USE_CUDA
#include "ytensor_cuda.hpp"
#else
namespace yt::cuda::seam {
template <typename A, typename B> constexpr bool inplace_op(const char*, A&, const B&) { return false; }
}
#endif
""", where="before")

    # ---- YTensor::matmul: one more case of the switch on the backend
    P.edit("src/ytensor_math.inl", "switch (backend) {", """\
#if YT_USE_CUDA
            case yt::infos::MatmulBackend::CUDA:
                return yt::cuda::seam::matmul(*this, other);  // refuses what it cannot run: no CPU fallback
#endif""", nth=0)
    # ---- in-place operators (the generating macro: no preprocessor conditionals inside, so the call is always there)
    P.edit("src/ytensor_math.inl", r"operator OP##=\(const yt::YTensor<T, dim1>& other\) \{", """\
        if (yt::cuda::seam::inplace_op(#OP, *this, other)) return *this;                              \\""", regex=True)

    # ---- scaledDotProductAttention: both overloads test the backend in sequence
    for nth in (0, 1):
        pred = nth == 1
        call = ("yt::cuda::seam::sdpa_pred(query, key, value, scale, std::forward<MaskFunc>(mask), bias)" if pred else
                "yt::cuda::seam::sdpa(query, key, value, scale, mask ? 2 : 0, 0, mask, bias)")
        P.edit("src/function/ops.inl", "if (backend == sdpaBackend::FLASH_AVX2) {", f"""\
#if YT_USE_CUDA
    if (backend == sdpaBackend::FLASH_CUDA) {{
        return {call};
    }}
#endif""", where="before", nth=nth)

    # ---- named functions: device-resident tensors stay on the device
    sig = r"yt::function::softmax\(const yt::YTensor<T, dim>& x, const std::vector<int>& axes\) \{"
    P.edit("src/function/activation.inl", sig, """\
#if YT_USE_CUDA
    if constexpr (yt::cuda::seam::device_type_v<T>) if (yt::cuda::on_device(x)) return yt::cuda::dev::softmax(x, axes);
#endif""", regex=True)
    sig = r"yt::function::softmax_\(yt::YTensor<T, dim>& x, const std::vector<int>& axes\) \{"
    P.edit("src/function/activation.inl", sig, """\
#if YT_USE_CUDA
    if constexpr (yt::cuda::seam::device_type_v<T>) if (yt::cuda::on_device(x)) return yt::cuda::dev::softmax_(x, axes);
#endif""", regex=True)
    body = """\
#if YT_USE_CUDA
    if constexpr (yt::cuda::seam::device_type_v<T>) if (yt::cuda::on_device(x)) return yt::cuda::dev::{name}(x, weight, axes, eps);
#endif"""
    # the overloads taking `const std::vector<int>& axes` come first for each name: rmsNorm, then rmsNorm_
    P.edit("src/function/normalization.inl", r"yt::function::rmsNorm\($", body.replace("{name}", "rmsNorm"),
           where="after_brace", regex=True, nth=0)
    P.edit("src/function/normalization.inl", r"yt::function::rmsNorm_\($", body.replace("{name}", "rmsNorm_"),
           where="after_brace", regex=True, nth=0)

    # ---- copy_: device <-> device with conversion, host <-> device of equal type
    P.edit("src/ytensor_core.inl", "::copy_(const yt::YTensorBase& src) {", """\
#if YT_USE_CUDA
    if constexpr (yt::cuda::seam::device_type_v<T>) {
        if (yt::cuda::seam::copy_any(*this, src)) return *this;
    }
#endif""")
    return P.count


def main() -> None:
    if len(sys.argv) != 3:
        raise SystemExit(__doc__)
    ref, out = Path(sys.argv[1]), Path(sys.argv[2])
    if not (ref / "ytensor.hpp").exists():
        raise SystemExit(f"{ref} does not hold ytensor.hpp")
    n = apply(ref, out)
    print(f"{out}: {n} insertions applied")


if __name__ == "__main__":
    main()
