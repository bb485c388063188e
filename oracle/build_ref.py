#!/usr/bin/env python
"""Builds oracle/_ref/libmnref.so: the reference's own CPU helpers for the dequantise + matmul
path, compiled from the reference checkout where it lies.

TEST INFRASTRUCTURE ONLY.  The helpers (pack_int4, dequant_reference_int4/int8,
matmul_reference, fp16_to_fp32, fp32_to_fp16) are lines 103-259 of
tests/cpp/test_dequant_matmul.mm, member functions of a GoogleTest fixture whose file needs
Objective-C++, Metal headers and GoogleTest as a whole.  Those lines alone are plain C++:
this script copies them, byte for byte, into oracle/_ref/ref_helpers.inc and compiles
ref_shim.cpp, which includes that file as the body of a struct and puts C entry points over
it.  Nothing of the reference is committed: oracle/_ref/ is a build product.

    python oracle/build_ref.py [--reference /path/to/metal-native] [--force]

Compiled with g++ -O2 -ffp-contract=off and no fast-math: source-order IEEE fp32, the same
flags as the restatement it validates.  (The reference's own build passes no floating-point
flags for host code, cmake/AppleSiliconFlags.cmake:4-56.)
"""
from __future__ import annotations

import argparse
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
OUT_DIR = HERE / "_ref"
LIB = OUT_DIR / "libmnref.so"
SOURCE = "tests/cpp/test_dequant_matmul.mm"
FIRST_LINE, LAST_LINE = 103, 259
# the range must start and end where expected, or the reference differs from the one surveyed
EXPECT_FIRST = "// Helper: Pack pairs of INT4 values into bytes"
EXPECT_INSIDE = ("std::vector<uint8_t> pack_int4(", "std::vector<float> dequant_reference_int4(",
                 "std::vector<float> dequant_reference_int8(", "std::vector<float> matmul_reference(",
                 "static float fp16_to_fp32(", "static uint16_t fp32_to_fp16(")


def extract(reference: Path) -> str:
    lines = (reference / SOURCE).read_text().splitlines(keepends=True)
    body = "".join(lines[FIRST_LINE - 1:LAST_LINE])
    if EXPECT_FIRST not in lines[FIRST_LINE - 1]:
        raise RuntimeError(f"{SOURCE}:{FIRST_LINE} is not the start of the CPU helpers")
    for needle in EXPECT_INSIDE:
        if needle not in body:
            raise RuntimeError(f"{SOURCE}:{FIRST_LINE}-{LAST_LINE} lacks `{needle}`")
    if body.count("{") != body.count("}"):
        raise RuntimeError(f"{SOURCE}:{FIRST_LINE}-{LAST_LINE} is not a whole number of functions")
    return body


def build(reference: Path, force: bool = False) -> Path | None:
    """Returns the library path, or None when the reference checkout is absent (the GPU box: the
    prebuilt library travels there)."""
    src = reference / SOURCE
    if not src.exists():
        return LIB if LIB.exists() else None
    shim = HERE / "ref_shim.cpp"
    if not force and LIB.exists() and LIB.stat().st_mtime >= max(src.stat().st_mtime, shim.stat().st_mtime,
                                                                Path(__file__).stat().st_mtime):
        return LIB
    OUT_DIR.mkdir(exist_ok=True)
    (OUT_DIR / "ref_helpers.inc").write_text(extract(reference))
    cmd = ["g++", "-O2", "-fPIC", "-shared", "-std=c++17", "-fno-fast-math", "-ffp-contract=off",
           "-I", str(HERE), "-o", str(LIB), str(shim)]
    subprocess.run(cmd, check=True)
    return LIB


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default="/root/reference")
    ap.add_argument("--force", action="store_true")
    a = ap.parse_args()
    out = build(Path(a.reference), a.force)
    print(out if out else "reference checkout not found; nothing built")
    sys.exit(0)
