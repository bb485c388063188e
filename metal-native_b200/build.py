"""Builds metal_native/lib/libmnq.so from csrc/*.cu with nvcc for sm_100a.

Usage: python metal-native_b200/build.py [--force] [--verbose]
nvcc cross-compiles; no GPU is needed to build.
"""
from __future__ import annotations

import argparse
import os
import shutil
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
CSRC = HERE / "csrc"
LIB_DIR = HERE / "metal_native" / "lib"
LIB = LIB_DIR / "libmnq.so"
SOURCES = ["api.cu", "dequantize.cu", "gemv.cu", "gemv_stream.cu", "gemv_lean.cu", "gemv_mid.cu", "gemm_tcgen05.cu", "no_alloc.cu", "residual_norm.cu"]
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden", "--expt-relaxed-constexpr",
]


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise RuntimeError("nvcc not found (set NVCC=/path/to/nvcc)")


def sources() -> list[Path]:
    missing = [s for s in SOURCES if not (CSRC / s).exists()]
    if missing:
        raise RuntimeError(f"listed sources are missing from {CSRC}: {missing}")
    return [CSRC / s for s in SOURCES]


def is_stale() -> bool:
    if not LIB.exists():
        return True
    t = LIB.stat().st_mtime
    deps = list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + [HERE.parent / "include" / "mnq.h", Path(__file__)]
    return any(d.stat().st_mtime > t for d in deps if d.exists())


def build(force: bool = False, verbose: bool = False, out: Path | None = None, extra_flags: list[str] | None = None) -> Path:
    """Compiles and links the library.  `out` and `extra_flags` build a variant elsewhere (for
    example with -D switches) without touching the in-tree library."""
    variant = out is not None or bool(extra_flags)
    if not variant and not force and not is_stale():
        return LIB
    nvcc = find_nvcc()
    target = Path(out) if out is not None else LIB
    target.parent.mkdir(parents=True, exist_ok=True)
    obj_dir = HERE / "build" / ("variant_" + target.parent.name if variant else "")
    obj_dir.mkdir(parents=True, exist_ok=True)
    procs = []
    objs = []
    for src in sources():
        obj = obj_dir / (src.stem + ".o")
        objs.append(obj)
        cmd = [nvcc, *NVCC_FLAGS, *(extra_flags or []), "-c", str(src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas")
            cmd.insert(2, "-v")
            print(" ".join(cmd), flush=True)
        procs.append((src, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
    failed = False
    for src, p in procs:
        out, _ = p.communicate()
        if p.returncode != 0 or verbose:
            sys.stderr.write(out)
        failed |= p.returncode != 0
    if failed:
        raise RuntimeError("nvcc failed")
    tmp = target.with_suffix(".so.tmp")
    link = [nvcc, "-Wno-deprecated-gpu-targets", "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"]
    subprocess.run(link, check=True)
    os.replace(tmp, target)
    return target


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--force", action="store_true")
    ap.add_argument("--verbose", action="store_true")
    ap.add_argument("--out", default=None, help="write the library here instead of metal_native/lib/libmnq.so")
    ap.add_argument("--flag", action="append", default=[], help="extra nvcc flag (repeatable), e.g. --flag=-DNAME")
    a = ap.parse_args()
    print(build(a.force, a.verbose, Path(a.out) if a.out else None, a.flag))
