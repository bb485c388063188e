"""ctypes front end of ``oracle/_ref/libmnref.so``: the reference's own CPU helpers
(``tests/cpp/test_dequant_matmul.mm:103-259``) compiled from the reference checkout by
``build_ref.py``.

TEST INFRASTRUCTURE ONLY: used by ``tests/`` to check the restatement in ``dequant_oracle.c``
bit for bit, and by ``bench.py``'s CPU legs as the timed reference implementation.
"""
from __future__ import annotations

import ctypes
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
LIB_PATH = _HERE / "_ref" / "libmnref.so"
_lib = None


def available() -> bool:
    return LIB_PATH.exists()


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        if not LIB_PATH.exists():
            raise FileNotFoundError(f"{LIB_PATH} is missing: run oracle/build_ref.py next to a reference checkout")
        L = ctypes.CDLL(str(LIB_PATH))
        u32, sz, vp = ctypes.c_uint32, ctypes.c_size_t, ctypes.c_void_p
        L.ref_pack_int4.restype = None
        L.ref_pack_int4.argtypes = [vp, sz, vp]
        L.ref_fp16_to_fp32.restype = ctypes.c_float
        L.ref_fp16_to_fp32.argtypes = [ctypes.c_uint16]
        L.ref_fp32_to_fp16.restype = ctypes.c_uint16
        L.ref_fp32_to_fp16.argtypes = [ctypes.c_float]
        L.ref_dequant_int4.restype = None
        L.ref_dequant_int4.argtypes = [vp, vp, vp, u32, u32, u32, vp]
        L.ref_dequant_int8.restype = None
        L.ref_dequant_int8.argtypes = [vp, vp, vp, u32, u32, u32, vp]
        L.ref_matmul.restype = None
        L.ref_matmul.argtypes = [vp, vp, u32, u32, u32, vp]
        L.ref_dequant_matmul_rows.restype = None
        L.ref_dequant_matmul_rows.argtypes = [vp, vp, vp, vp, u32, u32, u32, ctypes.c_int, u32, u32, vp]
        _lib = L
    return _lib


def _p(a: np.ndarray):
    return a.ctypes.data_as(ctypes.c_void_p)


def pack_int4(values) -> np.ndarray:
    v = np.ascontiguousarray(values, np.int8).ravel()
    out = np.zeros((v.size + 1) // 2, np.uint8)
    lib().ref_pack_int4(_p(v), v.size, _p(out))
    return out


def fp16_to_fp32(bits: int) -> float:
    return float(lib().ref_fp16_to_fp32(int(bits)))


def fp32_to_fp16(v: float) -> int:
    return int(lib().ref_fp32_to_fp16(float(v)))


def dequant(wq, scales, zeros, K, N, group_size, quant: str) -> np.ndarray:
    s = np.ascontiguousarray(scales, np.float32)
    z = np.zeros_like(s) if zeros is None else np.ascontiguousarray(zeros, np.float32)
    out = np.empty((N, K), np.float32)
    if quant == "int4":
        w = np.ascontiguousarray(wq).view(np.uint8)
        lib().ref_dequant_int4(_p(w), _p(s), _p(z), K, N, group_size, _p(out))
    else:
        w = np.ascontiguousarray(wq).view(np.int8)
        lib().ref_dequant_int8(_p(w), _p(s), _p(z), K, N, group_size, _p(out))
    return out


def matmul(A, B) -> np.ndarray:
    A = np.ascontiguousarray(A, np.float32)
    B = np.ascontiguousarray(B, np.float32)
    M, K = A.shape
    N = B.shape[0]
    C = np.empty((M, N), np.float32)
    lib().ref_matmul(_p(A), _p(B), M, N, K, _p(C))
    return C


def dequant_matmul(A, wq, scales, zeros, group_size, quant: str, threads: int = 1) -> np.ndarray:
    """The reference's CPU path, dequantise everything to fp32 then the naive matmul, with the
    output columns cut into ``threads`` contiguous ranges that run on as many host threads (each
    range is an independent call of the reference helpers; the library call releases the GIL)."""
    A = np.ascontiguousarray(A, np.float32)
    M, K = A.shape
    w = np.ascontiguousarray(wq)
    N = w.shape[0]
    G = (K + group_size - 1) // group_size
    s = np.ascontiguousarray(scales, np.float32).reshape(N, G)
    z = np.zeros_like(s) if zeros is None else np.ascontiguousarray(zeros, np.float32).reshape(N, G)
    q = 0 if quant == "int4" else 1
    threads = max(1, min(int(threads), N))
    bounds = [N * t // threads for t in range(threads + 1)]
    parts = [np.empty((M, bounds[t + 1] - bounds[t]), np.float32) for t in range(threads)]
    L = lib()

    def run(t):
        L.ref_dequant_matmul_rows(_p(A), _p(w), _p(s), _p(z), M, K, group_size, q, bounds[t], bounds[t + 1],
                                  _p(parts[t]))

    if threads == 1:
        run(0)
    else:
        with ThreadPoolExecutor(threads) as ex:
            list(ex.map(run, range(threads)))
    return np.concatenate(parts, axis=1)
