"""ctypes + numpy front end of the CPU oracle (``dequant_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by ``__graft_entry__.smoke()``
and by ``bench.py``'s CPU-baseline / reference arm, never by the shipped package.

All arrays are numpy; fp16 travels as ``np.float16`` or raw ``uint16`` bits, bf16
only as raw ``uint16`` bits (numpy has no bf16).  The arithmetic is done by the C
functions, which follow the reference's CPU helpers
(``tests/cpp/test_dequant_matmul.mm:104-259``) and standalone dequantise shaders
(``shaders/dequantize_kernel.metal``).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_LIB_PATH = _HERE / "_build" / "liboracle.so"
_lib = None


def build(force: bool = False) -> Path:
    """Compile ``dequant_oracle.c`` with gcc (``make -C oracle``) if needed."""
    src = _HERE / "dequant_oracle.c"
    stale = (not _LIB_PATH.exists()) or (_LIB_PATH.stat().st_mtime < src.stat().st_mtime)
    if force or stale:
        subprocess.run(["make", "-C", str(_HERE), "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def _u8p(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8))


def _i8p(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_int8))


def _u16p(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_uint16))


def _f32p(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def lib() -> ctypes.CDLL:
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(str(_LIB_PATH))
        u32, sz = ctypes.c_uint32, ctypes.c_size_t
        PU8, PI8 = ctypes.POINTER(ctypes.c_uint8), ctypes.POINTER(ctypes.c_int8)
        PU16, PF = ctypes.POINTER(ctypes.c_uint16), ctypes.POINTER(ctypes.c_float)
        L.oracle_fp16_to_fp32.restype = ctypes.c_float
        L.oracle_fp16_to_fp32.argtypes = [ctypes.c_uint16]
        L.oracle_fp32_to_fp16_trunc.restype = ctypes.c_uint16
        L.oracle_fp32_to_fp16_trunc.argtypes = [ctypes.c_float]
        L.oracle_fp32_to_fp16_rn.restype = ctypes.c_uint16
        L.oracle_fp32_to_fp16_rn.argtypes = [ctypes.c_float]
        L.oracle_bf16_to_fp32.restype = ctypes.c_float
        L.oracle_bf16_to_fp32.argtypes = [ctypes.c_uint16]
        L.oracle_fp32_to_bf16_rn.restype = ctypes.c_uint16
        L.oracle_fp32_to_bf16_rn.argtypes = [ctypes.c_float]
        for name, a, b in (("oracle_fp16_to_fp32_array", PU16, PF),
                           ("oracle_fp32_to_fp16_rn_array", PF, PU16),
                           ("oracle_bf16_to_fp32_array", PU16, PF),
                           ("oracle_fp32_to_bf16_rn_array", PF, PU16)):
            fn = getattr(L, name)
            fn.restype = None
            fn.argtypes = [a, b, sz]
        L.oracle_pack_int4.restype = None
        L.oracle_pack_int4.argtypes = [PI8, sz, PU8]
        L.oracle_dequant_int4.restype = None
        L.oracle_dequant_int4.argtypes = [PU8, PF, PF, u32, u32, u32, PF]
        L.oracle_dequant_int8.restype = None
        L.oracle_dequant_int8.argtypes = [PI8, PF, PF, u32, u32, u32, PF]
        L.oracle_matmul.restype = None
        L.oracle_matmul.argtypes = [PF, PF, u32, u32, u32, PF]
        L.oracle_dequant_matmul.restype = ctypes.c_int
        L.oracle_dequant_matmul.argtypes = [PF, ctypes.c_void_p, PF, PF, u32, u32, u32, u32,
                                            ctypes.c_int, ctypes.c_int, PF, PF]
        L.oracle_dequantize_flat_int8.restype = None
        L.oracle_dequantize_flat_int8.argtypes = [PI8, PU16, PU16, u32, u32]
        L.oracle_dequantize_flat_int4.restype = None
        L.oracle_dequantize_flat_int4.argtypes = [PU8, PU16, PU16, u32, u32]
        _lib = L
    return _lib


# ---------------------------------------------------------------------------
# dtype helpers
# ---------------------------------------------------------------------------

def fp16_bits_to_fp32(bits: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(bits).view(np.uint16)
    out = np.empty(bits.shape, np.float32)
    lib().oracle_fp16_to_fp32_array(_u16p(bits), _f32p(out), bits.size)
    return out


def fp32_to_fp16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().oracle_fp32_to_fp16_rn_array(_f32p(x), _u16p(out), x.size)
    return out


def bf16_bits_to_fp32(bits: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(bits).view(np.uint16)
    out = np.empty(bits.shape, np.float32)
    lib().oracle_bf16_to_fp32_array(_u16p(bits), _f32p(out), bits.size)
    return out


def fp32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    x = np.ascontiguousarray(x, np.float32)
    out = np.empty(x.shape, np.uint16)
    lib().oracle_fp32_to_bf16_rn_array(_f32p(x), _u16p(out), x.size)
    return out


def widen(a: np.ndarray, kind: str) -> np.ndarray:
    """Any of fp32 / fp16 (np.float16 or bits) / bf16 bits -> fp32, exactly."""
    if kind == "fp32":
        return np.ascontiguousarray(a, np.float32)
    if kind == "fp16":
        return fp16_bits_to_fp32(np.ascontiguousarray(a).view(np.uint16))
    if kind == "bf16":
        return bf16_bits_to_fp32(a)
    raise ValueError(kind)


# ---------------------------------------------------------------------------
# the reference's CPU helpers
# ---------------------------------------------------------------------------

def pack_int4(values: np.ndarray) -> np.ndarray:
    """tests/cpp/test_dequant_matmul.mm:104-116 over a flat int8 array."""
    v = np.ascontiguousarray(values, np.int8).ravel()
    out = np.zeros((v.size + 1) // 2, np.uint8)
    lib().oracle_pack_int4(_i8p(v), v.size, _u8p(out))
    return out


def dequant_int4(packed, scales, zeros, K, N, group_size) -> np.ndarray:
    packed = np.ascontiguousarray(packed, np.uint8)
    scales = np.ascontiguousarray(scales, np.float32)
    zeros = np.ascontiguousarray(zeros, np.float32)
    groups = (K + group_size - 1) // group_size
    assert packed.size == N * ((K + 1) // 2), (packed.size, N, K)
    assert scales.size == N * groups and zeros.size == N * groups
    out = np.empty((N, K), np.float32)
    lib().oracle_dequant_int4(_u8p(packed), _f32p(scales), _f32p(zeros), K, N, group_size, _f32p(out))
    return out


def dequant_int8(data, scales, zeros, K, N, group_size) -> np.ndarray:
    data = np.ascontiguousarray(data, np.int8)
    scales = np.ascontiguousarray(scales, np.float32)
    zeros = np.ascontiguousarray(zeros, np.float32)
    groups = (K + group_size - 1) // group_size
    assert data.size == N * K
    assert scales.size == N * groups and zeros.size == N * groups
    out = np.empty((N, K), np.float32)
    lib().oracle_dequant_int8(_i8p(data), _f32p(scales), _f32p(zeros), K, N, group_size, _f32p(out))
    return out


def matmul(A, B) -> np.ndarray:
    """tests/cpp/test_dequant_matmul.mm:191-213; A [M,K], B [N,K] -> [M,N]."""
    A = np.ascontiguousarray(A, np.float32)
    B = np.ascontiguousarray(B, np.float32)
    M, K = A.shape
    N, K2 = B.shape
    assert K == K2
    C = np.empty((M, N), np.float32)
    lib().oracle_matmul(_f32p(A), _f32p(B), M, N, K, _f32p(C))
    return C


def dequant_matmul(A, wq, scales, zeros, group_size, quant: str, threads: int = 1,
                   scratch: np.ndarray | None = None) -> np.ndarray:
    """Dequantise the whole weight to fp32, then the naive matmul; fp32 in, fp32 out.

    ``A`` [M,K] fp32; ``wq`` uint8 [N,K/2] (int4) or int8 [N,K]; ``scales``/``zeros``
    fp32 [N, ceil(K/g)] (``zeros=None`` means all zero).  ``threads`` only slices N.
    """
    A = np.ascontiguousarray(A, np.float32)
    M, K = A.shape
    q = 0 if quant == "int4" else 1
    if q == 0:
        wq = np.ascontiguousarray(wq).view(np.uint8)
        N = wq.shape[0]
        assert wq.shape[1] == (K + 1) // 2
    else:
        assert quant == "int8"
        wq = np.ascontiguousarray(wq).view(np.int8)
        N = wq.shape[0]
        assert wq.shape[1] == K
    groups = (K + group_size - 1) // group_size
    scales = np.ascontiguousarray(scales, np.float32).reshape(N, groups)
    zeros = (np.zeros((N, groups), np.float32) if zeros is None
             else np.ascontiguousarray(zeros, np.float32).reshape(N, groups))
    if scratch is None:
        scratch = np.empty((N, K), np.float32)
    assert scratch.size >= N * K and scratch.dtype == np.float32
    C = np.empty((M, N), np.float32)
    rc = lib().oracle_dequant_matmul(_f32p(A), wq.ctypes.data_as(ctypes.c_void_p), _f32p(scales),
                                     _f32p(zeros), M, N, K, group_size, q, int(threads),
                                     _f32p(scratch), _f32p(C))
    if rc != 0:
        raise RuntimeError("oracle_dequant_matmul: could not start worker threads")
    return C


def dequantize_flat(q, scales_fp16_bits, num_elements, group_size, quant: str) -> np.ndarray:
    """shaders/dequantize_kernel.metal semantics; returns fp16 bits (uint16)."""
    s = np.ascontiguousarray(scales_fp16_bits).view(np.uint16)
    out = np.zeros(num_elements, np.uint16)
    if quant == "int4":
        qq = np.ascontiguousarray(q).view(np.uint8).ravel()
        assert qq.size * 2 >= num_elements
        lib().oracle_dequantize_flat_int4(_u8p(qq), _u16p(s), _u16p(out), num_elements, group_size)
    else:
        qq = np.ascontiguousarray(q).view(np.int8).ravel()
        assert qq.size >= num_elements
        lib().oracle_dequantize_flat_int8(_i8p(qq), _u16p(s), _u16p(out), num_elements, group_size)
    return out


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:  # pragma: no cover
        return os.cpu_count() or 1


def residual_rms_norm(inp: np.ndarray, residual: np.ndarray, weight: np.ndarray, eps: float, kind: str):
    """CPU restatement of the reference's fused residual + RMSNorm kernel
    (``shaders/fused_residual_norm.metal:43-76``, fp16 variant; the same steps for bf16): per row,
    ``s = float(input) + float(residual)`` (``:62``), the sum is rounded to the 16-bit type and stored
    (``:63``), the sum of squares is taken over the unrounded ``s`` in fp32 (``:64``),
    ``rms_inv = rsqrt(sum_sq / n + eps)`` (``:68``), and the output is the rounded sum times ``rms_inv``
    times the weight, rounded (``:70-73``).  The reference adds the squares lane by lane and then
    across the SIMD group; here they are added in float64 and rounded once, so a comparison has to
    allow the output's last bit.

    Parity unpinned: the reference holds no value test or golden vector for this operator (its
    Metal kernels cannot run here).  What the reference's test suite does hold is the numpy formula
    ``reference_rms_norm`` (``tests/test_numerical_accuracy.py:68-84``: ``x / sqrt(mean(x^2) + eps) *
    weight``); tests/test_residual_norm.py checks this restatement against that formula applied to
    ``input + residual``, to the precision of the 16-bit roundings.

    ``inp``, ``residual`` [rows, n] and ``weight`` [n] as fp32 arrays holding fp16 / bf16 values
    (``kind``).  Returns (normalised, rounded sums), both fp32 arrays of values exact in ``kind``."""
    to_bits, from_bits = ((fp32_to_fp16_bits, fp16_bits_to_fp32) if kind == "fp16"
                          else (fp32_to_bf16_bits, bf16_bits_to_fp32))
    s = np.asarray(inp, np.float32) + np.asarray(residual, np.float32)
    h = from_bits(to_bits(s))
    n = s.shape[-1]
    mean = (s.astype(np.float64) ** 2).sum(axis=-1, keepdims=True) / n
    rms_inv = (1.0 / np.sqrt(mean.astype(np.float32) + np.float32(eps))).astype(np.float32)
    out = (h * rms_inv).astype(np.float32) * np.asarray(weight, np.float32)
    return from_bits(to_bits(out.astype(np.float32))), h
