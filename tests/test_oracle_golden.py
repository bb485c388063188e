"""Pins the CPU oracle against the reference's own value-checked tests
(tests/cpp/test_dequant_matmul.mm) via tests/golden/reference_kats.json, and against
hand-computed cases for what the reference leaves unpinned (non-zero zero, several
groups per row, odd tails, the standalone dequantise shaders)."""
import json
from pathlib import Path

import numpy as np
import pytest

from oracle import oracle

GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_kats.json").read_text())


def _run_case(c):
    M, N, K, g = c["M"], c["N"], c["K"], c["group_size"]
    A = np.array(c["A"], np.float32).reshape(M, K)
    s = np.array(c["scales"], np.float32)
    z = np.array(c["zeros"], np.float32)
    if c["quant"] == "int4":
        packed = oracle.pack_int4(np.array(c["q"], np.int8)).reshape(N, K // 2)
        W = oracle.dequant_int4(packed, s, z, K, N, g)
        wq = packed
    else:
        wq = np.array(c["q"], np.int8).reshape(N, K)
        W = oracle.dequant_int8(wq, s, z, K, N, g)
    C = oracle.matmul(A, W)
    C2 = oracle.dequant_matmul(A, wq, s, z, g, c["quant"])
    assert np.array_equal(C, C2)
    return C, wq


@pytest.mark.parametrize("case", GOLDEN["cases"], ids=[c["name"] for c in GOLDEN["cases"]])
def test_reference_known_answers(case):
    C, wq = _run_case(case)
    exp = np.array(case["expected"], np.float64).reshape(case["M"], case["N"])
    # the reference's own tolerance ...
    assert np.max(np.abs(C - exp)) <= case["ref_tol"]
    # ... and what fp32 arithmetic on these small sums should actually deliver
    assert np.max(np.abs(C - exp)) <= 2e-5 * max(1.0, float(np.max(np.abs(exp))))
    if "packed" in case:
        assert wq.ravel().tolist() == case["packed"]


def test_pack_int4_nibble_order_and_odd_tail():
    # low nibble first (tests/cpp/test_dequant_matmul.mm:104-116); odd count pads high with 0
    assert oracle.pack_int4(np.array([1, 2, 3], np.int8)).tolist() == [0x21, 0x03]
    assert oracle.pack_int4(np.array([15, 0, -1, 7], np.int8)).tolist() == [0x0F, 0x7F]


def test_dequant_int4_nonzero_zero_and_group_boundaries():
    # N=2, K=8, g=4 -> 2 groups per row; w = (q-8)*s - z with z a post-scale offset
    q = np.array([[0, 15, 8, 9, 1, 2, 3, 4], [7, 7, 7, 7, 8, 8, 8, 8]], np.int8)
    packed = oracle.pack_int4(q.ravel()).reshape(2, 4)
    s = np.array([[0.5, 0.25], [2.0, 1.0]], np.float32)
    z = np.array([[0.125, -1.0], [0.0, 3.0]], np.float32)
    W = oracle.dequant_int4(packed, s, z, 8, 2, 4)
    exp = np.empty((2, 8), np.float32)
    for n in range(2):
        for k in range(8):
            exp[n, k] = (float(q[n, k]) - 8.0) * float(s[n, k // 4]) - float(z[n, k // 4])
    assert np.array_equal(W, exp)
    assert W[0].tolist() == [-4.125, 3.375, -0.125, 0.375, -0.75, -0.5, -0.25, 0.0]
    assert W[1].tolist() == [-2.0, -2.0, -2.0, -2.0, -3.0, -3.0, -3.0, -3.0]


def test_dequant_int8_nonzero_zero_ragged_last_group():
    # K=6, g=4 -> groups = ceil(6/4) = 2, the second one ragged
    q = np.array([[-128, 127, 0, 1, -1, 2]], np.int8)
    s = np.array([[0.5, 2.0]], np.float32)
    z = np.array([[1.0, -0.5]], np.float32)
    W = oracle.dequant_int8(q, s, z, 6, 1, 4)
    assert W[0].tolist() == [-65.0, 62.5, -1.0, -0.5, -1.5, 4.5]


def test_dequant_int4_odd_K_row_stride():
    # odd K: packed row stride (K+1)/2 (tests/cpp/test_dequant_matmul.mm:134)
    q = np.array([[1, 2, 3], [4, 5, 6]], np.int8)
    packed = np.stack([oracle.pack_int4(q[0]), oracle.pack_int4(q[1])])
    assert packed.shape == (2, 2)
    W = oracle.dequant_int4(packed, np.ones((2, 1), np.float32), np.zeros((2, 1), np.float32), 3, 2, 32)
    assert W.tolist() == [[-7.0, -6.0, -5.0], [-4.0, -3.0, -2.0]]


def test_matmul_is_k_ascending_fp32():
    # 2^24 + 1 + 1: k-ascending fp32 accumulation loses both ones, a pairwise sum would not
    A = np.array([[16777216.0, 1.0, 1.0]], np.float32)
    B = np.ones((1, 3), np.float32)
    assert oracle.matmul(A, B)[0, 0] == np.float32(16777216.0)


def test_threads_do_not_change_results():
    rng = np.random.default_rng(3)
    M, N, K, g = 3, 37, 64, 32
    A = rng.standard_normal((M, K)).astype(np.float32)
    wq = rng.integers(0, 256, (N, K // 2), dtype=np.uint8)
    s = rng.uniform(0.005, 0.02, (N, K // g)).astype(np.float32)
    z = rng.uniform(-0.1, 0.1, (N, K // g)).astype(np.float32)
    c1 = oracle.dequant_matmul(A, wq, s, z, g, "int4", threads=1)
    c5 = oracle.dequant_matmul(A, wq, s, z, g, "int4", threads=5)
    assert np.array_equal(c1, c5)
    w8 = rng.integers(-127, 128, (N, K), dtype=np.int8)
    assert np.array_equal(oracle.dequant_matmul(A, w8, s, None, g, "int8", threads=1),
                          oracle.dequant_matmul(A, w8, s, None, g, "int8", threads=4))


def test_fp16_helpers():
    L = oracle.lib()
    # exhaustive: every finite fp16 survives widen -> RN narrow, and matches numpy
    bits = np.arange(0x10000, dtype=np.uint32).astype(np.uint16)
    wide = oracle.fp16_bits_to_fp32(bits)
    ref = bits.view(np.float16).astype(np.float32)
    finite = np.isfinite(ref)
    assert np.array_equal(wide[finite], ref[finite])
    assert np.array_equal(oracle.fp32_to_fp16_bits(wide[finite]), bits[finite])
    # RN narrowing agrees with numpy on random and on tie values
    rng = np.random.default_rng(0)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 10,
                        rng.uniform(-1e-6, 1e-6, 5000).astype(np.float32),
                        np.array([65504.0, 65519.9, 65520.0, 1e9, 2.0 ** -25, 2.0 ** -24,
                                  1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -11, -0.0], np.float32)])
    with np.errstate(over="ignore"):
        assert np.array_equal(oracle.fp32_to_fp16_bits(x), x.astype(np.float16).view(np.uint16))
    # the fixture's own narrowing truncates (tests/cpp/test_dequant_matmul.mm:258)
    assert L.oracle_fp32_to_fp16_trunc(0.1) == 0x2E66
    assert L.oracle_fp32_to_fp16_rn(0.1) == 0x2E66
    assert L.oracle_fp32_to_fp16_trunc(0.05) == 0x2A66      # 0.05f = 0x3D4CCCCD -> truncated
    assert oracle.fp32_to_fp16_bits(np.array([0.05], np.float32))[0] == 0x2A66
    assert L.oracle_fp32_to_fp16_trunc(1.0 + 3 * 2.0 ** -11) == 0x3C01
    assert L.oracle_fp32_to_fp16_rn(1.0 + 3 * 2.0 ** -11) == 0x3C02


def test_bf16_helpers():
    import torch

    x = torch.randn(10000, dtype=torch.float32) * 7
    bits = oracle.fp32_to_bf16_bits(x.numpy())
    ref = x.to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)
    assert np.array_equal(bits, ref)
    back = oracle.bf16_bits_to_fp32(bits)
    assert np.array_equal(back, x.to(torch.bfloat16).float().numpy())


def test_dequantize_flat_matches_shader_semantics():
    # shaders/dequantize_kernel.metal:26-54: out[2j] = half((b&15)-8)*s, out[2j+1] = half((b>>4)-8)*s,
    # flat group index i / group_size, no zero-point
    b = np.array([0x80, 0xF0, 0x07, 0x21], np.uint8)       # q = 0,8 | 0,15 | 7,0 | 1,2
    s = np.array([0.5, 0.25], np.float16)
    out = oracle.dequantize_flat(b, s.view(np.uint16), 8, 4, "int4").view(np.float16)
    assert out.tolist() == [-4.0, 0.0, -4.0, 3.5, -0.25, -2.0, -1.75, -1.5]
    # odd element count: the last high nibble is not written
    out7 = oracle.dequantize_flat(b, s.view(np.uint16), 7, 4, "int4").view(np.float16)
    assert out7.tolist() == [-4.0, 0.0, -4.0, 3.5, -0.25, -2.0, -1.75]
    # int8 (:9-22)
    q = np.array([-128, 127, 3, -3, 10], np.int8)
    s8 = np.array([0.5, 0.1], np.float16)
    o8 = oracle.dequantize_flat(q, s8.view(np.uint16), 5, 4, "int8").view(np.float16)
    exp = [np.float16(np.float32(v) * np.float32(sc)) for v, sc in
           zip([-128, 127, 3, -3, 10], [s8[0]] * 4 + [s8[1]])]
    assert o8.tolist() == [float(e) for e in exp]
