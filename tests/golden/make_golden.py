"""Writes tests/golden/reference_kats.json: the value-checked cases of the reference's
own test for the dequant-matmul path (tests/cpp/test_dequant_matmul.mm), with
expected outputs.

The reference's Python package cannot be imported without its Metal extension, and
its CPU helpers live inside an Objective-C++ fixture, so nothing here imports the
reference.  Inputs are the literals / index formulas the fixture uses; expected
outputs are
  * the numbers written in the fixture where it has them (INT4_SmallKnownAnswer:
    [-3.3, -9.0], tolerance 0.2, :334-335), and
  * for the formula-seeded square cases (:338-398, :651-705), where the fixture only
    compares its GPU result with its own CPU helper, an independent float64
    evaluation of w = (q-8)*s - z (int4) / q*s - z (int8) and C = A . W^T,
    done here with numpy and no oracle code.

A second file, tests/golden/reference_cpu_outputs.json, holds outputs of the reference's own
CPU helpers (tests/cpp/test_dequant_matmul.mm:103-259, compiled from the reference checkout
into oracle/_ref/libmnref.so by oracle/build_ref.py) on small seeded cases the fixture never
checks: non-zero zeros, several groups per row, a ragged last group, odd K, int8.  It is
written only where that library exists; inputs and outputs are stored as fp32 bit patterns.

Run:  python tests/golden/make_golden.py
"""
import sys
import json
from pathlib import Path

import numpy as np


def small_int4():
    return {
        "name": "INT4_SmallKnownAnswer", "ref": "tests/cpp/test_dequant_matmul.mm:269-336",
        "quant": "int4", "M": 1, "N": 2, "K": 4, "group_size": 32,
        "A": [1.0, 2.0, 3.0, 4.0],
        "q": [3, 5, 2, 7, 1, 4, 6, 2],
        "scales": [0.1, 0.2], "zeros": [0.0, 0.0],
        "expected": [-3.3, -9.0], "expected_source": "literal in the fixture (:334-335)",
        "ref_tol": 0.2,
        "packed": [0x53, 0x72, 0x41, 0x26],
    }


def small_int8():
    # The fixture asserts only the shape here (:612-649); the answer follows from its data.
    return {
        "name": "INT8_SmallKnownAnswer", "ref": "tests/cpp/test_dequant_matmul.mm:612-649",
        "quant": "int8", "M": 1, "N": 2, "K": 4, "group_size": 32,
        "A": [1.0, 2.0, 3.0, 4.0],
        "q": [10, 20, 30, 40, 5, 15, 25, 35],
        "scales": [0.1, 0.1], "zeros": [0.0, 0.0],
        "expected": [30.0, 25.0], "expected_source": "hand-computed from the fixture's data",
        "ref_tol": 1e-2,
    }


def square(quant):
    M = N = 16
    K = 32
    g = 32
    A = np.array([((i % 7) - 3.0) * 0.5 for i in range(M * K)], np.float64).reshape(M, K)
    if quant == "int4":
        q = np.array([i % 16 for i in range(N * K)], np.int64).reshape(N, K)
        centred = q - 8
        tol, ref, name = 5e-2, "tests/cpp/test_dequant_matmul.mm:338-398", "INT4_SquareMatrix"
    else:
        q = np.array([(i % 50) - 25 for i in range(N * K)], np.int64).reshape(N, K)
        centred = q
        tol, ref, name = 1e-2, "tests/cpp/test_dequant_matmul.mm:651-705", "INT8_SquareMatrix"
    s = float(np.float32(0.05))  # the fixture's CPU helper consumes the fp32 literal 0.05f
    W = centred.astype(np.float64) * s
    C = A @ W.T
    return {
        "name": name, "ref": ref, "quant": quant, "M": M, "N": N, "K": K, "group_size": g,
        "A": A.ravel().tolist(), "q": q.ravel().tolist(),
        "scales": [0.05] * N, "zeros": [0.0] * N,
        "expected": C.ravel().tolist(),
        "expected_source": "float64 numpy evaluation in make_golden.py",
        "ref_tol": tol,
    }


def reference_outputs():
    """Small seeded cases through the reference's own helpers."""
    sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
    from oracle import ref
    if not ref.available():
        print("oracle/_ref/libmnref.so is not built: reference_cpu_outputs.json left as it is")
        return
    rng = np.random.default_rng(20240607)
    cases = []
    for name, quant, M, N, K, g in [("int4_zeros_groups", "int4", 2, 5, 64, 32), ("int4_ragged_group", "int4", 1, 3, 80, 32),
                                    ("int4_odd_K", "int4", 1, 2, 7, 32), ("int8_zeros_groups", "int8", 3, 4, 96, 32),
                                    ("int8_per_channel", "int8", 1, 6, 40, 40), ("int4_g64", "int4", 1, 4, 256, 64)]:
        G = (K + g - 1) // g
        x = rng.standard_normal((M, K)).astype(np.float16).astype(np.float32)
        s = rng.uniform(0.005, 0.02, (N, G)).astype(np.float16).astype(np.float32)
        z = ((rng.integers(0, 16, (N, G)) - 8) * s).astype(np.float16).astype(np.float32)
        if quant == "int4":
            q = rng.integers(0, 16, (N, K)).astype(np.int8)
            wq = np.stack([ref.pack_int4(q[n]) for n in range(N)])
        else:
            wq = rng.integers(-127, 128, (N, K)).astype(np.int8)
        w = ref.dequant(wq, s, z, K, N, g, quant)
        out = ref.matmul(x, w)
        cases.append({"name": name, "quant": quant, "M": M, "N": N, "K": K, "group_size": g,
                      "x_bits": x.view(np.uint32).ravel().tolist(), "scales_bits": s.view(np.uint32).ravel().tolist(),
                      "zeros_bits": z.view(np.uint32).ravel().tolist(), "wq": wq.astype(np.int16).ravel().tolist()
                      if quant == "int8" else wq.ravel().tolist(),
                      "w_bits": w.view(np.uint32).ravel().tolist(), "out_bits": out.view(np.uint32).ravel().tolist(),
                      "source": "reference helpers dequant_reference_int4/int8 + matmul_reference via oracle/_ref"})
    out_path = Path(__file__).with_name("reference_cpu_outputs.json")
    out_path.write_text(json.dumps({"cases": cases}) + "\n")
    print("wrote", out_path, "with", len(cases), "cases")


def main():
    cases = [small_int4(), small_int8(), square("int4"), square("int8")]
    out = Path(__file__).with_name("reference_kats.json")
    out.write_text(json.dumps({"cases": cases}, indent=1) + "\n")
    print("wrote", out, "with", len(cases), "cases")
    reference_outputs()


if __name__ == "__main__":
    main()
