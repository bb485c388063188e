"""The allocation-free entry point, mnq_dequant_matmul_static, called through the C ABI.

It exists for callers that are only handed input and output buffers and may not allocate
device memory themselves (plugins of a runtime that owns all memory, allocator callbacks,
serving loops with a frozen budget): the split-K scratch sits in a fixed array inside the
library instead of a caller-provided workspace.  Its results must equal those of the
ordinary entry point, call after call, because both run the same kernels.

This file sorts last on purpose: a run that stops at the first failure has then already
run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def C():
    import metal_native
    assert torch.cuda.is_available()
    lib = metal_native._C._lib
    i32, i64, vp = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p
    lib.mnq_dequant_matmul_static.restype = ctypes.c_int
    lib.mnq_dequant_matmul_static.argtypes = [vp, vp, vp, vp, vp, i64, i64, i64, i64, i64, i32, i32, i32, i32, vp]
    return metal_native._C


def _static_call(C, L, out):
    stream = torch.cuda.current_stream().cuda_stream
    dt = {torch.float16: C.FP16, torch.bfloat16: C.BF16}
    return C._lib.mnq_dequant_matmul_static(
        L.x.data_ptr(), L.wq.data_ptr(), L.scales.data_ptr(), L.zeros.data_ptr() if L.zeros is not None else None,
        out.data_ptr(), L.M, L.N, L.K, L.K, L.N, L.group_size, C.INT4 if L.quant_type == "int4" else C.INT8,
        dt[L.x.dtype], dt[L.scales.dtype], stream)


@pytest.mark.parametrize("M,K,N,quant,g", [(1, 4096, 512, "int4", 128),      # few rows: K is split, scratch in use
                                           (5, 8192, 256, "int8", 8192),
                                           (1, 1024, 8192, "int4", 128)])    # many rows: no split needed
def test_static_entry_point_matches_the_ordinary_one_twice(C, M, K, N, quant, g):
    from metal_native import workloads
    L = workloads.make_layer("t", M, K, N, quant_type=quant, group_size=g, asymmetric=(quant == "int4"),
                             seed=K + N).to("cuda")
    expected = C.dequant_matmul(*L.args())
    torch.cuda.synchronize()
    for call in range(2):                       # the second call finds the scratch as the first left it
        out = torch.full((M, N), float("nan"), dtype=L.x.dtype, device="cuda")
        rc = _static_call(C, L, out)
        assert rc == 0, C._lib.mnq_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all(), f"call {call}: output not fully written"
        # same kernels, same plan: equal up to the test suite's matmul tolerance
        err = (out.float() - expected.float()).norm() / expected.float().norm()
        assert float(err) <= 1e-3, f"call {call}: rel-L2 {float(err):.3e}"
        assert float((out.float() - expected.float()).abs().max()) <= 2e-2
    assert C.device_status() == 0


def test_static_entry_point_refuses_oversized_problems(C):
    # M = 32 rows of 57344 outputs would want more split-K scratch than the built-in 4 MiB
    need = C._lib.mnq_workspace_bytes(32, 57344, 8192, 8192, C.INT8)
    assert need > 4 << 20
    fake = 1 << 20
    rc = C._lib.mnq_dequant_matmul_static(fake, fake, fake, None, fake, 32, 57344, 8192, 8192, 57344, 8192, C.INT8,
                                          C.BF16, C.FP16, None)
    assert rc == 4   # InvalidArgument, before anything is launched
    assert "built-in area" in C._lib.mnq_last_error().decode()
