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
    return metal_native._C


def _static_call(C, L, out):
    stream = torch.cuda.current_stream().cuda_stream
    dt = {torch.float16: C.FP16, torch.bfloat16: C.BF16}
    return C._lib.mnq_dequant_matmul_static(
        L.x.data_ptr(), L.wq.data_ptr(), L.scales.data_ptr(), L.zeros.data_ptr() if L.zeros is not None else None,
        out.data_ptr(), L.M, L.N, L.K, L.K, L.N, L.group_size, C.INT4 if L.quant_type == "int4" else C.INT8,
        dt[L.x.dtype], dt[L.scales.dtype], stream)


def _free_bytes():
    free, _total = torch.cuda.mem_get_info()
    return free


CASES = [(1, 4096, 512, "int4", 128),      # few rows: K is split, counters and partial sums in the array
         (5, 8192, 256, "int8", 8192),
         (64, 8192, 2048, "int4", 128),    # tensor-core path: K-split planes [split][M][N] in the same array
         (1, 1024, 8192, "int4", 128)]     # many rows


@pytest.mark.parametrize("M,K,N,quant,g", CASES)
def test_static_entry_point_matches_the_ordinary_one_twice(C, M, K, N, quant, g):
    import mnq_workloads as workloads
    L = workloads.make_layer("t", M, K, N, quant_type=quant, group_size=g, asymmetric=(quant == "int4"),
                             seed=K + N).to("cuda")
    expected = C.dequant_matmul(*L.args())
    out = torch.empty((M, N), dtype=L.x.dtype, device="cuda")
    # a dry run of everything the loop below does: the first call on a device looks the array's address
    # up, and a kernel's first launch (ours, or torch's fill and compare) loads its code into device memory
    out.fill_(float("nan"))
    assert _static_call(C, L, out) == 0, C._lib.mnq_last_error().decode()
    torch.cuda.synchronize()
    assert torch.equal(out, expected)
    free_before, torch_before = _free_bytes(), torch.cuda.memory_allocated()
    for call in range(2):                       # the second call finds the scratch as the first left it
        out.fill_(float("nan"))
        rc = _static_call(C, L, out)
        assert rc == 0, C._lib.mnq_last_error().decode()
        torch.cuda.synchronize()
        # same kernels, same plan, same order of additions: the same bits
        assert torch.equal(out, expected), f"call {call}: differs from the ordinary entry point"
    # the point of the entry point: it allocated nothing, on the device or through torch
    assert _free_bytes() == free_before and torch.cuda.memory_allocated() == torch_before
    assert C.device_status() == 0


def test_decode_and_tensor_core_layouts_share_the_array(C):
    """A tensor-core call leaves fp32 planes where a decode call's partial sums go, and the other
    way round; each call clears the counters it needs, so alternating them stays exact."""
    import mnq_workloads as workloads
    layers = [workloads.make_layer("t", M, K, N, quant_type=q, group_size=g, asymmetric=(q == "int4"), seed=N).to("cuda")
              for (M, K, N, q, g) in CASES[:3]]
    want = [C.dequant_matmul(*L.args()) for L in layers]
    outs = [torch.empty_like(w) for w in want]
    for _ in range(2):
        for L, o in zip(layers, outs):
            assert _static_call(C, L, o) == 0, C._lib.mnq_last_error().decode()
    torch.cuda.synchronize()
    for w, o in zip(want, outs):
        assert torch.equal(o, w)
    # and through the shim's binding of the same entry point
    o = torch.empty_like(want[0])
    assert torch.equal(C.dequant_matmul_static(*layers[0].args(), out=o), want[0])


def test_static_entry_point_refuses_oversized_problems(C):
    # M = 32 rows of 57344 outputs would want more split-K scratch than the built-in 4 MiB
    need = C._lib.mnq_workspace_bytes(32, 57344, 8192, 8192, C.INT8)
    assert need > 4 << 20
    fake = 1 << 20
    rc = C._lib.mnq_dequant_matmul_static(fake, fake, fake, None, fake, 32, 57344, 8192, 8192, 57344, 8192, C.INT8,
                                          C.BF16, C.FP16, None)
    assert rc == 4   # InvalidArgument, before anything is launched
    assert "built-in area" in C._lib.mnq_last_error().decode()
