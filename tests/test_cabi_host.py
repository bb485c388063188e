"""Host-side checks that need no GPU: the C-ABI library loads and exports every symbol
include/mnq.h declares, its argument validation answers before any CUDA call, and the
kernel-selection logic picks the intended family for the benchmark shapes."""
import ctypes
import re
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parents[1]
HEADER = ROOT / "include" / "mnq.h"


@pytest.fixture(scope="module")
def C():
    import metal_native
    return metal_native._C


def declared_symbols():
    text = HEADER.read_text()
    return sorted(set(re.findall(r"MNQ_API[^;(]*?\b(mnq_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol(C):
    syms = declared_symbols()
    assert len(syms) >= 9
    lib = ctypes.CDLL(C.library_path())
    for name in syms:
        assert hasattr(lib, name), f"{name} is declared in include/mnq.h but not exported"
    assert set(C.exported_symbols()) <= set(syms)


def test_status_names_match_reference_enum(C):
    names = ["Success", "DeviceNotFound", "AllocationFailed", "KernelCompilationFailed", "InvalidArgument",
             "OutOfMemory", "TimeoutError", "InternalError", "NotImplemented"]
    assert [C._status_name(i) for i in range(9)] == names
    assert C._status_name(99) == "Unknown"
    assert re.fullmatch(r"\d+\.\d+\.\d+", C.version())


FAKE = 1 << 20  # an aligned non-null address; validation never dereferences it


def _mm(C, M=1, N=64, K=128, lda=None, ldc=None, g=128, q=0, adt=0, sdt=0, x=FAKE, w=FAKE, s=FAKE, out=FAKE):
    return C._lib.mnq_dequant_matmul(x, w, s, None, out, M, N, K, K if lda is None else lda,
                                     N if ldc is None else ldc, g, q, adt, sdt, None, 0, None)


@pytest.mark.parametrize("kw,msg", [
    (dict(adt=2), "activations must be Float16 or BFloat16"),
    (dict(g=48), "group_size must be"),
    (dict(g=0), "group_size must be"),
    (dict(q=2), "quant_type must be INT4 or INT8"),
    (dict(sdt=2), "scales must be Float16 or BFloat16"),
    (dict(M=-1), "negative dimension"),
    (dict(K=127, g=128), "K must be even"),
    (dict(lda=64), "lda must be >= K"),
    (dict(ldc=8), "ldc must be >= N"),
    (dict(x=None), "null activations, weights_packed or scales"),
    (dict(out=None), "null output"),
])
def test_validation_runs_on_the_host(C, kw, msg):
    rc = _mm(C, **kw)
    assert rc == 4, rc   # InvalidArgument
    assert msg in C._lib.mnq_last_error().decode()


def test_empty_problem_is_success_without_a_device(C):
    assert _mm(C, M=0) == 0
    assert _mm(C, N=0) == 0


def test_shim_rejects_cpu_tensors_and_bad_strings(C):
    x = torch.zeros((1, 128), dtype=torch.float16)
    w = torch.zeros((64, 64), dtype=torch.uint8)
    s = torch.ones((64, 1), dtype=torch.float16)
    with pytest.raises(C.MetalNativeError, match="InvalidArgument: .*CUDA tensor"):
        C.dequant_matmul(x, w, s, None, 128, "int4")
    with pytest.raises(C.MetalNativeError, match="quant_type must be 'int4' or 'int8'"):
        C.dequant_matmul(x, w, s, None, 128, "INT4")
    e = C.MetalNativeError(7, "boom")
    assert str(e) == "InternalError: boom" and e.code == 7


def test_kernel_selection_for_benchmark_shapes(C):
    sp = C.select_path
    # decode shapes stream through the GEMV kernels
    assert sp(1, 896, 4864, 64, "int4") == "gemv"                      # config 0
    assert sp(1, 37888, 3584, 128, "int4") == "gemv"                   # config 1
    assert sp(1, 3584, 18944, 128, "int4") == "gemv"
    for M in (4, 16, 32):                                              # config 2
        assert sp(M, 14336, 4096, 128, "int4", torch.bfloat16) == "gemv"
        assert sp(M, 4096, 14336, 128, "int4", torch.bfloat16) == "gemv"
    assert sp(1, 57344, 8192, 8192, "int8", torch.bfloat16) == "gemv"  # config 4, M=1
    assert sp(1, 8192, 28672, 28672, "int8", torch.bfloat16) == "gemv"
    # shapes no vector path can take fall to the guarded kernel, never to an error
    assert sp(1, 2, 4, 32, "int4") == "generic"                        # the reference's known-answer shape
    assert sp(3, 9, 7, 32, "int8") == "generic"
    # unaligned weight base address: narrower loads, then the guarded kernel
    assert sp(1, 64, 128, 128, "int4", alignment=256) == "gemv"


def test_workspace_bytes(C):
    wb = C._lib.mnq_workspace_bytes
    assert wb(0, 64, 128, 128, 0) == 0
    assert wb(512, 18944, 3584, 128, 0) == 0     # enough tiles to fill the GPU: no split-K workspace
    assert wb(512, 3584, 18944, 128, 0) == (64 << 10) + 5 * 512 * 3584 * 4   # 28 tiles: K split 5 ways, one fp32 plane each
    small = wb(1, 3584, 18944, 128, 0)
    assert 3584 * 4 * 2 < small < 4 << 20
    assert wb(32, 57344, 8192, 8192, 1) < 64 << 20


def test_gather_entry_point_validates_before_any_cuda_call(C):
    """mnq_dequant_matmul_gather rejects a bad rank table without touching a device."""
    import ctypes
    vp = ctypes.c_void_p
    one = (vp * 1)(vp(4096))
    none = (vp * 1)(vp(None))
    call = C._lib.mnq_dequant_matmul_gather
    base = (vp(4096), vp(4096), vp(4096), None)
    tail = (0, 1, 64, 128, 128, 64, 128, C.INT4, C.FP16, C.FP16, None, 0, None)
    assert call(*base, one, one, 0, 0, *tail) == 4          # world 0
    assert call(*base, one, one, 9, 0, *tail) == 4          # world too large
    assert call(*base, one, one, 1, 1, *tail) == 4          # rank outside the world
    assert call(*base, none, one, 1, 0, *tail) == 4         # null output buffer
    assert call(*base, one, one, 1, 0, 32, 1, 64, 128, 128, 64, 128, C.INT4, C.FP16, C.FP16, None, 0, None) \
        == 4                                                # columns past ldc
    assert b"ldc" in C._lib.mnq_last_error()
