"""Parity of the CUDA kernels with the CPU oracle, through the Python shim that calls the
C ABI (libmnq.so).  Needs a B200; run with -m gpu."""
import json
from pathlib import Path

import numpy as np
import pytest
import torch

from oracle import oracle
from oracle import check as H

pytestmark = pytest.mark.gpu

GOLDEN = json.loads((Path(__file__).parent / "golden" / "reference_kats.json").read_text())


@pytest.fixture(scope="module")
def mn():
    import metal_native
    assert torch.cuda.is_available()
    return metal_native


def _tuning(mn, **kw):
    t = mn._C.Tuning()
    for k, v in kw.items():
        setattr(t, k, v)
    return t


# --------------------------------------------------------------------------- dequantise

@pytest.mark.parametrize("quant,N,K,g,zeros,sdt", [
    ("int4", 896, 4864, 64, True, torch.float16),      # config 0, whole matrix
    ("int4", 512, 3584, 128, True, torch.float16),     # config 1 rows
    ("int4", 300, 4096, 128, False, torch.bfloat16),   # config 2 style
    ("int8", 256, 8192, 8192, False, torch.float16),   # config 4 style (per channel)
    ("int4", 7, 48, 32, True, torch.float16),          # ragged: K % 8 == 0 but tiny
    ("int4", 5, 6, 32, True, torch.float16),           # K % 8 != 0 -> scalar kernel
    ("int8", 3, 5, 4, True, torch.float16),            # odd K int8, ragged last group
    ("int8", 64, 256, 32, True, torch.bfloat16),
])
def test_dequantize_bit_exact(mn, quant, N, K, g, zeros, sdt):
    import mnq_workloads as workloads
    L = workloads.make_layer("t", 1, K, N, quant_type=quant, group_size=g, scale_dtype=sdt,
                             asymmetric=zeros, seed=11)
    ref = H.oracle_dequant(L)
    d = L.to("cuda")
    w32 = mn.dequantize(d.wq, d.scales, d.zeros, g, quant, torch.float32).cpu().numpy()
    assert np.array_equal(w32.view(np.uint32), ref.view(np.uint32)), "fp32 dequantised weights differ"
    w16 = mn.dequantize(d.wq, d.scales, d.zeros, g, quant, torch.float16).cpu()
    assert torch.equal(w16, torch.from_numpy(ref).to(torch.float16))
    wb = mn.dequantize(d.wq, d.scales, d.zeros, g, quant, torch.bfloat16).cpu()
    assert torch.equal(wb, torch.from_numpy(ref).to(torch.bfloat16))


@pytest.mark.parametrize("quant,n,g", [("int4", 4096 * 64, 64), ("int8", 4096 * 32, 128),
                                       ("int4", 1001, 32), ("int8", 77, 16), ("int4", 14, 4)])
def test_dequantize_flat_matches_reference_kernels(mn, quant, n, g):
    gen = torch.Generator().manual_seed(5)
    nbytes = (n + 1) // 2 if quant == "int4" else n
    q = torch.randint(0, 256, (nbytes,), generator=gen, dtype=torch.uint8)
    s = (torch.rand(((n + g - 1) // g,), generator=gen) * 0.02 + 0.001).to(torch.float16)
    ref = oracle.dequantize_flat(q.numpy(), s.view(torch.int16).numpy().view(np.uint16), n, g, quant)
    got = mn.dequantize_flat(q.cuda(), s.cuda(), g, quant, n).cpu()
    assert np.array_equal(got.view(torch.int16).numpy().view(np.uint16), ref)


def test_quant_weight_cache(mn):
    gen = torch.Generator().manual_seed(6)
    q = torch.randint(0, 256, (64, 128), generator=gen, dtype=torch.uint8).cuda()   # int4 [64, 256]
    s = (torch.rand((64, 4), generator=gen) * 0.02).to(torch.float16).cuda()        # group 64
    cache = mn.QuantWeightCache(pressure_fn=lambda: 1.0)
    cache.register_weight("w", q, s, mn.QuantFormat.INT4)
    w = cache.get_dequantized("w")
    assert w.shape == (64, 256) and w.dtype == torch.float16
    ref = oracle.dequantize_flat(q.cpu().numpy(), s.cpu().view(torch.int16).numpy().view(np.uint16),
                                 64 * 256, 64, "int4")
    assert np.array_equal(w.cpu().view(torch.int16).numpy().view(np.uint16).ravel(), ref)
    assert cache.get_dequantized("w") is w                      # cached
    assert cache.dequantized_footprint() == 64 * 256 * 2
    assert cache.total_footprint() == 64 * 128 + 64 * 4 * 2 + 64 * 256 * 2
    cache.evict_dequantized()
    assert cache.dequantized_footprint() == 0
    low = mn.QuantWeightCache(pressure_fn=lambda: 0.1)          # under pressure: not cached
    low.register_weight("w", q, s, mn.QuantFormat.INT4)
    low.get_dequantized("w")
    assert low.dequantized_footprint() == 0
    with pytest.raises(mn.MetalNativeError, match="InvalidArgument: quant_weight_cache: weight not registered"):
        cache.get_dequantized("nope")


# --------------------------------------------------------------------------- known answers

@pytest.mark.parametrize("case", GOLDEN["cases"], ids=[c["name"] for c in GOLDEN["cases"]])
def test_reference_known_answers_on_gpu(mn, case):
    M, N, K, g = case["M"], case["N"], case["K"], case["group_size"]
    x = torch.tensor(case["A"], dtype=torch.float32).reshape(M, K).to(torch.float16)
    s = torch.tensor(case["scales"], dtype=torch.float32).reshape(N, 1).to(torch.float16)
    z = torch.tensor(case["zeros"], dtype=torch.float32).reshape(N, 1).to(torch.float16)
    if case["quant"] == "int4":
        wq = torch.from_numpy(oracle.pack_int4(np.array(case["q"], np.int8)).reshape(N, K // 2))
    else:
        wq = torch.tensor(case["q"], dtype=torch.int8).reshape(N, K)
    out = mn._C.dequant_matmul(x.cuda(), wq.cuda(), s.cuda(), z.cuda(), g, case["quant"])
    mn._C.synchronize()
    exp = np.array(case["expected"], np.float64).reshape(M, N)
    got = out.cpu().float().numpy()
    assert out.dtype == torch.float16 and out.shape == (M, N)
    assert np.max(np.abs(got - exp)) <= case["ref_tol"]
    # and against the oracle fed the same fp16 bits
    ref = oracle.dequant_matmul(H.f32(x), wq.numpy(), H.f32(s), H.f32(z), g, case["quant"])
    H.assert_close_to_oracle(out, ref, case["name"])


# --------------------------------------------------------------------------- shape sweep

SWEEP = [
    # quant, M, N, K, g, asym, act dtype, scale dtype
    ("int4", 1, 64, 128, 32, True, torch.float16, torch.float16),     # reference VecMat shape
    ("int4", 4, 64, 128, 32, True, torch.float16, torch.float16),     # reference VecMatBatch: all rows
    ("int4", 4, 8, 48, 32, True, torch.float16, torch.float16),       # reference NonAlignedK
    ("int4", 4, 48, 32, 32, True, torch.float16, torch.float16),      # reference NonAlignedN
    ("int4", 16, 32, 128, 32, True, torch.float16, torch.float16),    # reference GroupSize_Variants
    ("int4", 16, 32, 128, 64, True, torch.float16, torch.float16),
    ("int4", 16, 32, 128, 128, True, torch.float16, torch.float16),
    ("int4", 1, 100, 512, 128, True, torch.float16, torch.float16),   # N not a multiple of 16
    ("int4", 3, 130, 1024, 128, False, torch.float16, torch.float16),
    ("int4", 8, 257, 2048, 128, True, torch.bfloat16, torch.bfloat16),
    ("int4", 9, 64, 640, 128, True, torch.float16, torch.float16),    # K not a multiple of step*U
    ("int4", 17, 48, 384, 64, True, torch.bfloat16, torch.float16),
    ("int4", 32, 200, 1536, 128, False, torch.bfloat16, torch.bfloat16),
    ("int4", 2, 33, 96, 96, True, torch.float16, torch.float16),      # g == K (single group), K%128 != 0
    ("int4", 5, 16, 200, 1 << 20, False, torch.float16, torch.float16),  # g > K, K % 32 != 0 -> LW 4
    ("int8", 1, 64, 256, 64, True, torch.float16, torch.float16),
    ("int8", 1, 96, 512, 512, False, torch.bfloat16, torch.float16),  # per channel, config 4 style
    ("int8", 7, 40, 192, 32, True, torch.float16, torch.float16),
    ("int8", 12, 130, 1024, 128, True, torch.bfloat16, torch.bfloat16),
    ("int8", 32, 72, 320, 64, False, torch.float16, torch.float16),
    ("int8", 2, 20, 100, 100, True, torch.float16, torch.float16),    # K % 16 != 0 -> LW 4
    ("int8", 3, 9, 7, 32, True, torch.float16, torch.float16),        # odd K -> generic kernel
    ("int4", 2, 5, 6, 32, True, torch.float16, torch.float16),        # tiny K -> generic kernel
    ("int4", 40, 70, 96, 32, True, torch.float16, torch.float16),     # M > 32, K % 64 != 0 -> generic
    ("int8", 33, 10, 24, 24, False, torch.bfloat16, torch.bfloat16),
]


@pytest.mark.parametrize("quant,M,N,K,g,asym,adt,sdt", SWEEP)
def test_shape_sweep(mn, quant, M, N, K, g, asym, adt, sdt):
    import mnq_workloads as workloads
    L = workloads.make_layer("t", M, K, N, quant_type=quant, group_size=g, act_dtype=adt,
                             scale_dtype=sdt, asymmetric=asym, seed=M * 1000 + N + K)
    ref = H.oracle_matmul(L, threads=1)
    d = L.to("cuda")
    # output with a leading dimension larger than N and canaries around it
    buf = torch.full((M + 2, N + 5), 777.0, dtype=adt, device="cuda")
    out = buf[1:M + 1, 2:N + 2]
    mn._C.dequant_matmul(*d.args(), out=out)
    mn._C.synchronize()
    H.assert_close_to_oracle(out, ref, f"{quant} {M}x{N}x{K} g{g}")
    chk = buf.clone()
    chk[1:M + 1, 2:N + 2] = 777.0
    assert bool((chk == 777.0).all()), "kernel wrote outside its [M, N] output block"


@pytest.mark.parametrize("split", [1, 2, 3, 7])
@pytest.mark.parametrize("quant,M,g,adt", [("int4", 1, 128, torch.float16), ("int4", 6, 128, torch.bfloat16),
                                           ("int8", 20, 4096, torch.bfloat16), ("int4", 3, 64, torch.float16)])
def test_split_k_reduction_and_workspace_reuse(mn, split, quant, M, g, adt):
    import mnq_workloads as workloads
    K = 4096
    L = workloads.make_layer("t", M, K, 272, quant_type=quant, group_size=g, act_dtype=adt,
                             scale_dtype=torch.float16, asymmetric=(quant == "int4"), seed=split)
    ref = H.oracle_matmul(L, threads=4)
    d = L.to("cuda")
    t = _tuning(mn, path=mn._C.PATH_GEMV, split_k=split, warps_per_cta=4)
    outs = [mn._C.dequant_matmul(*d.args(), tuning=t) for _ in range(3)]   # same workspace, three times
    mn._C.synchronize()
    H.assert_close_to_oracle(outs[0], ref, f"split {split}")
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2]), "split-K result is not deterministic"


@pytest.mark.parametrize("quant,M,N,K,g,asym,adt", [
    ("int4", 1, 4096, 3584, 128, True, torch.float16),      # a step is a group: scales as 8-byte loads
    ("int4", 1, 528, 18944, 128, True, torch.float16),      # few rows: K split, last-arriver reduction
    ("int4", 4, 1000, 4096, 128, False, torch.bfloat16),    # bf16 activations and scales, ragged last row block
    ("int4", 8, 2048, 2048, 128, True, torch.bfloat16),
    ("int8", 1, 2048, 8192, 8192, False, torch.bfloat16),   # one group per row
    ("int8", 6, 272, 28672, 28672, False, torch.bfloat16),  # one group per row, K split
    ("int8", 3, 1024, 1024, 64, True, torch.float16),       # int8 with a group per step
])
def test_compact_and_general_decode_kernels(mn, quant, M, N, K, g, asym, adt):
    """Shapes the compact decode kernel takes, through it (the default) and through the general
    streaming kernel (kernel variant 3): both against the oracle, twice in a row on one workspace."""
    import mnq_workloads as workloads
    C = mn._C
    L = workloads.make_layer("t", M, K, N, quant_type=quant, group_size=g, act_dtype=adt,
                             scale_dtype=adt if quant == "int4" else torch.float16, asymmetric=asym, seed=N + K)
    ref = H.oracle_matmul(L)
    d = L.to("cuda")
    general = _tuning(mn, gemv_variant=3)
    compact = _tuning(mn, gemv_variant=4)   # (from 5 tokens the default is the batched kernel)
    for call in range(2):
        a = C.dequant_matmul(*d.args())
        b = C.dequant_matmul(*d.args(), tuning=general)
        c = C.dequant_matmul(*d.args(), tuning=compact)
        C.synchronize()
        assert C.device_status() == 0
        H.assert_close_to_oracle(a, ref, f"default {quant} {M}x{N}x{K} call {call}")
        H.assert_close_to_oracle(b, ref, f"general {quant} {M}x{N}x{K} call {call}")
        H.assert_close_to_oracle(c, ref, f"compact {quant} {M}x{N}x{K} call {call}")
    a32 = C.dequant_matmul_fused(*d.args(), out_dtype=torch.float32)
    H.assert_fp32_gate(a32, ref, f"compact fp32 {quant} {M}x{N}x{K}")


def test_activation_row_stride_and_unaligned_views(mn):
    import mnq_workloads as workloads
    L = workloads.make_layer("t", 4, 256, 64, seed=3)
    ref = H.oracle_matmul(L, threads=1)
    d = L.to("cuda")
    wide = torch.zeros((4, 300), dtype=torch.float16, device="cuda")
    wide[:, 3:259] = d.x                      # lda = 300, base address 6 bytes past alignment
    out = mn._C.dequant_matmul(wide[:, 3:259], d.wq, d.scales, d.zeros, d.group_size, "int4")
    H.assert_close_to_oracle(out, ref, "strided x")
    # int4 weights handed over as 32-bit words (8 nibbles per word, nibble i at bits 4i)
    out2 = mn._C.dequant_matmul(d.x, d.wq.view(torch.int32), d.scales, d.zeros, d.group_size, "int4")
    assert torch.equal(out2, mn._C.dequant_matmul(*d.args()))


@pytest.mark.parametrize("scale", [3e5, 1.0, 1e-7])
@pytest.mark.parametrize("quant,g", [("int4", 128), ("int8", 1024)])
def test_bf16_activation_range(mn, scale, quant, g):
    """bf16 activations run on fp16 tensor-core instructions after an exact power-of-two
    rescale per CTA: magnitudes far outside the fp16 range must still come out right."""
    import mnq_workloads as workloads
    L = workloads.make_layer("t", 3, 1024, 160, quant_type=quant, group_size=g, act_dtype=torch.bfloat16,
                             scale_dtype=torch.bfloat16, asymmetric=(quant == "int4"), seed=17)
    L.x = (L.x.float() * scale).to(torch.bfloat16)
    ref = H.oracle_matmul(L, threads=1)
    out = mn._C.dequant_matmul(*L.to("cuda").args())
    assert mn._C.select_path(3, 160, 1024, g, quant, torch.bfloat16) == "gemv"
    H.assert_close_to_oracle(out, ref, f"bf16 x{scale:g}")


def test_paths_agree(mn):
    """The three kernel families compute the same function."""
    import mnq_workloads as workloads
    L = workloads.make_layer("t", 8, 1024, 256, seed=9).to("cuda")
    a = mn._C.dequant_matmul(*L.args(), tuning=_tuning(mn, path=mn._C.PATH_GEMV))
    b = mn._C.dequant_matmul(*L.args(), tuning=_tuning(mn, path=mn._C.PATH_GENERIC))
    assert float((a.float() - b.float()).abs().max()) <= 2e-2


# --------------------------------------------------------------------------- benchmark configurations

def test_config0_qwen05b_down(mn):
    import mnq_workloads as workloads
    (L,) = workloads.config0()
    ref = H.oracle_matmul(L)
    out = mn._C.dequant_matmul(*L.to("cuda").args())
    assert mn._C.select_path(L.M, L.N, L.K, L.group_size, "int4") == "gemv"
    H.assert_close_to_oracle(out, ref, "config0")


def test_config1_qwen7b_decode_full_size(mn):
    import mnq_workloads as workloads
    for L in workloads.config1():
        ref = H.oracle_matmul(L)
        d = L.to("cuda")
        out = mn._C.dequant_matmul(*d.args())
        assert mn._C.select_path(L.M, L.N, L.K, L.group_size, "int4") == "gemv"
        H.assert_close_to_oracle(out, ref, L.name)
        # linearity, a size-independent property: f(2x) == 2 f(x) up to output rounding
        out2 = mn._C.dequant_matmul(d.x * 2, d.wq, d.scales, d.zeros, d.group_size, "int4")
        assert torch.allclose(out2.float(), out.float() * 2, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("M", [4, 16, 32])
def test_config2_llama8b_batched_decode(mn, M):
    import mnq_workloads as workloads
    rng = np.random.default_rng(M)
    for L in workloads.config2(M):
        d = L.to("cuda")
        out = mn._C.dequant_matmul(*d.args())
        cols = np.sort(rng.choice(L.N, 1024, replace=False))
        ref = H.oracle_matmul(L, cols=cols)
        H.assert_close_to_oracle(out[:, torch.as_tensor(cols, device="cuda")], ref, f"{L.name} M={M}")
        # bf16 outputs cannot meet rel-L2 1e-3; the same kernel's fp32 output must
        out32 = mn._C.dequant_matmul_fused(*d.args(), out_dtype=torch.float32)
        H.assert_fp32_gate(out32[:, torch.as_tensor(cols, device="cuda")], ref, f"{L.name} M={M}")
        assert torch.equal(out32.to(torch.bfloat16), out)
        # whole output against fp32 math on the (bit-exactly verified) dequantised weights
        W = mn.dequantize(d.wq, d.scales, None, d.group_size, "int4", torch.float32)
        full = d.x.float() @ W.t()
        rel = float((out.float() - full).norm() / full.norm())
        assert rel < 4e-3, rel


@pytest.mark.parametrize("M", [1])
def test_config4_llama70b_decode_int8_full_size(mn, M):
    import mnq_workloads as workloads
    rng = np.random.default_rng(4)
    for L in workloads.config4(M):
        d = L.to("cuda")
        out = mn._C.dequant_matmul(*d.args())
        cols = np.sort(rng.choice(L.N, 512, replace=False))
        ref = H.oracle_matmul(L, cols=cols)
        H.assert_close_to_oracle(out[:, torch.as_tensor(cols, device="cuda")], ref, L.name)
        out32 = mn._C.dequant_matmul_fused(*d.args(), out_dtype=torch.float32)
        H.assert_fp32_gate(out32[:, torch.as_tensor(cols, device="cuda")], ref, L.name)
        assert torch.equal(out32.to(torch.bfloat16), out)
        W = mn.dequantize(d.wq, d.scales, None, d.group_size, "int8", torch.float32)
        full = d.x.float() @ W.t()
        rel = float((out.float() - full).norm() / full.norm())
        assert rel < 4e-3, rel
        del W, d, out
        torch.cuda.empty_cache()


# --------------------------------------------------------------------------- errors

def test_errors_are_raised_before_any_launch(mn):
    import mnq_workloads as workloads
    L = workloads.make_layer("t", 2, 128, 32, seed=1).to("cuda")
    E = mn.MetalNativeError
    with pytest.raises(E, match="InvalidArgument: dequant_matmul: activations must be 2D"):
        mn._C.dequant_matmul(L.x[0], L.wq, L.scales, L.zeros, 128, "int4")
    with pytest.raises(E, match="InvalidArgument: dequant_matmul: activations must be Float16"):
        mn._C.dequant_matmul(L.x.float(), L.wq, L.scales, L.zeros, 128, "int4")
    with pytest.raises(E, match="group_size must be"):
        mn._C.dequant_matmul(L.x, L.wq, L.scales, L.zeros, 48, "int4")
    with pytest.raises(E, match=r"INT4 weights must be \[N, K/2\]"):
        mn._C.dequant_matmul(L.x, L.wq[:, :32].contiguous(), L.scales, L.zeros, 128, "int4")
    with pytest.raises(E, match=r"INT8 weights must be \[N, K\]"):
        mn._C.dequant_matmul(L.x, L.wq.view(torch.int8), L.scales, L.zeros, 128, "int8")
    with pytest.raises(E, match="quant_type must be 'int4' or 'int8'"):
        mn._C.dequant_matmul(L.x, L.wq, L.scales, L.zeros, 128, "fp4")
    with pytest.raises(E, match="scales must be contiguous"):
        mn._C.dequant_matmul(L.x, L.wq, L.scales[:16], L.zeros, 128, "int4")
    with pytest.raises(E, match="must be a CUDA tensor"):      # weights never live on the host: no CPU path
        mn._C.dequant_matmul(L.x, L.wq.cpu(), L.scales, L.zeros, 128, "int4")
    assert E(6, "x").code_name == "TimeoutError"
    # the context is still healthy
    out = mn._C.dequant_matmul(*L.args())
    assert torch.isfinite(out.float()).all()


def test_empty_inputs(mn):
    x = torch.zeros((0, 128), dtype=torch.float16, device="cuda")
    wq = torch.zeros((32, 64), dtype=torch.uint8, device="cuda")
    s = torch.ones((32, 1), dtype=torch.float16, device="cuda")
    assert mn._C.dequant_matmul(x, wq, s, None, 128, "int4").shape == (0, 32)
    x1 = torch.ones((3, 128), dtype=torch.float16, device="cuda")
    assert mn._C.dequant_matmul(x1, wq[:0], s[:0], None, 128, "int4").shape == (3, 0)
    # K == 0: an empty sum
    out = mn._C.dequant_matmul(x1[:, :0], wq[:, :0], s[:, :0], None, 128, "int4")
    assert out.shape == (3, 32) and bool((out == 0).all())


@pytest.mark.parametrize("M,K,N,quant,g,adt", [(1, 1024, 512, "int4", 128, torch.float16),
                                                (4, 2048, 384, "int8", 2048, torch.bfloat16),
                                                (64, 256, 256, "int4", 128, torch.float16)])
def test_host_activations_and_output(mn, M, K, N, quant, g, adt):
    """Activations filled on the CPU, result read on the CPU after synchronize(), as the reference's
    callers do with its shared-memory tensors; the two copies are enqueued with the kernel
    (mnq_dequant_matmul_host).  Same bits as the device-tensor call."""
    import mnq_workloads as workloads
    L = workloads.make_layer("t", M, K, N, quant_type=quant, group_size=g, act_dtype=adt,
                             asymmetric=adt == torch.float16, seed=M + K)
    d = L.to("cuda")
    want = mn._C.dequant_matmul(*d.args()).cpu()
    # a K-split problem that shares the cached workspace: its arrival counters sit at the front of
    # the workspace and must survive the host calls' staging copies
    S = workloads.make_layer("s", 1, 4096, 256, seed=5).to("cuda")
    split_want = mn._C.dequant_matmul(*S.args()).clone()
    x_host = L.x.clone().pin_memory()
    out_host = torch.empty((M, N), dtype=adt).pin_memory()
    for _ in range(3):   # successive calls share the cached workspace and its staging area
        out_host.zero_()
        got = mn._C.dequant_matmul(x_host, d.wq, d.scales, d.zeros, g, quant, out=out_host)
        mn._C.synchronize()
        assert got is out_host and torch.equal(out_host, want)
    fresh = mn._C.dequant_matmul(L.x, d.wq, d.scales, d.zeros, g, quant)      # pageable input, output allocated
    mn._C.synchronize()
    assert not fresh.is_cuda and torch.equal(fresh, want)
    assert torch.equal(mn._C.dequant_matmul(*S.args()), split_want)
    assert mn._C.device_status() == 0


@pytest.mark.parametrize("M,K,Hd,quant,g,adt", [(1, 1024, 512, "int4", 128, torch.float16),
                                                (1, 3584, 1000, "int4", 128, torch.float16),    # H not a multiple of 8
                                                (4, 2048, 256, "int8", 2048, torch.bfloat16),
                                                (16, 512, 384, "int4", 128, torch.bfloat16)])
def test_fused_swiglu_epilogue(mn, M, K, Hd, quant, g, adt):
    """gate+up projection with silu(gate) * up applied in the decode kernel's epilogue
    (mnq_dequant_matmul_swiglu) against the oracle's fp32 projections followed by the reference's
    SwiGLU formula (shaders/fused_swiglu.metal:48-84).  Two roundings of 16-bit inputs would give
    the unfused pipeline about 2x the relative error of one projection; the fused kernel rounds
    once, and is held to 2e-3 relative L2 (fp16) or the bf16 rounding floor."""
    import mnq_workloads as workloads
    L = workloads.make_layer("t", M, K, 2 * Hd, quant_type=quant, group_size=g, act_dtype=adt,
                             asymmetric=adt == torch.float16, seed=Hd + K)
    ref = H.oracle_matmul(L).astype(np.float64)
    gate, up = ref[:, :Hd], ref[:, Hd:]
    want = gate / (1.0 + np.exp(-gate)) * up
    d = L.to("cuda")
    buf = torch.full((M + 2, Hd + 16), 5.0, dtype=adt, device="cuda")
    out = buf[1:M + 1, 8:8 + Hd]
    got = mn._C.dequant_matmul_swiglu(*d.args(), out=out)
    mn._C.synchronize()
    assert mn._C.device_status() == 0
    got = got.float().cpu().numpy().astype(np.float64)
    rel = np.linalg.norm(got - want) / max(np.linalg.norm(want), 1e-30)
    assert rel <= (2e-3 if adt == torch.float16 else 4e-3), rel
    chk = buf.clone()
    chk[1:M + 1, 8:8 + Hd] = 5.0
    assert bool((chk == 5.0).all()), "kernel wrote outside its [M, H] output block"
    # the unfused pipeline through the same library agrees to rounding
    y = mn._C.dequant_matmul(*d.args()).float()
    unfused = (torch.nn.functional.silu(y[:, :Hd]) * y[:, Hd:]).cpu().numpy()
    assert np.linalg.norm(got - unfused) / np.linalg.norm(unfused) <= 6e-3
