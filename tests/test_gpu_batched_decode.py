"""The batched-decode kernel (5 to 32 tokens, activations prepared once per call; gemv_mid.cu)
against the CPU oracle and against the general streaming kernel, through the C ABI.  Needs a B200.
(Kernel variant 9 asks for it on the small layers most of these cases are, which the default
route gives to the other decode kernels.)"""
import pytest
import torch

from oracle import check as H

pytestmark = pytest.mark.gpu


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


CASES = [
    # quant, M, N, K, group, asymmetric, activation dtype
    ("int4", 5, 4096, 3584, 128, True, torch.float16),       # one token tile
    ("int4", 8, 37888, 512, 128, False, torch.bfloat16),
    ("int8", 7, 1040, 8192, 8192, True, torch.bfloat16),
    ("int4", 9, 4096, 3584, 128, True, torch.float16),       # two token tiles, one sweep
    ("int4", 16, 1000, 4096, 128, False, torch.bfloat16),    # ragged last row block, bf16 activations and scales
    ("int4", 16, 48, 512, 128, True, torch.float16),         # three row blocks, one K piece
    ("int4", 12, 528, 18944, 128, True, torch.float16),      # few rows: K cut, planes added by the second kernel
    ("int4", 17, 4096, 3584, 128, True, torch.float16),      # four token tiles, two row blocks per sweep
    ("int4", 32, 2064, 4096, 128, True, torch.bfloat16),     # odd number of row blocks per warp
    ("int4", 24, 37888, 1024, 128, True, torch.float16),     # many row blocks: several sweeps per warp
    ("int4", 32, 272, 14336, 128, False, torch.bfloat16),    # K cut with four token tiles
    ("int8", 16, 2048, 8192, 8192, False, torch.bfloat16),   # one group per row
    ("int8", 32, 1040, 4096, 4096, True, torch.float16),     # one group per row with zeros
    ("int8", 20, 272, 28672, 28672, False, torch.bfloat16),  # one group per row, K cut
    ("int8", 12, 1024, 1024, 64, True, torch.float16),       # int8 with a group per step
    ("int8", 32, 4096, 2048, 64, False, torch.bfloat16),
    # 33 to 64 tokens, bf16 activations with group-wise scales or zeros: six or eight token tiles
    ("int4", 33, 4096, 2048, 128, True, torch.bfloat16),
    ("int4", 48, 1000, 4096, 128, False, torch.bfloat16),
    ("int4", 64, 14336, 1024, 128, True, torch.bfloat16),
    ("int4", 57, 272, 14336, 128, True, torch.bfloat16),     # K cut
    ("int8", 40, 528, 2048, 64, True, torch.bfloat16),
    ("int8", 300 // 5, 1040, 4096, 64, False, torch.bfloat16),
]


@pytest.mark.parametrize("quant,M,N,K,g,asym,adt", CASES)
def test_batched_decode_kernel(mn, quant, M, N, K, g, asym, adt):
    """The batched-decode kernel, the general streaming kernel (variant 3) and the default route, all
    against the oracle, twice in a row on one workspace; fp32 output against the tighter gate."""
    import mnq_workloads as workloads
    C = mn._C
    try:
        if M <= 32:
            C.set_option("gemv_max_m", 32)   # keep every case on the decode family (above 32 tokens the automatic choice does)
        L = workloads.make_layer("t", M, K, N, quant_type=quant, group_size=g, act_dtype=adt,
                                 scale_dtype=adt if quant == "int4" else torch.float16, asymmetric=asym, seed=N + K + M)
        ref = H.oracle_matmul(L)
        d = L.to("cuda")
        assert C.select_path(M, N, K, g, quant, adt) == "gemv"
        general = _tuning(mn, gemv_variant=3)
        batched = _tuning(mn, gemv_variant=9)
        for call in range(2):
            a = C.dequant_matmul(*d.args(), tuning=batched)
            b = C.dequant_matmul(*d.args(), tuning=general if M <= 32 else None)   # (no other decode kernel above 32 tokens)
            C.synchronize()
            assert C.device_status() == 0
            H.assert_close_to_oracle(a, ref, f"batched {quant} {M}x{N}x{K} call {call}")
            H.assert_close_to_oracle(b, ref, f"general {quant} {M}x{N}x{K} call {call}")
        a2 = C.dequant_matmul(*d.args(), tuning=batched)
        assert torch.equal(a, a2), "result is not deterministic"
        H.assert_close_to_oracle(C.dequant_matmul(*d.args()), ref, f"default route {quant} {M}x{N}x{K}")
        a32 = C.dequant_matmul_fused(*d.args(), out_dtype=torch.float32)
        H.assert_fp32_gate(a32, ref, f"batched fp32 {quant} {M}x{N}x{K}")
    finally:
        C.set_option("gemv_max_m", 0)


@pytest.mark.parametrize("split", [1, 2, 5])
def test_batched_decode_forced_k_cuts_and_epilogue(mn, split):
    import mnq_workloads as workloads
    C = mn._C
    M, N, K = 24, 1008, 4096
    L = workloads.make_layer("t", M, K, N, act_dtype=torch.bfloat16, scale_dtype=torch.bfloat16, seed=split)
    ref = H.oracle_matmul(L)
    d = L.to("cuda")
    g = torch.Generator(device="cpu").manual_seed(7)
    bias = (torch.randn(N, generator=g) * 0.5).to(torch.bfloat16)
    want = torch.relu(torch.from_numpy(ref) + bias.float())
    try:
        C.set_option("gemv_max_m", 32)
        t = _tuning(mn, path=C.PATH_GEMV, split_k=split, gemv_variant=9)
        out = C.dequant_matmul_fused(*d.args(), epilogue="bias_relu", bias=bias.cuda())
        plain = C.dequant_matmul(*d.args(), tuning=t)
        C.synchronize()
    finally:
        C.set_option("gemv_max_m", 0)
    assert C.device_status() == 0
    H.assert_close_to_oracle(plain, ref, f"split {split}")
    H.assert_close_to_oracle(out, want.numpy(), f"split {split} with bias + relu")


def test_batched_decode_strided_activations_and_bf16_range(mn):
    """Token rows 2 K apart (a view of a wider buffer); bf16 activations whose magnitudes differ by
    2^40 between tokens: every token is rescaled by its own power of two."""
    import mnq_workloads as workloads
    C = mn._C
    M, N, K = 16, 512, 2048
    L = workloads.make_layer("t", M, K, N, act_dtype=torch.bfloat16, scale_dtype=torch.bfloat16, seed=3)
    factors = torch.tensor([2.0 ** (-20 + 40 * (m % 2)) for m in range(M)], dtype=torch.float32)[:, None]
    L.x = (L.x.float() * factors).to(torch.bfloat16)
    ref = H.oracle_matmul(L)
    d = L.to("cuda")
    wide = torch.zeros((M, 2 * K), dtype=torch.bfloat16, device="cuda")
    wide[:, :K] = d.x
    try:
        C.set_option("gemv_max_m", 32)
        out = C.dequant_matmul(wide[:, :K], d.wq, d.scales, d.zeros, L.group_size, L.quant_type)
        C.synchronize()
    finally:
        C.set_option("gemv_max_m", 0)
    assert C.device_status() == 0
    for m in range(M):   # per token: the tokens' magnitudes differ too much for one norm
        H.assert_close_to_oracle(out[m:m + 1], ref[m:m + 1], f"token {m}")


@pytest.mark.parametrize("M,N,K", [(16, 4096, 2048), (24, 528, 14336)])
def test_batched_decode_step_replayed_from_a_cuda_graph(mn, M, N, K):
    """A batched-decode call is two or three launches (activation image, kernel, K-cut reduction);
    recorded into a CUDA graph through PhasePipeline and replayed with new activations in the same
    buffer, it must give the eager result every time."""
    import mnq_workloads as workloads
    C = mn._C
    L = workloads.make_layer("t", M, K, N, act_dtype=torch.bfloat16, scale_dtype=torch.bfloat16, seed=M + N)
    d = L.to("cuda")
    out = torch.zeros((M, N), dtype=torch.bfloat16, device="cuda")
    pipe = mn.PhasePipeline()
    pipe.set_phase(mn.InferencePhase.Decode)
    batched = _tuning(mn, gemv_variant=9)
    step = pipe.capture_step(lambda: C.dequant_matmul(*d.args(), out=out, tuning=batched))
    for scale in (1.0, 0.5, -3.0):
        d.x.copy_((L.x.float() * scale).to(torch.bfloat16))
        want = C.dequant_matmul(*d.args(), tuning=batched).clone()
        out.zero_()
        step()
        torch.cuda.synchronize()
        assert C.device_status() == 0
        assert torch.equal(out, want), f"graph replay differs from the eager call at scale {scale}"
    ref = H.oracle_matmul(L)
    d.x.copy_(L.x)
    step()
    torch.cuda.synchronize()
    H.assert_close_to_oracle(out, ref, f"replayed {M}x{N}x{K}")
