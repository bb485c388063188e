"""Parity of the tensor-core (tcgen05 / TMEM) prefill kernel with the CPU oracle, through
the Python shim over the C ABI.  Needs a B200; run with -m gpu."""
import numpy as np
import pytest
import torch

from oracle import check as H

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mn():
    import metal_native
    assert torch.cuda.is_available()
    return metal_native


def _gemm_tuning(mn):
    t = mn._C.Tuning()
    t.path = mn._C.PATH_GEMM
    return t


CASES = [
    # quant, M, N, K, g, asym, act dtype, scale dtype
    ("int4", 64, 128, 64, 64, True, torch.float16, torch.float16),        # one k-block, one tile
    ("int4", 64, 128, 256, 128, True, torch.float16, torch.float16),      # reference LargeMatrix class
    ("int4", 128, 256, 512, 128, True, torch.float16, torch.float16),
    ("int4", 100, 200, 256, 64, True, torch.float16, torch.float16),      # ragged M (tok 112) and N
    ("int4", 33, 130, 128, 128, False, torch.float16, torch.float16),     # smallest M on this path
    ("int4", 300, 128, 1024, 128, True, torch.float16, torch.float16),    # two token tiles of 160
    ("int4", 512, 384, 640, 128, True, torch.float16, torch.float16),     # more k-blocks than stages
    ("int4", 64, 128, 192, 1 << 20, True, torch.float16, torch.float16),  # one group per row
    ("int8", 64, 128, 256, 128, True, torch.float16, torch.float16),
    ("int8", 96, 160, 512, 64, False, torch.float16, torch.float16),
    ("int8", 64, 256, 512, 512, False, torch.bfloat16, torch.float16),    # config 4 style: scale in epilogue
    ("int4", 80, 128, 256, 256, False, torch.bfloat16, torch.bfloat16),
    # bf16 activations with group-wise scales (and zeros): every weight as two bf16 values, two MMAs
    ("int4", 64, 256, 512, 128, False, torch.bfloat16, torch.bfloat16),   # config 2 style
    ("int4", 200, 384, 1024, 128, True, torch.bfloat16, torch.bfloat16),
    ("int8", 96, 128, 256, 64, True, torch.bfloat16, torch.float16),
    ("int4", 512, 512, 640, 128, True, torch.bfloat16, torch.bfloat16),   # CTA pairs
    ("int8", 64, 128, 256, 256, True, torch.bfloat16, torch.bfloat16),    # one group per row, but zeros
]


@pytest.mark.parametrize("quant,M,N,K,g,asym,adt,sdt", CASES)
def test_gemm_shapes(mn, quant, M, N, K, g, asym, adt, sdt):
    import mnq_workloads as workloads
    L = workloads.make_layer("t", M, K, N, quant_type=quant, group_size=g, act_dtype=adt, scale_dtype=sdt,
                             asymmetric=asym, seed=M + N + K)
    # (33 to 64 tokens of bf16 activations with group-wise scales go to the batched-decode kernel by default;
    # this test forces the tensor-core kernel either way)
    decode_range = adt == torch.bfloat16 and 32 < M <= 64 and g < K
    assert mn._C.select_path(M, N, K, g, quant, adt) in (("gemv",) if decode_range else ("gemm", "generic"))
    ref = H.oracle_matmul(L)
    d = L.to("cuda")
    buf = torch.full((M + 2, N + 8), 777.0, dtype=adt, device="cuda")
    out = buf[1:M + 1, 3:N + 3]
    mn._C.dequant_matmul(*d.args(), out=out, tuning=_gemm_tuning(mn))
    mn._C.synchronize()
    assert mn._C.device_status() == 0
    H.assert_close_to_oracle(out, ref, f"gemm {quant} {M}x{N}x{K} g{g}")
    chk = buf.clone()
    chk[1:M + 1, 3:N + 3] = 777.0
    assert bool((chk == 777.0).all()), "kernel wrote outside its [M, N] output block"


PAIR_CASES = [
    # quant, M, N, K, g, act dtype, split
    ("int4", 64, 256, 256, 128, torch.float16, 1),      # forced pairs on a 64-token tile (32 tokens per CTA)
    ("int4", 48, 384, 512, 64, torch.float16, 1),       # three 128-row tiles: the last pair has an idle CTA
    ("int4", 200, 200, 1024, 128, torch.float16, 1),    # ragged N inside the second CTA of the pair
    ("int4", 512, 512, 1280, 128, torch.float16, 1),    # two accumulators, more k-blocks than stages
    ("int4", 300, 256, 1024, 128, torch.float16, 3),    # two token tiles, K split
    ("int8", 160, 512, 768, 768, torch.bfloat16, 1),    # integer tile, scale in the epilogue
    ("int8", 128, 256, 512, 128, torch.float16, 2),
]


RAW_CASES = [
    # int8 with one scale per row, at most 256 tokens: raw-integer tiles (activations prepared once per call)
    # M, N, K, asym, act dtype, scale dtype, K splits (0 = the plan's)
    (64, 256, 512, False, torch.bfloat16, torch.float16, 0),     # config 4 style
    (64, 200, 1024, True, torch.bfloat16, torch.float16, 0),     # with zeros: offset term through the token sums
    (33, 128, 64, True, torch.float16, torch.float16, 0),        # fp16 activations are used as they are
    (256, 384, 2048, True, torch.bfloat16, torch.bfloat16, 3),   # K split: the offset goes into the first plane only
    (100, 130, 4096, False, torch.float16, torch.bfloat16, 2),   # fp16 activations with bf16 scales
    (16, 256, 1024, True, torch.bfloat16, torch.float16, 0),     # few tokens (forced onto the tensor-core path)
]


@pytest.mark.parametrize("M,N,K,asym,adt,sdt,split", RAW_CASES)
def test_gemm_raw_integer_tiles(mn, M, N, K, asym, adt, sdt, split):
    """Raw-integer tiles against the oracle, against the dequantising tile path (kernel variant 5) where that
    path takes the problem, in the fp32 output mode, and with wide-ranged bf16 activations (the per-token
    rescale)."""
    import mnq_workloads as workloads
    C = mn._C
    L = workloads.make_layer("t", M, K, N, quant_type="int8", group_size=K, act_dtype=adt, scale_dtype=sdt,
                             asymmetric=asym, seed=M + N + K)
    if adt == torch.bfloat16:   # rows of very different magnitude: every token gets its own power of two
        L.x.mul_(torch.logspace(-6, 4, M).to(torch.bfloat16)[:, None])
    ref = H.oracle_matmul(L)
    d = L.to("cuda")
    t = _gemm_tuning(mn)
    t.split_k = split
    out = C.dequant_matmul(*d.args(), tuning=t)
    C.synchronize()
    assert C.device_status() == 0
    # rows differ by ten orders of magnitude: compare row by row
    for m in range(0, M, max(1, M // 8)):
        H.assert_close_to_oracle(out[m:m + 1], ref[m:m + 1], f"raw int8 {M}x{N}x{K} row {m}")
    if M > 32:
        out32 = C.dequant_matmul_fused(*d.args(), out_dtype=torch.float32)
        assert torch.equal(out32.to(adt), C.dequant_matmul(*d.args()))
        for m in range(0, M, max(1, M // 4)):
            scale = float(np.abs(ref[m]).max()) or 1.0
            H.assert_fp32_gate(out32[m:m + 1] / scale * 8.0, ref[m:m + 1] / scale * 8.0, f"raw int8 fp32 row {m}")
    if not (adt == torch.float16 and sdt == torch.bfloat16):
        t5 = _gemm_tuning(mn)
        t5.gemv_variant = 5                      # the dequantising tile path
        t5.split_k = split
        other = C.dequant_matmul(*d.args(), tuning=t5)
        for m in range(0, M, max(1, M // 8)):
            H.assert_close_to_oracle(other[m:m + 1], ref[m:m + 1], f"dequantised tiles row {m}")


@pytest.mark.parametrize("variant", [1, 2])
@pytest.mark.parametrize("quant,M,N,K,g,adt,split", PAIR_CASES)
def test_gemm_single_cta_and_cta_pairs(mn, quant, M, N, K, g, adt, split, variant):
    """The same problems through single-CTA tiles (variant 1) and through clusters of two CTAs
    sharing each activation tile (variant 2): both match the oracle, and they agree with
    each other bit for bit (same products, same accumulation order)."""
    import mnq_workloads as workloads
    L = workloads.make_layer("t", M, K, N, quant_type=quant, group_size=g, act_dtype=adt,
                             asymmetric=adt == torch.float16, seed=N + K + M)
    ref = H.oracle_matmul(L)
    d = L.to("cuda")
    t = _gemm_tuning(mn)
    t.split_k = split
    t.gemv_variant = variant
    out = mn._C.dequant_matmul(*d.args(), tuning=t)
    t.gemv_variant = 3 - variant
    other = mn._C.dequant_matmul(*d.args(), tuning=t)
    mn._C.synchronize()
    assert mn._C.device_status() == 0
    H.assert_close_to_oracle(out, ref, f"gemm variant {variant} {quant} {M}x{N}x{K}")
    assert torch.equal(out, other)


@pytest.mark.parametrize("quant,M,N,K,g,adt,split", [
    ("int4", 64, 1024, 512, 128, torch.float16, 1),
    ("int4", 200, 640, 1024, 128, torch.float16, 2),     # ragged tokens and rows, K split
    ("int8", 96, 2048, 256, 256, torch.bfloat16, 1),     # integer tile, scale in the epilogue
    ("int4", 256, 384, 2048, 128, torch.float16, 1),     # the largest tile that still allows two CTAs per SM
])
def test_gemm_one_and_two_ctas_per_sm(mn, quant, M, N, K, g, adt, split):
    """Tiles of at most 256 tokens may run two CTAs per SM (variant 4 forces it, variant 3 forbids
    it): same kernel body planned for half the shared memory, so the results are identical."""
    import mnq_workloads as workloads
    L = workloads.make_layer("t", M, K, N, quant_type=quant, group_size=g, act_dtype=adt,
                             asymmetric=adt == torch.float16, seed=N + M)
    ref = H.oracle_matmul(L)
    d = L.to("cuda")
    t = _gemm_tuning(mn)
    t.split_k = split
    t.gemv_variant = 4
    two = mn._C.dequant_matmul(*d.args(), tuning=t)
    t.gemv_variant = 3
    one = mn._C.dequant_matmul(*d.args(), tuning=t)
    mn._C.synchronize()
    assert mn._C.device_status() == 0
    H.assert_close_to_oracle(two, ref, f"gemm two CTAs per SM {quant} {M}x{N}x{K}")
    assert torch.equal(one, two)


@pytest.mark.parametrize("split", [1, 2, 3, 5])
def test_gemm_split_k_is_deterministic_and_reuses_workspace(mn, split):
    import mnq_workloads as workloads
    L = workloads.make_layer("t", 200, 1024, 256, seed=split)
    ref = H.oracle_matmul(L)
    d = L.to("cuda")
    t = _gemm_tuning(mn)
    t.split_k = split
    outs = [mn._C.dequant_matmul(*d.args(), tuning=t) for _ in range(3)]
    mn._C.synchronize()
    assert mn._C.device_status() == 0
    H.assert_close_to_oracle(outs[0], ref, f"gemm split {split}")
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])


def test_gemm_is_selected_for_prefill_shapes(mn):
    sp = mn._C.select_path
    assert sp(512, 18944, 3584, 128, "int4") == "gemm"
    assert sp(512, 3584, 18944, 128, "int4") == "gemm"
    assert sp(64, 57344, 8192, 8192, "int8", torch.bfloat16, zeros=False) == "gemm"
    assert sp(64, 8192, 28672, 28672, "int8", torch.bfloat16, zeros=False) == "gemm"
    assert sp(128, 14336, 4096, 128, "int4", torch.bfloat16, zeros=False) == "gemm"   # bf16, group-wise
    assert sp(40, 70, 96, 32, "int4") == "generic"        # K % 64 != 0


def test_gemm_agrees_with_other_paths(mn):
    import mnq_workloads as workloads
    L = workloads.make_layer("t", 64, 1024, 256, seed=5).to("cuda")
    a = mn._C.dequant_matmul(*L.args(), tuning=_gemm_tuning(mn))
    t = mn._C.Tuning(); t.path = mn._C.PATH_GENERIC
    b = mn._C.dequant_matmul(*L.args(), tuning=t)
    assert float((a.float() - b.float()).abs().max()) <= 2e-2


def test_config3_prefill_full_size(mn):
    import mnq_workloads as workloads
    rng = np.random.default_rng(3)
    for L in workloads.config3():
        d = L.to("cuda")
        out = mn._C.dequant_matmul(*d.args())
        mn._C.synchronize()
        assert mn._C.device_status() == 0
        cols = np.sort(rng.choice(L.N, 96, replace=False))
        ref = H.oracle_matmul(L, cols=cols)
        H.assert_close_to_oracle(out[:, torch.as_tensor(cols, device="cuda")], ref, L.name)
        # whole output against fp32 math on the (bit-exactly verified) dequantised weights
        W = mn.dequantize(d.wq, d.scales, d.zeros, d.group_size, "int4", torch.float32)
        full = d.x.float() @ W.t()
        rel = float((out.float() - full).norm() / full.norm())
        assert rel < 1e-3, rel
        del W, full


def test_config4_m64_int8_bf16_full_size(mn):
    """Llama-3-70B layers at 64 tokens, full size (N = 57344 and 8192): the grid, the two CTAs per
    SM, the integer tile with the scale in the epilogue and the K split of the long layer are the
    ones the benchmark runs.  Oracle on sampled columns; north-star gate on the fp32 output."""
    import mnq_workloads as workloads
    rng = np.random.default_rng(5)
    for L in workloads.config4(64):
        d = L.to("cuda")
        out = mn._C.dequant_matmul(*d.args())
        out32 = mn._C.dequant_matmul_fused(*d.args(), out_dtype=torch.float32)
        mn._C.synchronize()
        assert mn._C.device_status() == 0
        cols = np.sort(rng.choice(L.N, 64, replace=False))
        ref = H.oracle_matmul(L, cols=cols)
        idx = torch.as_tensor(cols, device="cuda")
        H.assert_close_to_oracle(out[:, idx], ref, L.name)
        H.assert_fp32_gate(out32[:, idx], ref, L.name)
        assert torch.equal(out32.to(torch.bfloat16), out), "the 16-bit output is the rounded fp32 output"
        del d, out, out32
        torch.cuda.empty_cache()


@pytest.mark.parametrize("quant,M,N,K,g,adt", [
    ("int4", 64, 384, 1024, 128, torch.float16),      # group-wise fp16: dequantised tiles
    ("int4", 128, 200, 4096, 128, torch.float16),     # 128 tokens: four tensor-memory slots
    ("int4", 40, 256, 2048, 2048, torch.bfloat16),    # bf16, one scale per row, no zeros: integer tiles
    ("int8", 96, 272, 2048, 2048, torch.bfloat16),    # raw-integer tiles
    ("int8", 33, 128, 512, 64, torch.float16),        # int8 group-wise
    ("int4", 100, 400, 4096, 128, torch.bfloat16),    # bf16 group-wise: two tiles per k-block, 64-column slots
    ("int8", 128, 256, 1024, 64, torch.bfloat16),
])
def test_weight_tiles_in_tensor_memory_match_shared_memory_tiles(mn, quant, M, N, K, g, adt):
    """Tiles of at most 128 tokens keep the dequantised weight tile in tensor memory (the default);
    kernel variant 6 sends it through shared memory.  Same arithmetic: the outputs are bit-identical,
    and both meet the oracle gate; split K too."""
    import mnq_workloads as workloads
    C = mn._C
    per_channel = g >= K
    L = workloads.make_layer("t", M, K, N, quant_type=quant, group_size=g, act_dtype=adt,
                             scale_dtype=torch.float16 if (quant == "int8" or adt == torch.float16) else adt,
                             asymmetric=not (per_channel and quant == "int4"), seed=M + N + K)
    ref = H.oracle_matmul(L)
    d = L.to("cuda")
    for split in (0, 2):
        t = _gemm_tuning(mn)
        t.split_k = split
        a = C.dequant_matmul(*d.args(), tuning=t)
        t6 = _gemm_tuning(mn)
        t6.split_k = split
        t6.gemv_variant = 6
        b = C.dequant_matmul(*d.args(), tuning=t6)
        C.synchronize()
        assert C.device_status() == 0
        H.assert_close_to_oracle(a, ref, f"tensor-memory tiles {quant} {M}x{N}x{K} split {split}")
        H.assert_close_to_oracle(b, ref, f"shared-memory tiles {quant} {M}x{N}x{K} split {split}")
        assert torch.equal(a, b), "the two tile paths differ"


@pytest.mark.parametrize("quant,M,N,K,g,asym,sdt", [
    ("int4", 64, 384, 1024, 128, True, torch.bfloat16),
    ("int4", 200, 272, 4096, 128, False, torch.bfloat16),     # two accumulators, no zeros
    ("int4", 512, 512, 640, 128, True, torch.bfloat16),       # CTA pairs
    ("int8", 96, 128, 512, 64, True, torch.float16),          # int8 group-wise, fp16 scales
    ("int8", 300, 256, 2048, 2048, True, torch.bfloat16),     # one scale per row with zeros, more tokens than raw-integer tiles take
])
def test_bf16_activations_through_fp16_tiles_when_opted_in(mn, quant, M, N, K, g, asym, sdt):
    """MNQ_OPT_BF16_FP16_TILES: one fp16 weight tile per k-block for bf16 activations.  The result meets
    the north-star gate in the fp32 output mode (rel-L2 <= 1e-3, max-abs <= 2e-2) and the bf16 rounding
    floor in rel-L2; element-wise it carries the fp16 tile's rounding noise, about 2.8e-4 of the output
    RMS per element (the default two-tile path is held to one bf16 ulp + 1e-4 RMS).  Scales and zeros far outside fp16's range (2^30 and
    2^-30 times the usual) are normalised per row, so they change nothing."""
    import numpy as np
    import mnq_workloads as workloads
    C = mn._C
    for factor in (1.0, 2.0 ** 30, 2.0 ** -30) if sdt == torch.bfloat16 else (1.0,):
        L = workloads.make_layer("t", M, K, N, quant_type=quant, group_size=g, act_dtype=torch.bfloat16,
                                 scale_dtype=sdt, asymmetric=asym, seed=M + N + K)
        if factor != 1.0:
            L.scales = (L.scales.float() * factor).to(sdt)
            if L.zeros is not None:
                L.zeros = (L.zeros.float() * factor).to(sdt)
        ref = H.oracle_matmul(L)
        d = L.to("cuda")
        exact = C.dequant_matmul(*d.args(), tuning=_gemm_tuning(mn))
        try:
            C.set_option("bf16_fp16_tiles", 1)
            fast = C.dequant_matmul(*d.args(), tuning=_gemm_tuning(mn))
            fast32 = C.dequant_matmul_fused(*d.args(), out_dtype=torch.float32) if M > 32 else None
            again = C.dequant_matmul(*d.args(), tuning=_gemm_tuning(mn))
            forced = _gemm_tuning(mn)
            forced.gemv_variant = 8
            two_tiles = C.dequant_matmul(*d.args(), tuning=forced)
        finally:
            C.set_option("bf16_fp16_tiles", 0)
        C.synchronize()
        assert C.device_status() == 0
        H.assert_close_to_oracle(exact, ref, f"two tiles {quant} {M}x{N}x{K} x{factor:g}")
        assert torch.equal(two_tiles, exact), "variant 8 must keep the two-tile path"
        assert torch.equal(fast, again), "not deterministic"
        if fast32 is not None and factor == 1.0:   # (the gate's max-abs is absolute: unscaled outputs only)
            H.assert_fp32_gate(fast32, ref, f"fp16 tiles, fp32 output {quant} {M}x{N}x{K}")
        got = fast.float().cpu().numpy()
        rel, _ = H.errors(got, ref)
        rel0, _ = H.errors(torch.from_numpy(ref).to(torch.bfloat16).float().numpy(), ref)
        assert rel <= rel0 * 1.05 + 1e-6, f"rel-L2 {rel:.3e} vs bf16 rounding floor {rel0:.3e}"
        rms = float(np.sqrt((ref.astype(np.float64) ** 2).mean()))
        bound = np.abs(ref) * 2.0 ** -7 + 1.5e-3 * rms   # one bf16 ulp + five sigma of the tile noise
        assert np.all(np.abs(got - ref) <= bound), f"element error {float(np.max(np.abs(got - ref) / bound)):.2f}x the bound"


@pytest.mark.parametrize("quant,M,N,K,g,adt,epilogue", [
    ("int8", 64, 300 * 128, 2048, 2048, torch.bfloat16, None),             # raw-integer tiles: 4 tiles past two full rounds
    ("int8", 48, 301 * 128 - 88, 2048, 2048, torch.float16, "bias_relu"),  # ragged last tile, epilogue in the second launch
    ("int4", 64, 300 * 128, 2048, 128, torch.float16, "residual"),         # dequantised tiles with a scale table per part
    ("int4", 72, 150 * 128 + 64, 4096, 128, torch.bfloat16, None),         # two bf16 tiles per k-block: one CTA per SM
])
def test_last_round_of_tiles_cut_along_k(mn, quant, M, N, K, g, adt, epilogue):
    """More tiles along N than CTAs that run at once: the tiles of the last, partly empty round are cut
    along K (their partial sums added by a second launch).  Against the oracle, against the uncut kernel
    (variant 7), with an epilogue and with the fp32 output; deterministic."""
    import mnq_workloads as workloads
    C = mn._C
    per_channel = g >= K
    L = workloads.make_layer("t", M, K, N, quant_type=quant, group_size=g, act_dtype=adt,
                             scale_dtype=torch.float16 if (quant == "int8" or adt == torch.float16) else adt,
                             asymmetric=not (per_channel and quant == "int4"), seed=M + K)
    ref = H.oracle_matmul(L)
    d = L.to("cuda")
    t = _gemm_tuning(mn)
    t7 = _gemm_tuning(mn)
    t7.gemv_variant = 7
    a = C.dequant_matmul(*d.args(), tuning=t)
    a2 = C.dequant_matmul(*d.args(), tuning=t)
    b = C.dequant_matmul(*d.args(), tuning=t7)
    a32 = C.dequant_matmul_fused(*d.args(), out_dtype=torch.float32)   # (these shapes take the tensor-core kernel by themselves)
    C.synchronize()
    assert C.device_status() == 0
    H.assert_close_to_oracle(a, ref, f"cut tail {quant} {M}x{N}x{K}")
    H.assert_close_to_oracle(b, ref, f"uncut {quant} {M}x{N}x{K}")
    H.assert_fp32_gate(a32, ref, f"cut tail fp32 {quant} {M}x{N}x{K}")
    assert torch.equal(a, a2), "result is not deterministic"
    # the columns before the tail are computed exactly as without the cut
    assert torch.equal(a[:, :128 * 148], b[:, :128 * 148])
    if epilogue:
        gen = torch.Generator(device="cpu").manual_seed(11)
        ref_t = torch.from_numpy(ref)
        if epilogue == "residual":
            res = (torch.randn(M, N, generator=gen) * 0.5).to(adt)
            want = ref_t + res.float()
            out = C.dequant_matmul_fused(*d.args(), epilogue="residual", residual=res.cuda())
        else:
            bias = (torch.randn(N, generator=gen) * 0.5).to(adt)
            want = torch.relu(ref_t + bias.float())
            out = C.dequant_matmul_fused(*d.args(), epilogue="bias_relu", bias=bias.cuda())
        C.synchronize()
        assert C.device_status() == 0
        H.assert_close_to_oracle(out, want.numpy(), f"cut tail with {epilogue}")
