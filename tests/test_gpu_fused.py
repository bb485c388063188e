"""GPU tests of what surrounds the plain operator call: the fused epilogues (bias, bias+ReLU,
bias+SiLU, residual: the reference's MatmulEpilogue, include/metal_native/ops/fused_matmul.h:18-24,
arithmetic of shaders/matmul_fused_epilogue.metal:97-124), the fp32 output mode, the decode /
tensor-core threshold, a bounded wait that runs out, and the phase pipeline's graph capture."""
import ctypes

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


def _epilogue_ref(acc: np.ndarray, kind: str, bias, residual) -> np.ndarray:
    """fp32 restatement of apply_epilogue (matmul_fused_epilogue.metal:97-124) over the oracle's
    fp32 matmul result."""
    v = acc.astype(np.float32)
    if kind == "residual":
        return v + residual.astype(np.float32)
    if kind != "none":
        v = v + bias.astype(np.float32)[None, :]
    if kind == "bias_relu":
        v = np.maximum(np.float32(0), v)
    if kind == "bias_silu":
        v = (v / (np.float32(1) + np.exp(-v, dtype=np.float32))).astype(np.float32)
    return v


# one shape per kernel family and result path: streaming decode kernel (direct store; K split with the
# last-arriver reduction; many tokens with the reduce kernel), register-prefetch decode kernel, any-shape
# kernel, tensor-core kernel (direct epilogue; K split + reduce kernel; CTA pairs)
SHAPES = [
    ("stream", 1, 2048, 1024, "int4", 128, torch.float16),
    ("stream-splitk", 2, 8192, 256, "int4", 128, torch.float16),
    ("stream-many", 16, 4096, 512, "int4", 128, torch.bfloat16),
    ("prefetch", 3, 1000, 96, "int8", 1000, torch.bfloat16),
    ("generic", 2, 100, 37, "int4", 32, torch.float16),
    ("gemm", 96, 1024, 384, "int4", 128, torch.float16),
    ("gemm-splitk", 64, 8192, 256, "int8", 8192, torch.bfloat16),
    ("gemm-pair", 300, 512, 512, "int4", 128, torch.float16),
]


@pytest.mark.parametrize("kind", ["none", "bias", "bias_relu", "bias_silu", "residual"])
@pytest.mark.parametrize("name,M,K,N,quant,g,adt", SHAPES, ids=[s[0] for s in SHAPES])
def test_fused_epilogues_match_oracle_plus_reference_epilogue(mn, name, M, K, N, quant, g, adt, kind):
    import mnq_workloads as workloads
    L = workloads.make_layer(name, M, K, N, quant_type=quant, group_size=g, act_dtype=adt,
                             scale_dtype=adt if quant == "int4" else torch.float16,
                             asymmetric=(adt == torch.float16 and quant == "int4"), seed=M + N)
    gen = torch.Generator().manual_seed(N)
    bias = (torch.randn(N, generator=gen) * 2).to(adt)
    residual = (torch.randn(M, N, generator=gen) * 3).to(adt)
    want = _epilogue_ref(H.oracle_matmul(L), kind, bias.float().numpy(), residual.float().numpy())
    d = L.to("cuda")
    kw = {}
    if kind == "residual":
        kw["residual"] = residual.cuda()
    elif kind != "none":
        kw["bias"] = bias.cuda()
    out = mn._C.dequant_matmul_fused(*d.args(), kind, **kw)
    out32 = mn._C.dequant_matmul_fused(*d.args(), kind, out_dtype=torch.float32, **kw)
    mn._C.synchronize()
    assert mn._C.device_status() == 0
    H.assert_close_to_oracle(out, want, f"{name} {kind}")
    H.assert_fp32_gate(out32, want, f"{name} {kind}")
    assert torch.equal(out32.to(adt), out), "16-bit output = rounded fp32 output"
    if kind == "none":
        assert torch.equal(out, mn._C.dequant_matmul(*d.args())), "no epilogue = the plain operator"


def test_fused_rejects_missing_tensors_and_bad_shapes(mn):
    import mnq_workloads as workloads
    C = mn._C
    d = workloads.make_layer("t", 2, 256, 64, seed=1).to("cuda")
    for kind in ("bias", "bias_relu", "bias_silu", "residual"):
        with pytest.raises(C.MetalNativeError, match="InvalidArgument"):
            C.dequant_matmul_fused(*d.args(), kind)
    with pytest.raises(C.MetalNativeError, match="InvalidArgument"):
        C.dequant_matmul_fused(*d.args(), "bias", bias=torch.zeros(63, dtype=torch.float16, device="cuda"))
    with pytest.raises(C.MetalNativeError, match="InvalidArgument"):
        C.dequant_matmul_fused(*d.args(), "gelu")
    with pytest.raises(C.MetalNativeError, match="InvalidArgument"):
        C.dequant_matmul_fused(*d.args(), out_dtype=torch.bfloat16)


def test_residual_may_alias_a_strided_view_and_zero_K(mn):
    import mnq_workloads as workloads
    C = mn._C
    L = workloads.make_layer("t", 4, 512, 128, seed=2)
    d = L.to("cuda")
    wide = torch.randn(4, 200, device="cuda").half()
    res = wide[:, 8:136]                          # leading dimension 200
    out = C.dequant_matmul_fused(*d.args(), "residual", residual=res)
    want = H.oracle_matmul(L) + res.float().cpu().numpy()
    H.assert_close_to_oracle(out, want, "strided residual")
    # an empty reduction leaves the epilogue alone: out = bias
    x0 = torch.empty((3, 0), dtype=torch.float16, device="cuda")
    w0 = torch.empty((16, 0), dtype=torch.uint8, device="cuda")
    s0 = torch.empty((16, 0), dtype=torch.float16, device="cuda")
    b = torch.arange(16, device="cuda").half()
    o = C.dequant_matmul_fused(x0, w0, s0, None, 128, "int4", "bias", bias=b)
    assert torch.equal(o, b.expand(3, 16))


@pytest.mark.parametrize("adt,sdt", [(torch.float16, torch.float16), (torch.float16, torch.bfloat16),
                                     (torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float16)])
@pytest.mark.parametrize("M", [8, 24, 64])
def test_select_path_names_the_kernel_that_runs(mn, adt, sdt, M):
    """For every activation / scale dtype pair the host-side answer is the family dispatch takes:
    forcing that family succeeds, and where the tensor-core kernel cannot take the problem (the answer
    is the any-shape kernel), forcing it is refused (it is never silently replaced)."""
    import mnq_workloads as workloads
    C = mn._C
    L = workloads.make_layer("t", M, 1024, 256, act_dtype=adt, scale_dtype=sdt, asymmetric=True, seed=M)
    d = L.to("cuda")
    said = C.select_path(M, 256, 1024, 128, "int4", adt, scale_dtype=sdt)
    code = {"gemv": C.PATH_GEMV, "gemm": C.PATH_GEMM, "generic": C.PATH_GENERIC}[said]
    ref = H.oracle_matmul(L)
    t = C.Tuning()
    t.path = code
    out = C.dequant_matmul(*d.args(), tuning=t)
    assert torch.equal(out, C.dequant_matmul(*d.args())), f"auto dispatch is not the '{said}' kernel"
    H.assert_close_to_oracle(out, ref, f"{said} {adt} {sdt}")
    if M > 32 and said == "generic":
        t.path = C.PATH_GEMM
        with pytest.raises(C.MetalNativeError, match="InvalidArgument"):
            C.dequant_matmul(*d.args(), tuning=t)


def test_gemv_max_m_moves_the_threshold(mn):
    import mnq_workloads as workloads
    C = mn._C
    L = workloads.make_layer("t", 16, 1024, 256, seed=4)
    d = L.to("cuda")
    ref = H.oracle_matmul(L)
    assert C.get_option("gemv_max_m") == 0 and C.select_path(16, 256, 1024, 128, "int4") == "gemv"
    a = C.dequant_matmul(*d.args())
    try:
        C.set_option("gemv_max_m", 8)
        assert C.select_path(16, 256, 1024, 128, "int4") == "gemm"
        assert C.select_path(8, 256, 1024, 128, "int4") == "gemv"
        b = C.dequant_matmul(*d.args())
        with pytest.raises(C.MetalNativeError, match="InvalidArgument"):
            C.set_option("gemv_max_m", 33)
    finally:
        C.set_option("gemv_max_m", 0)
    H.assert_close_to_oracle(a, ref, "gemv at M=16")
    H.assert_close_to_oracle(b, ref, "gemm at M=16")


def test_a_wait_for_a_rank_that_never_comes_runs_out_and_returns(mn):
    """A sharded call on a world of two where the second rank does not exist: its gathered
    output and flag words are ordinary local buffers nobody signals.  With the poll limit set
    low the kernel gives up within milliseconds, returns, and reports bit 2 of the status word
    (TimeoutError); nothing faults or hangs, and the device and the workspace stay usable."""
    import mnq_workloads as workloads
    C = mn._C
    L = workloads.make_layer("t", 1, 4096, 512, seed=6)       # few rows: K is split, arrival counters in use
    d = L.to("cuda")
    want = C.dequant_matmul(*d.args())
    x, w, s, z, g, q = d.args()
    half = 256
    outs = [torch.zeros((1, 512), dtype=torch.float16, device="cuda") for _ in range(2)]
    flags = [torch.zeros(C.GATHER_FLAG_WORDS, dtype=torch.int32, device="cuda") for _ in range(2)]
    assert C.get_option("peer_wait_polls") == 1 << 22
    try:
        C.set_option("peer_wait_polls", 1 << 10)
        C.dequant_matmul_gather(x, w[:half], s[:half], z[:half], g, q, [o.data_ptr() for o in outs],
                                [f.data_ptr() for f in flags], 0, 0, 512)
        C.synchronize()                                        # the call returns: the wait was bounded
        assert C.device_status(clear=False) == 4
        with pytest.raises(C.MetalNativeError, match="TimeoutError"):
            C.check_device_status()
        assert C.device_status() == 0                          # cleared by the check
    finally:
        C.set_option("peer_wait_polls", 1 << 22)
    # the same workspace, the same device: ordinary calls are exact afterwards
    assert torch.equal(C.dequant_matmul(*d.args()), want)
    one = torch.zeros((1, 512), dtype=torch.float16, device="cuda")
    f1 = torch.zeros(C.GATHER_FLAG_WORDS, dtype=torch.int32, device="cuda")
    C.dequant_matmul_gather(x, w, s, z, g, q, [one.data_ptr()], [f1.data_ptr()], 0, 0, 512)
    C.synchronize()
    assert C.device_status() == 0 and torch.equal(one, want)


def test_phase_pipeline_applies_threshold_and_replays_a_captured_decode_step(mn):
    import mnq_workloads as workloads
    C = mn._C
    pipe = mn.PhasePipeline()
    L = workloads.make_layer("t", 1, 2048, 512, seed=8).to("cuda")
    out = torch.zeros((1, 512), dtype=torch.float16, device="cuda")
    want = C.dequant_matmul(*L.args())
    try:
        assert pipe.auto_detect_phase(batch_size=1, seq_len=1) is mn.InferencePhase.Decode
        step = pipe.capture_step(lambda: C.dequant_matmul(*L.args(), out=out))
        for _ in range(3):
            out.zero_()
            step()
            torch.cuda.synchronize()
            assert torch.equal(out, want)
        cfg = pipe.prefill_config()
        cfg.gemv_max_m = 4
        pipe.set_prefill_config(cfg)
        assert pipe.auto_detect_phase(batch_size=4, seq_len=6) is mn.InferencePhase.Prefill
        assert pipe.apply().gemv_max_m == 4 and C.get_option("gemv_max_m") == 4
        assert pipe.strategy_for(24) == "gemm" and C.select_path(24, 512, 2048, 128, "int4") == "gemm"
    finally:
        C.set_option("gemv_max_m", 0)


def test_repeated_calls_replay_the_checked_arguments(mn):
    """A decode loop calls the operator with the same tensor objects step after step; from the second
    call on the shim replays the checked argument list.  The replay must see new contents of the same
    buffers, must not outlive its tensors, and must not be used on another stream."""
    import mnq_workloads as workloads
    C = mn._C
    L = workloads.make_layer("t", 1, 2048, 512, seed=11)
    d = L.to("cuda")
    out = torch.zeros((1, 512), dtype=torch.float16, device="cuda")
    ref = H.oracle_matmul(L)
    for _ in range(3):
        out.zero_()
        assert C.dequant_matmul(*d.args(), out=out) is out
        H.assert_close_to_oracle(out, ref, "replay")
    d.x.mul_(2.0)                                             # same buffer, new contents
    C.dequant_matmul(*d.args(), out=out)
    H.assert_close_to_oracle(out, 2.0 * ref, "replay after an in-place update")
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):                             # another stream: another workspace, no replay
        C.dequant_matmul(*d.args(), out=out)
    side.synchronize()
    H.assert_close_to_oracle(out, 2.0 * ref, "other stream")
    # host activations and output
    xh = L.x.pin_memory()
    oh = torch.zeros((1, 512), dtype=torch.float16).pin_memory()
    for scale in (1.0, 3.0, 1.0):
        xh.copy_(L.x * scale)
        C.dequant_matmul(xh, d.wq, d.scales, d.zeros, d.group_size, d.quant_type, out=oh)
        C.synchronize()
        H.assert_close_to_oracle(oh, scale * ref, f"host replay x{scale}")
    # pageable host memory takes the copying path
    xp = (L.x * 1.0).clone()
    op = torch.zeros((1, 512), dtype=torch.float16)
    C.dequant_matmul(xp, d.wq, d.scales, d.zeros, d.group_size, d.quant_type, out=op)
    C.synchronize()
    H.assert_close_to_oracle(op, ref, "pageable host tensors")
    del out
    out2 = torch.zeros((1, 512), dtype=torch.float16, device="cuda")   # may reuse the freed tensor's id and address
    C.dequant_matmul(*d.args(), out=out2)
    H.assert_close_to_oracle(out2, 2.0 * ref, "fresh output tensor")
