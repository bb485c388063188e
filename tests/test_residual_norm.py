"""The fused residual + RMSNorm operator (the reference's fast::fused_residual_norm): the CPU
restatement on a hand-checked case (CPU), the exported symbol and host-side validation (CPU), and
the CUDA kernel against the restatement (GPU)."""
import ctypes

import numpy as np
import pytest
import torch

from oracle import oracle


def test_restatement_on_a_hand_checked_row():
    # input + residual = [3, 4, 0, 0]: mean of squares 25/4, rms_inv = 0.4 with eps = 0
    x = np.array([[1.0, 1.5, -2.0, 0.25]], np.float32)
    r = np.array([[2.0, 2.5, 2.0, -0.25]], np.float32)
    w = np.array([1.0, 0.5, 3.0, 7.0], np.float32)
    out, h = oracle.residual_rms_norm(x, r, w, 0.0, "fp16")
    assert h.tolist() == [[3.0, 4.0, 0.0, 0.0]]
    want = oracle.fp16_bits_to_fp32(oracle.fp32_to_fp16_bits(np.array([[1.2, 0.8, 0.0, 0.0]], np.float32)))
    assert np.array_equal(out, want)
    # the sum is rounded before it is normalised, the mean uses the unrounded sum: 2049 is not an fp16 value
    x = np.array([[2048.0, 0.0]], np.float32)
    r = np.array([[1.0, 0.0]], np.float32)
    out, h = oracle.residual_rms_norm(x, r, np.ones(2, np.float32), 0.0, "fp16")
    assert h[0, 0] == 2048.0
    inv = np.float32(1.0) / np.sqrt(np.float32(2049.0 * 2049.0 / 2.0))
    assert out[0, 0] == oracle.fp16_bits_to_fp32(oracle.fp32_to_fp16_bits(np.array([np.float32(2048.0) * inv], np.float32)))[0]


def test_restatement_against_the_reference_test_suites_rms_norm_formula():
    """x / sqrt(mean(x^2) + eps) * weight on x = input + residual, in float64 (the formula of the
    reference's tests/test_numerical_accuracy.py:68-84): the restatement differs only by its
    16-bit roundings (the sum, the output)."""
    rng = np.random.default_rng(11)
    for kind, ulp in (("fp16", 2.0 ** -10), ("bf16", 2.0 ** -7)):
        to_bits, from_bits = ((oracle.fp32_to_fp16_bits, oracle.fp16_bits_to_fp32) if kind == "fp16"
                              else (oracle.fp32_to_bf16_bits, oracle.bf16_bits_to_fp32))
        q = lambda a: from_bits(to_bits(a.astype(np.float32)))
        x, r = q(rng.standard_normal((5, 768)) * 3), q(rng.standard_normal((5, 768)))
        w = q(1.0 + 0.2 * rng.standard_normal(768))
        out, h = oracle.residual_rms_norm(x, r, w, 1e-5, kind)
        s = x.astype(np.float64) + r.astype(np.float64)
        want = s / np.sqrt((s ** 2).mean(axis=-1, keepdims=True) + 1e-5) * w.astype(np.float64)
        # one rounding of the sum (relative ulp/2) and one of the output (ulp/2), plus slack
        assert np.all(np.abs(out - want) <= 1.6 * ulp * np.abs(want) + 1e-6)
        assert np.all(np.abs(h - s) <= 0.5 * ulp * np.abs(s) + 1e-12)


def test_symbol_is_exported_and_validates_on_the_host():
    from metal_native import _C
    assert "mnq_residual_rmsnorm" in _C.exported_symbols()
    f = _C._lib.mnq_residual_rmsnorm
    one = ctypes.c_void_p(4096)
    # nothing is launched: empty shapes succeed, bad arguments are refused before any CUDA call
    assert f(None, None, None, None, None, 0, 128, 128, 128, 128, 0, 1e-6, 0, None) == 0
    assert f(one, one, one, one, None, 4, 128, 64, 128, 128, 0, 1e-6, 0, None) == 4     # row stride < row length
    assert f(one, one, one, one, None, 4, 128, 128, 128, 128, 0, 1e-6, 2, None) == 4    # fp32 is not a storage type here
    assert f(one, None, one, one, None, 4, 128, 128, 128, 128, 0, 1e-6, 0, None) == 4   # null tensor
    assert b"fused_residual_norm" in _C._lib.mnq_last_error()


def _close(got: torch.Tensor, ref: np.ndarray, what: str):
    """Within two units in the last place of the 16-bit type (the order in which the squares are
    added moves rms_inv by an fp32 ulp or two, which can move a rounding boundary)."""
    g = got.detach().float().cpu().numpy()
    rel = 2.0 ** (-9 if got.dtype == torch.float16 else -6)
    bad = np.abs(g - ref) > rel * np.abs(ref) + 1e-7
    assert not bad.any(), f"{what}: {int(bad.sum())} elements off, worst {np.abs(g - ref).max():.3e}"


@pytest.mark.gpu
@pytest.mark.parametrize("rows,hidden,dt", [
    (1, 3584, torch.float16), (32, 4096, torch.bfloat16), (7, 8192, torch.float16), (5, 16384, torch.bfloat16),
    (3, 100, torch.float16),          # not a multiple of 8: the any-length path
    (2, 18944, torch.float16),        # longer than the register cache
    (64, 896, torch.bfloat16),
])
def test_kernel_matches_the_restatement(rows, hidden, dt):
    import metal_native
    g = torch.Generator(device="cpu").manual_seed(rows * 131 + hidden)
    x = (torch.randn((rows, hidden), generator=g) * 2.0).to(dt)
    r = (torch.randn((rows, hidden), generator=g) * 0.5).to(dt)
    w = (1.0 + 0.1 * torch.randn(hidden, generator=g)).to(dt)
    kind = "fp16" if dt == torch.float16 else "bf16"
    ref, ref_sum = oracle.residual_rms_norm(x.float().numpy(), r.float().numpy(), w.float().numpy(), 1e-6, kind)
    xs = torch.empty_like(x, device="cuda")
    out = metal_native.fused_residual_norm(x.cuda(), r.cuda(), w.cuda(), 1e-6, sum_out=xs)
    metal_native.synchronize()
    _close(out, ref, f"{rows}x{hidden} {kind}")
    assert np.array_equal(xs.float().cpu().numpy(), ref_sum), "rounded sums differ"
    # in place: the result over the input, the new residual stream over the residual
    xi, ri = x.cuda(), r.cuda()
    metal_native.fused_residual_norm(xi, ri, w.cuda(), 1e-6, out=xi, sum_out=ri)
    metal_native.synchronize()
    assert torch.equal(xi, out) and torch.equal(ri, xs)


@pytest.mark.gpu
def test_strided_rows_leading_dimensions_and_errors():
    import metal_native
    C = metal_native._C
    g = torch.Generator(device="cpu").manual_seed(5)
    wide = torch.randn((6, 3 * 512), generator=g).to(torch.float16).cuda()
    x, r = wide[:, :512], wide[:, 1024:]                 # rows 1536 apart
    w = torch.ones(512, dtype=torch.float16, device="cuda")
    ref, _ = oracle.residual_rms_norm(x.float().cpu().numpy(), r.float().cpu().numpy(), np.ones(512, np.float32), 1e-5, "fp16")
    out = C.fused_residual_norm(x, r, w, 1e-5)
    _close(out, ref, "strided")
    x3 = torch.randn((2, 3, 256), generator=g).to(torch.bfloat16).cuda()
    o3 = C.fused_residual_norm(x3, x3, torch.ones(256, dtype=torch.bfloat16, device="cuda"))
    assert o3.shape == x3.shape
    with pytest.raises(C.MetalNativeError, match="InvalidArgument"):
        C.fused_residual_norm(x, r[:, :256], w)
    with pytest.raises(C.MetalNativeError, match="InvalidArgument"):
        C.fused_residual_norm(x, r, w.float())
    with pytest.raises(C.MetalNativeError, match="InvalidArgument"):
        C.fused_residual_norm(x.cpu(), r, w)
