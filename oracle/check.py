"""Checker helpers: run the CPU oracle on a synthetic layer and compare a GPU result with it.

TEST INFRASTRUCTURE ONLY, like the rest of ``oracle/``: imported by ``tests/``, by
``__graft_entry__.smoke()`` and by ``bench.py`` where it checks outputs or times the CPU
path; never by the shipped package."""
from __future__ import annotations

import numpy as np
import torch

from . import oracle

# north-star gate for fp16 outputs, against the oracle's fp32 result
REL_L2_TOL = 1e-3
MAX_ABS_TOL = 2e-2


def f32(t: torch.Tensor | None):
    """Exact widening of an fp16 / bf16 / fp32 tensor to a numpy fp32 array."""
    return None if t is None else t.detach().to("cpu", torch.float32).contiguous().numpy()


def oracle_matmul(layer, cols=None, threads=None) -> np.ndarray:
    """fp32 result of the reference CPU path for ``layer`` (optionally only output
    columns ``cols``: each output element is computed by the same instruction sequence
    whether or not the other columns are present)."""
    wq, s, z = layer.wq.cpu(), layer.scales.cpu(), None if layer.zeros is None else layer.zeros.cpu()
    if cols is not None:
        idx = torch.as_tensor(cols, dtype=torch.long)
        wq, s = wq[idx], s[idx]
        z = None if z is None else z[idx]
    return oracle.dequant_matmul(f32(layer.x), wq.contiguous().numpy(), f32(s), f32(z), layer.group_size,
                                 layer.quant_type, threads=threads or oracle.host_threads())


def oracle_dequant(layer) -> np.ndarray:
    wq = layer.wq.cpu().contiguous().numpy()
    s = f32(layer.scales)
    z = f32(layer.zeros) if layer.zeros is not None else np.zeros_like(s)
    if layer.quant_type == "int4":
        return oracle.dequant_int4(wq, s, z, layer.K, layer.N, layer.group_size)
    return oracle.dequant_int8(wq, s, z, layer.K, layer.N, layer.group_size)


def errors(got: np.ndarray, ref: np.ndarray):
    got = got.astype(np.float64)
    ref = ref.astype(np.float64)
    diff = got - ref
    den = float(np.sqrt((ref ** 2).sum()))
    rel = float(np.sqrt((diff ** 2).sum())) / (den if den > 0 else 1.0)
    return rel, float(np.abs(diff).max()) if diff.size else 0.0


def assert_close_to_oracle(out: torch.Tensor, ref: np.ndarray, what: str = ""):
    """fp16 outputs: rel-L2 <= 1e-3 and max-abs <= 2e-2 against the oracle's fp32 result (for
    |y| >= 32, where adjacent fp16 values are further apart than that, one fp16 ulp).

    bf16 outputs cannot meet that gate whatever the kernel does (rounding the exact result
    to bf16 already costs ~1.6e-3 rel-L2), so they are held to the rounding floor instead:
    the error against the fp32 oracle may exceed the error of RN_bf16(oracle) by at most
    5 %, and every element must be within one bf16 ulp (2^-7 relative) of the oracle value,
    plus 1e-4 of the output RMS for outputs that nearly cancel."""
    got = out.detach().to("cpu", torch.float32).numpy()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert np.isfinite(got).all(), f"{what}: non-finite output"
    rel, mx = errors(got, ref)
    if out.dtype == torch.float16:
        assert rel <= REL_L2_TOL, f"{what}: rel-L2 {rel:.3e} > {REL_L2_TOL}"
        # max-abs <= 2e-2 wherever fp16 can deliver it.  From |y| >= 32 on the fp16 grid itself
        # is 3.1e-2 wide (6.3e-2 from 64), so there the bound is one fp16 ulp of the value.
        ulp = 2.0 ** (np.floor(np.log2(np.maximum(np.abs(ref), 1e-30))) - 10)
        bound = np.maximum(MAX_ABS_TOL, ulp)
        worst = float(np.max(np.abs(got - ref) / bound)) if ref.size else 0.0
        assert worst <= 1.0, f"{what}: max-abs {mx:.3e}: {worst:.2f}x the bound max(2e-2, 1 fp16 ulp)"
        return rel, mx
    assert out.dtype == torch.bfloat16
    ideal = torch.from_numpy(ref).to(torch.bfloat16)
    rel0, _ = errors(ideal.float().numpy(), ref)
    assert rel <= rel0 * 1.05 + 1e-6, f"{what}: rel-L2 {rel:.3e} vs bf16 rounding floor {rel0:.3e}"
    # element-wise: within one bf16 ulp of the oracle value (2^-7 relative), plus an
    # absolute allowance for fp32 summation-order noise on outputs that nearly cancel
    rms = float(np.sqrt(np.mean(ref.astype(np.float64) ** 2))) if ref.size else 0.0
    bound = np.abs(ref) * 2.0 ** -7 + 1e-4 * rms + 1e-30
    worst = float(np.max(np.abs(got - ref) / bound)) if ref.size else 0.0
    assert worst <= 1.0, f"{what}: element error {worst:.2f}x the bf16 one-ulp bound"
    return rel, mx


def assert_fp32_gate(out32: torch.Tensor, ref: np.ndarray, what: str = ""):
    """The north-star gate, rel-L2 <= 1e-3 and max-abs <= 2e-2 against the oracle's fp32 result,
    applied to the fp32 output mode of a kernel (its accumulators before the final rounding): how
    a bf16-output configuration is held to the stated tolerance, which no bf16 value can meet."""
    assert out32.dtype == torch.float32
    got = out32.detach().cpu().numpy()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    rel, mx = errors(got, ref)
    assert rel <= REL_L2_TOL, f"{what}: fp32-output rel-L2 {rel:.3e} > {REL_L2_TOL}"
    assert mx <= MAX_ABS_TOL, f"{what}: fp32-output max-abs {mx:.3e} > {MAX_ABS_TOL}"
    return rel, mx


def sampled_columns(N: int, count: int, world: int = 1, seed: int = 0) -> np.ndarray:
    """``count`` distinct output columns, the same number from every rank's slice of a
    column-sharded [., N] output, always including the first and last column of each slice."""
    rng = np.random.default_rng(seed)
    per = max(2, count // world)
    n_local = N // world
    cols = []
    for r in range(world):
        lo = r * n_local
        inner = rng.choice(np.arange(lo + 1, lo + n_local - 1), size=min(per - 2, n_local - 2), replace=False)
        cols.extend([lo, lo + n_local - 1, *inner.tolist()])
    return np.array(sorted(set(cols)), dtype=np.int64)
