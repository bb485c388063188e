"""Seeded random problems through the default dispatch (whatever kernel the library picks for each)
against the CPU oracle: token counts across every kernel family's range, ragged N, K that is or is
not a whole number of pieces, every weight format / group size / activation type combination the
operator accepts.  Needs a B200."""
import random

import pytest
import torch

from oracle import check as H

pytestmark = pytest.mark.gpu


def _cases():
    rng = random.Random(20240607)
    out = []
    for i in range(48):
        quant = rng.choice(["int4", "int4", "int8"])
        adt = rng.choice([torch.float16, torch.bfloat16])
        M = rng.choice([1, 2, 3, 4, 5, 6, 7, 8, 9, 12, 16, 17, 23, 24, 25, 31, 32, 33, 40, 64, 65, 100, 128, 129, 200])
        N = rng.choice([16, 24, 48, 100, 128, 272, 520, 1000, 1024, 2064, 4096])
        kind = rng.choice(["pieces", "blocks", "ragged"])
        if kind == "pieces":
            K = 512 * rng.choice([1, 2, 3, 5, 8, 16])
        elif kind == "blocks":
            K = 64 * rng.choice([1, 3, 5, 7, 9, 17, 33])
        else:
            K = 32 * rng.choice([1, 3, 5, 11])
        groups = [g for g in (32, 64, 128) if K % g == 0] + [K]
        g = rng.choice(groups)
        asym = rng.random() < 0.6
        if quant == "int8":
            sdt = torch.float16 if adt == torch.float16 or rng.random() < 0.5 else torch.bfloat16
        else:
            sdt = adt
        out.append((i, quant, M, N, K, g, asym, adt, sdt))
    return out


@pytest.mark.parametrize("i,quant,M,N,K,g,asym,adt,sdt", _cases())
def test_random_problem(i, quant, M, N, K, g, asym, adt, sdt):
    import metal_native
    import mnq_workloads as workloads
    C = metal_native._C
    L = workloads.make_layer("t", M, K, N, quant_type=quant, group_size=g, act_dtype=adt, scale_dtype=sdt,
                             asymmetric=asym, seed=1000 + i)
    ref = H.oracle_matmul(L, threads=4)
    d = L.to("cuda")
    path = C.select_path(M, N, K, g, quant, adt, scale_dtype=sdt)
    a = C.dequant_matmul(*d.args())
    b = C.dequant_matmul(*d.args())
    C.synchronize()
    assert C.device_status() == 0
    H.assert_close_to_oracle(a, ref, f"case {i}: {quant} {M}x{N}x{K} g{g} {adt} via {path}")
    assert torch.equal(a, b), f"case {i}: not deterministic ({path})"
