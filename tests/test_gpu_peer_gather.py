"""The fused operator + all-gather (mnq_dequant_matmul_gather): the decode kernel's epilogue
stores this rank's output columns into every rank's gathered buffer through peer pointers and
its last CTA exchanges arrival flags.

On one GPU the protocol is exercised with a world of one rank (the rank is its own only peer,
so nothing waits on another launch).  With two or more GPUs a second test starts one process
per GPU (torchrun, NCCL only for the rendezvous and the reference all-gather) and compares
the fused result with the ordinary operator followed by an all-gather.
"""
import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

from oracle import check as H

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def mn():
    import metal_native
    assert torch.cuda.is_available()
    return metal_native


@pytest.mark.parametrize("M,K,N,quant,g,adt", [
    (1, 1024, 512, "int4", 128, torch.float16),     # K split over chunks: the last-arriver path stores to peers
    (1, 512, 4096, "int4", 128, torch.float16),     # one chunk: the direct epilogue stores to peers
    (4, 2048, 256, "int8", 2048, torch.bfloat16),   # several tokens, per-channel int8, bf16
    (16, 1024, 208, "int4", 128, torch.bfloat16),   # two token tiles, N not a multiple of the CTA's rows
])
def test_world_of_one_matches_the_plain_operator(mn, M, K, N, quant, g, adt):
    import mnq_workloads as workloads
    C = mn._C
    L = workloads.make_layer("t", M, K, N, quant_type=quant, group_size=g, act_dtype=adt,
                             asymmetric=adt == torch.float16, seed=K + N).to("cuda")
    want = C.dequant_matmul(*L.args())
    ref = H.oracle_matmul(L.to("cpu"))
    ldc = N + 24
    wide = torch.full((M, ldc), 7.0, dtype=adt, device="cuda")
    flags = torch.zeros(C.GATHER_FLAG_WORDS, dtype=torch.int32, device="cuda")
    for call in (1, 2, 3):
        wide.fill_(7.0)
        C.dequant_matmul_gather(*L.args(), [wide.data_ptr()], [flags.data_ptr()], 0, 16, ldc)
        C.synchronize()
        assert C.device_status() == 0
        assert torch.equal(wide[:, 16:16 + N], want)
        assert bool((wide[:, :16] == 7.0).all()) and bool((wide[:, 16 + N:] == 7.0).all())
        f = flags.cpu().tolist()
        assert f[0] == call and f[16] == call and f[9] == call and f[8] == 0, f
    H.assert_close_to_oracle(want, ref, f"gather {quant} {M}x{N}x{K}")


def test_shapes_outside_the_decode_kernel_are_refused(mn):
    import mnq_workloads as workloads
    C = mn._C
    L = workloads.make_layer("t", 64, 256, 128, seed=3).to("cuda")    # M > 32: tensor-core path, no fused gather
    out = torch.empty((64, 128), dtype=torch.float16, device="cuda")
    flags = torch.zeros(C.GATHER_FLAG_WORDS, dtype=torch.int32, device="cuda")
    with pytest.raises(C.MetalNativeError, match="NotImplemented"):
        C.dequant_matmul_gather(*L.args(), [out.data_ptr()], [flags.data_ptr()], 0, 0, 128)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_gather_through_peer_stores():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", "29561", str(ROOT / "tests" / "peer_gather_worker.py")]
    r = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=240)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    assert "peer gather ok" in r.stdout
