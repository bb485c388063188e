"""Seeded synthetic layers with the shapes and value distributions of the benchmark
configurations (Qwen2.5 / Llama-3 MLP projections).  No model weights or datasets are
involved: nibbles are uniform 0..15, int8 values uniform -127..127, scales uniform in a
small positive range, activations standard normal.

Everything is generated on the CPU with a seeded ``torch.Generator`` so that a CPU
checker and the GPU see identical bits; tensors are moved by the caller.

Benchmark and test input only: this module sits beside the ``metal_native`` package, not in
it, and imports nothing from it, so generating inputs never loads the CUDA library.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch


def pack_int4(values: torch.Tensor) -> torch.Tensor:
    """[N, K] integers 0..15 -> [N, K/2] uint8, element k in the low nibble for even k and
    in the high nibble for odd k (the reference's ``pack_int4``,
    ``tests/cpp/test_dequant_matmul.mm:104-116``).  K must be even."""
    if values.dim() != 2 or values.shape[1] % 2:
        raise ValueError("pack_int4 expects [N, K] with K even")
    v = values.to(torch.uint8) & 0xF
    return (v[:, 0::2] | (v[:, 1::2] << 4)).contiguous()


@dataclass
class Layer:
    """One quantised projection: ``out = x @ dequant(wq, scales, zeros).T``."""
    name: str
    quant_type: str          # "int4" | "int8"
    M: int
    K: int
    N: int
    group_size: int          # == K for one scale per output row
    x: torch.Tensor          # [M, K] fp16 / bf16
    wq: torch.Tensor         # [N, K/2] uint8 or [N, K] int8
    scales: torch.Tensor     # [N, G]
    zeros: torch.Tensor | None

    @property
    def G(self) -> int:
        return (self.K + self.group_size - 1) // self.group_size

    @property
    def weight_bytes(self) -> int:
        """Packed weights + scales + zeros, each counted once."""
        n = self.wq.numel() * self.wq.element_size() + self.scales.numel() * self.scales.element_size()
        if self.zeros is not None:
            n += self.zeros.numel() * self.zeros.element_size()
        return n

    @property
    def total_bytes(self) -> int:
        """weight_bytes + activations + output, each counted once."""
        return self.weight_bytes + self.x.numel() * self.x.element_size() + self.M * self.N * self.x.element_size()

    @property
    def flops(self) -> int:
        return 2 * self.M * self.N * self.K

    def to(self, device) -> "Layer":
        return Layer(self.name, self.quant_type, self.M, self.K, self.N, self.group_size,
                     self.x.to(device), self.wq.to(device), self.scales.to(device),
                     None if self.zeros is None else self.zeros.to(device))

    def args(self):
        """Positional arguments of ``metal_native._C.dequant_matmul``."""
        return (self.x, self.wq, self.scales, self.zeros, self.group_size, self.quant_type)


def make_layer(name: str, M: int, K: int, N: int, *, quant_type: str = "int4", group_size: int = 128,
               act_dtype: torch.dtype = torch.float16, scale_dtype: torch.dtype = torch.float16,
               asymmetric: bool = True, scale_range=None, seed: int = 0,
               gen: torch.Generator | None = None) -> Layer:
    """Builds one layer.  Asymmetric int4 layers draw an integer zero-point zp in 0..15 per
    (row, group) and encode it as the post-scale offset the operator's formula uses,
    ``z = round_to_scale_dtype((zp - 8) * s)``, so that ``(q-8)*s - z == (q - zp)*s`` up to
    that rounding."""
    g = gen if gen is not None else torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn((M, K), generator=g, dtype=torch.float32).to(act_dtype)
    G = (K + group_size - 1) // group_size
    if quant_type == "int4":
        q = torch.randint(0, 16, (N, K), generator=g, dtype=torch.uint8)
        wq = pack_int4(q)
        del q
    elif quant_type == "int8":
        wq = torch.randint(-127, 128, (N, K), generator=g, dtype=torch.int8)
    else:
        raise ValueError(quant_type)
    if scale_range is None:   # keeps |w| <= ~0.16 for both formats
        scale_range = (0.005, 0.02) if quant_type == "int4" else (0.0003, 0.00125)
    lo, hi = scale_range
    scales32 = torch.rand((N, G), generator=g, dtype=torch.float32) * (hi - lo) + lo
    scales = scales32.to(scale_dtype)
    zeros = None
    if asymmetric:
        zp = torch.randint(0, 16, (N, G), generator=g, dtype=torch.int32).to(torch.float32)
        zeros = ((zp - 8.0) * scales.to(torch.float32)).to(scale_dtype)
    return Layer(name, quant_type, M, K, N, group_size, x, wq, scales, zeros)


# ---------------------------------------------------------------------------
# The benchmark configurations
# ---------------------------------------------------------------------------

def config0(seed: int = 0) -> list[Layer]:
    """Qwen2.5-0.5B down projection, M=1, K=4864, N=896, int4 group 64, asymmetric.
    The configuration is specified with fp32 activations; the operator takes fp16, so the
    activations are the fp16 rounding of the seeded normal draw (checker and GPU both
    consume those fp16 values)."""
    return [make_layer("qwen2.5-0.5b.down", 1, 4864, 896, group_size=64, seed=seed)]


def config1(seed: int = 1, M: int = 1) -> list[Layer]:
    """Qwen2.5-7B decode: fused gate+up (K=3584, N=37888) then down (K=18944, N=3584),
    int4 group 128 asymmetric, fp16."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return [make_layer("qwen2.5-7b.gate_up", M, 3584, 37888, gen=g),
            make_layer("qwen2.5-7b.down", M, 18944, 3584, gen=g)]


def config2(M: int, seed: int = 2) -> list[Layer]:
    """Llama-3-8B batched decode, M in {4, 16, 32}: gate/up (K=4096, N=14336) and down
    (K=14336, N=4096), int4 symmetric group 128, bf16 activations and scales."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    kw = dict(act_dtype=torch.bfloat16, scale_dtype=torch.bfloat16, asymmetric=False, gen=g)
    return [make_layer("llama3-8b.gate_up", M, 4096, 14336, **kw),
            make_layer("llama3-8b.down", M, 14336, 4096, **kw)]


def config3(seed: int = 3, M: int = 512) -> list[Layer]:
    """Prefill: M=512 against the Qwen2.5-7B up (K=3584, N=18944) and down
    (K=18944, N=3584) projections, int4 group 128 asymmetric, fp16."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    return [make_layer("qwen2.5-7b.up.prefill", M, 3584, 18944, gen=g),
            make_layer("qwen2.5-7b.down.prefill", M, 18944, 3584, gen=g)]


def config4(M: int, seed: int = 4, world_size: int = 1, rank: int = 0, scale_down: int = 1) -> list[Layer]:
    """Llama-3-70B layers, int8 per-channel symmetric (fp16 scales U(0.001, 0.01)), bf16
    activations: fused gate+up (K=8192, N=57344) and down (K=28672, N=8192).  The whole matrix is
    drawn from one seed whatever the world size; with ``world_size`` > 1 this rank keeps its block
    of output rows (column sharding over N), so the ranks' slices together are exactly the
    matrix a single GPU gets.  ``scale_down`` divides N (tests use it to keep the CPU checker
    fast)."""
    layers = []
    for i, (name, K, N) in enumerate((("llama3-70b.gate_up", 8192, 57344), ("llama3-70b.down", 28672, 8192))):
        N //= scale_down
        if N % world_size:
            raise ValueError(f"N={N} is not divisible by world_size={world_size}")
        gx = torch.Generator(device="cpu").manual_seed(seed * 1000 + i)
        x = torch.randn((M, K), generator=gx, dtype=torch.float32).to(torch.bfloat16)
        gw = torch.Generator(device="cpu").manual_seed(seed * 1000 + 100 + i)
        n_local = N // world_size
        # rows are drawn in blocks of 1024 from the one generator, every rank walking the same
        # sequence and keeping only its own rows (a whole [N, K] draw would need 470 MB per rank)
        lo, hi = rank * n_local, (rank + 1) * n_local
        wq = torch.empty((n_local, K), dtype=torch.int8)
        for r0 in range(0, N, 1024):
            r1 = min(N, r0 + 1024)
            blk = torch.randint(-127, 128, (r1 - r0, K), generator=gw, dtype=torch.int8)
            a, b = max(r0, lo), min(r1, hi)
            if a < b:
                wq[a - lo:b - lo] = blk[a - r0:b - r0]
        scales = (torch.rand((N, 1), generator=gw, dtype=torch.float32) * 0.009 + 0.001).to(torch.float16)[lo:hi].contiguous()
        layers.append(Layer(name, "int8", M, K, n_local, K, x, wq, scales, None))
    return layers
