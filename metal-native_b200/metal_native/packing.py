"""Packing of 4-bit weights into the operator's layout."""
from __future__ import annotations

import torch


def pack_int4(values: torch.Tensor) -> torch.Tensor:
    """[N, K] integers 0..15 -> [N, K/2] uint8, element k in the low nibble for even k and
    in the high nibble for odd k: the layout ``dequant_matmul`` reads
    (``shaders/matmul_dequant_kernel.metal:29-44``; the reference's own packer is the test
    helper ``tests/cpp/test_dequant_matmul.mm:104-116``).  K must be even."""
    if values.dim() != 2 or values.shape[1] % 2:
        raise ValueError("pack_int4 expects [N, K] with K even")
    v = values.to(torch.uint8) & 0xF
    return (v[:, 0::2] | (v[:, 1::2] << 4)).contiguous()
