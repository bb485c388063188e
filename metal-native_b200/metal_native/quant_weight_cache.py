"""QuantWeightCache: keeps quantised weights by name and hands out fp16 copies on demand.

Mirror of the reference's C++ class (``src/memory/quant_weight_cache.mm:41-191``,
``src/memory/quant_weight_cache.h``): ``register_weight`` / ``get_dequantized`` /
``evict_dequantized`` and the footprint queries, over torch CUDA tensors.  As in the
reference, dequantisation uses the standalone kernels (scale only, no zero-point, group
size inferred as ``elements / scales.numel()``) and the fp16 copy is cached only while
there is memory to spare.  The reference asks its memory-budget controller for a
"pressure multiplier" (cache if >= 0.5); here the same threshold is applied to the
fraction of device memory that is free.
"""
from __future__ import annotations

import enum
import threading
from dataclasses import dataclass

import torch

from . import _C


class QuantFormat(enum.Enum):
    INT8 = "int8"
    INT4 = "int4"


@dataclass
class _Entry:
    quantized: torch.Tensor
    scales: torch.Tensor
    fmt: QuantFormat
    num_elements: int
    group_size: int
    dequantized: torch.Tensor | None = None


class QuantWeightCache:
    def __init__(self, cache_threshold: float = 0.5, pressure_fn=None):
        self._mu = threading.Lock()
        self._weights: dict[str, _Entry] = {}
        self._threshold = cache_threshold
        self._pressure_fn = pressure_fn

    def register_weight(self, name: str, quantized: torch.Tensor, scales: torch.Tensor,
                        fmt: QuantFormat = QuantFormat.INT8) -> None:
        """src/memory/quant_weight_cache.mm:41-63: elements = numel (int8) or 2*numel (int4);
        group size = elements / scales.numel()."""
        if scales.numel() == 0:
            raise _C.MetalNativeError(4, "quant_weight_cache: scales is empty")
        n = quantized.numel() * (2 if fmt == QuantFormat.INT4 else 1)
        with self._mu:
            self._weights[name] = _Entry(quantized, scales, fmt, n, n // scales.numel())

    def _multiplier(self, device) -> float:
        if self._pressure_fn is not None:
            return float(self._pressure_fn())
        free, total = torch.cuda.mem_get_info(device)
        return free / total

    def get_dequantized(self, name: str) -> torch.Tensor:
        """src/memory/quant_weight_cache.mm:65-153.  Output has the shape of the quantised
        tensor, last dimension doubled for int4, dtype fp16."""
        with self._mu:
            e = self._weights.get(name)
            if e is None:
                raise _C.MetalNativeError(4, "quant_weight_cache: weight not registered")
            if e.dequantized is not None:
                return e.dequantized
            flat = _C.dequantize_flat(e.quantized, e.scales.to(torch.float16).contiguous().view(-1),
                                      e.group_size, e.fmt.value, e.num_elements)
            shape = list(e.quantized.shape)
            if e.fmt == QuantFormat.INT4:
                shape[-1] *= 2
            out = flat.view(shape)
            if self._multiplier(e.quantized.device) >= self._threshold:
                e.dequantized = out
            return out

    def evict_dequantized(self) -> None:
        with self._mu:
            for e in self._weights.values():
                e.dequantized = None

    def dequantized_footprint(self) -> int:
        """Bytes held by cached fp16 copies (src/memory/quant_weight_cache.mm:162-171)."""
        with self._mu:
            return sum(e.num_elements * 2 for e in self._weights.values() if e.dequantized is not None)

    def total_footprint(self) -> int:
        """Quantised storage + fp16 scales + cached fp16 copies
        (src/memory/quant_weight_cache.mm:173-191)."""
        with self._mu:
            total = 0
            for e in self._weights.values():
                total += e.num_elements if e.fmt == QuantFormat.INT8 else e.num_elements // 2
                total += e.scales.numel() * 2
                if e.dequantized is not None:
                    total += e.num_elements * 2
            return total
