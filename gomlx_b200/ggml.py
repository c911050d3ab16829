"""GGML block-format metadata: the Python face of compute.GGMLQuantType and of
ggml.CanDecompose (gomlx/gomlx ml/ggml/dequant.go:20-27,41,52)."""
from __future__ import annotations

import enum


class GGMLQuantType(enum.IntEnum):
    """compute.GGMLQuantType; the numeric values are GGML's own type ids."""

    Q4_0 = 2
    Q8_0 = 8
    Q4_K = 12
    Q6_K = 14
    IQ4NL = 20

    def bytes_per_block(self) -> int:
        """GGMLQuantType.BytesPerBlock (ml/ggml/dequant.go:41)."""
        return {2: 18, 8: 34, 12: 144, 14: 210, 20: 18}[int(self)]

    def values_per_block(self) -> int:
        """GGMLQuantType.ValuesPerBlock (ml/ggml/gather.go:25)."""
        return {2: 32, 8: 32, 12: 256, 14: 256, 20: 32}[int(self)]

    def __str__(self) -> str:
        return {2: "Q4_0", 8: "Q8_0", 12: "Q4_K", 14: "Q6_K", 20: "IQ4_NL"}[int(self)]


def can_decompose(t: GGMLQuantType) -> bool:
    """ggml.CanDecompose (ml/ggml/dequant.go:20-27): formats with a graph-level fallback."""
    return t in (GGMLQuantType.Q4_0, GGMLQuantType.Q8_0, GGMLQuantType.IQ4NL)


def row_bytes(t: GGMLQuantType, k: int) -> int:
    """Bytes per weight row for K logical values."""
    if k % t.values_per_block():
        raise ValueError(f"K={k} is not a multiple of {t.values_per_block()} for {t}")
    return k // t.values_per_block() * t.bytes_per_block()


def logical_k(t: GGMLQuantType, bytes_per_row: int) -> int:
    """K = (bytesPerRow / bytesPerBlock) * valuesPerBlock (ml/nn/quantized_gather.go:28-29)."""
    if bytes_per_row % t.bytes_per_block():
        raise ValueError(f"bytesPerRow={bytes_per_row} is not a multiple of {t.bytes_per_block()} for {t}")
    return bytes_per_row // t.bytes_per_block() * t.values_per_block()
