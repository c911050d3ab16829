"""Activation names and their backend mapping (gomlx/gomlx ml/layers/activation/activation.go:35-75)."""
from __future__ import annotations

import enum


class ActivationType(enum.IntEnum):
    """compute.ActivationType: what a fused backend op can apply in its epilogue."""

    NONE = 0
    GELU = 1
    RELU = 2
    SILU = 3
    HARD_SWISH = 4
    TANH = 5


class Type(enum.Enum):
    """activation.Type: the user-level activation names."""

    NONE = "none"
    RELU = "relu"
    LEAKY_RELU = "leaky_relu"
    SIGMOID = "sigmoid"
    HARD_SIGMOID = "hard_sigmoid"
    TANH = "tanh"
    SWISH = "swish"
    SILU = "silu"
    HARD_SWISH = "hard_swish"
    SELU = "selu"
    GELU = "gelu"
    GELU_APPROX = "gelu_approx"
    SWIGLU = "swiglu"

    def to_backend(self) -> ActivationType:
        """activation.Type.ToBackend (activation.go:58-75).  Types the fused op cannot apply map
        to NONE without an error, exactly as the reference does; exact and approximate GELU
        both map to GELU, which this backend evaluates in the exact erf form."""
        return {
            Type.GELU: ActivationType.GELU,
            Type.GELU_APPROX: ActivationType.GELU,
            Type.RELU: ActivationType.RELU,
            Type.SWISH: ActivationType.SILU,
            Type.SILU: ActivationType.SILU,
            Type.HARD_SWISH: ActivationType.HARD_SWISH,
            Type.TANH: ActivationType.TANH,
        }.get(self, ActivationType.NONE)
