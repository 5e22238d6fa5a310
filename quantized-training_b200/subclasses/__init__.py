"""Tensor subclasses that change how `F.linear` is computed for a weight, with the reference's
names (subclasses/__init__.py:1-18). INT8 weight-only, INT8 mixed precision and BitNet run on the
sm_100a kernels of `gn_kernels`; the INT4 weight-only subclass is outside this build."""
from .bitnet import BitNetTrainingLinearWeight, convert_bitnet
from .int8 import Int8LinearWeight, Int8QTConfig, convert_int8_quantized_training, quantize_int8
from .mixed_precision import MixedPrecisionConfig, MixedPrecisionLinearWeight, convert_mixed_precision


def convert_int4_quantized_training(*args, **kwargs):
    raise NotImplementedError("INT4 weight-only training is outside the INT8/FP8 path this build covers")


class Int4LinearWeight:  # placeholder so `from subclasses import Int4LinearWeight` keeps importing
    def __init__(self, *args, **kwargs):
        raise NotImplementedError("INT4 weight-only training is outside the INT8/FP8 path this build covers")


__all__ = [
    "BitNetTrainingLinearWeight",
    "convert_bitnet",
    "Int4LinearWeight",
    "convert_int4_quantized_training",
    "Int8LinearWeight",
    "Int8QTConfig",
    "convert_int8_quantized_training",
    "MixedPrecisionConfig",
    "MixedPrecisionLinearWeight",
    "convert_mixed_precision",
    "quantize_int8",
]
