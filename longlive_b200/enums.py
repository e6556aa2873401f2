"""Enumerations of the quantization API (same names and values as the reference's
fouroversix/src/fouroversix/utils.py:12-134, so configs written for it keep working)."""
from __future__ import annotations

from enum import Enum

import torch


class DataType(str, Enum):
    bfloat16 = "bfloat16"
    float16 = "float16"
    float32 = "float32"
    mxfp4 = "mxfp4"
    nvfp4 = "nvfp4"

    def block_size(self):
        return {"mxfp4": 32, "nvfp4": 16}.get(self.value)

    def scale_dtype(self):
        return {"mxfp4": torch.float8_e8m0fnu, "nvfp4": torch.float8_e4m3fn}.get(self.value)

    def torch_dtype(self):
        return {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32}.get(self.value)


class MatmulBackend(str, Enum):
    """``cutlass`` (and ``None``) select the tcgen05 kernel of this package; ``pytorch`` is not
    part of the product and is rejected."""
    cutlass = "cutlass"
    pytorch = "pytorch"


class QuantizeBackend(str, Enum):
    """``cuda`` (and ``None``) select the CUDA quantizer of this package; the other names exist
    so that reference configs parse, and are rejected when used."""
    cuda = "cuda"
    pytorch = "pytorch"
    transformer_engine = "transformer_engine"
    triton = "triton"


class RoundStyle(str, Enum):
    nearest = "nearest"
    stochastic = "stochastic"


class ScaleRule(str, Enum):
    abs_max = "abs_max"
    mae = "mae"
    mse = "mse"
    static_4 = "static_4"
    static_6 = "static_6"

    def cuda_id(self) -> int:
        return _RULE_IDS[self.value]

    def is_static(self) -> bool:
        return self.value.startswith("static")

    def max_allowed_e2m1_value(self) -> int:
        return 4 if self is ScaleRule.static_4 else 6

    def max_allowed_e4m3_value(self) -> int:
        return 448 if self.is_static() else 256


_RULE_IDS = {"static_6": 0, "static_4": 1, "mae": 2, "mse": 3, "abs_max": 4}
