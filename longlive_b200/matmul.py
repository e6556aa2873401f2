"""``fp4_matmul`` with the reference's signature (fouroversix/src/fouroversix/matmul/frontend.py:14-115)
on the tcgen05 block-scaled GEMM of this package."""
from __future__ import annotations

import torch

from . import ops
from .enums import DataType, MatmulBackend
from .quantize import QuantizationConfig, QuantizedTensor, quantize_to_fp4


def fp4_matmul(input, other, *, backend: MatmulBackend | None = None, input_config: QuantizationConfig | None = None,
               other_config: QuantizationConfig | None = None, out_dtype: DataType = DataType.bfloat16,
               bias: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """``input @ other.T`` for NVFP4 operands (high-precision operands are quantized first).

    ``bias`` / ``out`` are extensions: the bias add of the Linear layer is fused into the GEMM
    epilogue with the same bf16 rounding points.
    """
    if isinstance(backend, str):
        backend = MatmulBackend(backend)
    if isinstance(out_dtype, str):
        out_dtype = DataType(out_dtype)
    if isinstance(input, torch.Tensor):
        input = quantize_to_fp4(input, input_config or QuantizationConfig())
    if isinstance(other, torch.Tensor):
        other = quantize_to_fp4(other, other_config or QuantizationConfig())
    if input.dtype != other.dtype:
        raise ValueError("Both inputs must have the same dtype")
    if input.original_shape[1] != other.original_shape[1]:
        raise ValueError("The first input must be in row-major layout, the second input must be in column-major "
                         "layout, and both inputs must have the same inner dimension")
    if backend not in (None, MatmulBackend.cutlass) or input.device.type != "cuda":
        raise ValueError(f"Backend {backend} does not support the given parameters")
    if input.dtype != DataType.nvfp4 or out_dtype != DataType.bfloat16:
        raise ValueError(f"No gemm function found for dtype {input.dtype} and out_dtype {out_dtype}")
    m, n = input.original_shape[0], other.original_shape[0]
    k = input.padded_shape[1]
    if other.padded_shape[1] != k:
        raise ValueError("operands are padded to different inner dimensions")
    n_pad = other.padded_shape[0]
    if k % 256 != 0:
        raise ValueError(f"inner dimension must be a multiple of 256 after padding, got {k}")
    res = ops.gemm_nvfp4(input.values, input.scale_factors, input.amax, input.scale_rule.cuda_id(),
                         other.values, other.scale_factors, other.amax, other.scale_rule.cuda_id(),
                         m, n_pad, k, bias=_pad_bias(bias, n_pad), out=out if n_pad == n else None)
    return res if n_pad == n else res[:, :n]


def _pad_bias(bias, n_pad):
    if bias is None or bias.numel() == n_pad:
        return bias
    return torch.nn.functional.pad(bias, (0, n_pad - bias.numel()))
