"""``quantize_to_fp4`` / ``QuantizedTensor`` / ``QuantizationConfig`` with the reference's
signatures (fouroversix/src/fouroversix/quantize/frontend.py:19-122, config.py:6-51,
quantized_tensor.py:56-248), backed by the sm_100a CUDA quantizer of this package.

There is exactly one implementation: ``backend`` may be ``None``, ``"cuda"`` (quantize) or
``"cutlass"`` (matmul); every other backend name and every option the CUDA quantizer of the
reference does not support either (MXFP4, RHT, stochastic rounding, 2-D scales, transpose)
raises ``ValueError`` exactly where the reference's frontend raises it
(frontend.py:114-120)."""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from . import ops
from .enums import DataType, QuantizeBackend, RoundStyle, ScaleRule


@dataclass
class QuantizationConfig:
    backend: QuantizeBackend | None = None
    block_scale_2d: bool = False
    dtype: DataType = DataType.nvfp4
    rht: bool = False
    round_style: RoundStyle = RoundStyle.nearest
    scale_rule: ScaleRule = ScaleRule.mse
    transpose: bool = False

    def __post_init__(self) -> None:
        if isinstance(self.backend, str):
            self.backend = QuantizeBackend(self.backend)
        if isinstance(self.dtype, str):
            self.dtype = DataType(self.dtype)
        if isinstance(self.round_style, str):
            self.round_style = RoundStyle(self.round_style)
        if isinstance(self.scale_rule, str):
            self.scale_rule = ScaleRule(self.scale_rule)


def sf_offsets(rows: int, cols: int, device) -> torch.Tensor:
    """Flat offset of scale (r, c) in the 128x4 swizzled layout, as an int64 [rows, cols] tensor."""
    r = torch.arange(rows, device=device).view(-1, 1)
    c = torch.arange(cols, device=device).view(1, -1)
    return ((r // 128) * (cols // 4) + c // 4) * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + c % 4


def to_blocked(sf2d: torch.Tensor) -> torch.Tensor:
    """[rows, cols] scale matrix -> flat swizzled array (fouroversix/src/fouroversix/quantize/utils.py:88-96)."""
    out = torch.empty(sf2d.numel(), dtype=sf2d.dtype, device=sf2d.device)
    off = sf_offsets(sf2d.shape[0], sf2d.shape[1], sf2d.device).reshape(-1)
    out.view(torch.uint8)[off] = sf2d.reshape(-1).view(torch.uint8)
    return out


def from_blocked(flat: torch.Tensor, shape: tuple[int, int]) -> torch.Tensor:
    """Inverse of :func:`to_blocked` (fouroversix/src/fouroversix/quantize/quantized_tensor.py:10-18)."""
    off = sf_offsets(shape[0], shape[1], flat.device)
    return flat.reshape(-1).view(torch.uint8)[off].view(flat.dtype)


class QuantizedTensor:
    """Packed E2M1 codes + swizzled block scales + fp32 tensor amax, padded to (128, 64) multiples."""

    def __init__(self, values, scale_factors, amax, dtype, original_shape, scale_rule, padded_shape=None):
        self.dtype = DataType(dtype) if isinstance(dtype, str) else dtype
        self.original_shape = tuple(original_shape)
        self.scale_rule = ScaleRule(scale_rule) if isinstance(scale_rule, str) else scale_rule
        if padded_shape is not None:
            self.padded_shape = tuple(padded_shape)
        else:
            rows, cols = self.original_shape
            bs = self.dtype.block_size()
            self.padded_shape = (rows + (-rows) % 128, cols + (-cols) % (4 * bs))
            n_codes = self.padded_shape[0] * self.padded_shape[1] // 2
            n_sf = 2 * n_codes // bs
            if values.numel() != n_codes:
                values = F.pad(values, (0, self.padded_shape[1] // 2 - values.shape[1],
                                        0, self.padded_shape[0] - values.shape[0]))
            if scale_factors.ndim > 1 and scale_factors.numel() != n_sf:
                sf_u8 = F.pad(scale_factors.view(torch.uint8),
                              (0, self.padded_shape[1] // bs - scale_factors.shape[1],
                               0, self.padded_shape[0] - scale_factors.shape[0]))
                scale_factors = to_blocked(sf_u8).view(scale_factors.dtype)
            if values.numel() != n_codes:
                raise ValueError(f"Expected {n_codes} e2m1 values, got {values.numel()}")
            if scale_factors.numel() != n_sf:
                raise ValueError(f"Expected {n_sf} scale factors, got {scale_factors.numel()}")
        self.values = values
        self.scale_factors = scale_factors
        self.amax = amax

    def dequantize(self, dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """High-precision copy, rounding as the reference's ``QuantizedTensor.dequantize``."""
        if self.dtype != DataType.nvfp4:
            raise ValueError("only NVFP4 tensors are supported")
        rows, cols = self.original_shape
        cols16 = cols + (-cols) % 16
        out = ops.dequantize_nvfp4(self.values, self.scale_factors, self.amax, rows, cols16, self.padded_shape[1], dtype,
                                   self.scale_rule.max_allowed_e2m1_value(), self.scale_rule.max_allowed_e4m3_value(),
                                   ops.DEQ_PYTORCH)
        return out if cols16 == cols else out[:, :cols]

    @property
    def device(self) -> torch.device:
        return self.values.device


def _supported(x: torch.Tensor, config: QuantizationConfig) -> bool:
    if x.ndim != 2 or config.dtype not in (DataType.mxfp4, DataType.nvfp4):
        return False
    if config.dtype == DataType.mxfp4 and not config.scale_rule.is_static():
        raise ValueError("MXFP4 quantization only supports the `static_6` and `static_4` scale rules")
    return (x.device.type == "cuda" and x.dtype in (torch.float16, torch.bfloat16)
            and config.round_style == RoundStyle.nearest and config.dtype == DataType.nvfp4
            and not config.transpose and not config.rht and not config.block_scale_2d)


def quantize_to_fp4(x: torch.Tensor, config: QuantizationConfig | None = None, *, amax: torch.Tensor | None = None,
                    out: QuantizedTensor | None = None) -> QuantizedTensor:
    """Quantize a 2-D bf16/fp16 CUDA tensor to NVFP4.

    Same call as the reference's ``quantize_to_fp4(x, config)``.  Two optional extras:
    ``amax`` supplies the fp32 tensor scale (skips the reduction pass; the reference's oracle
    accepts the same, reference.py:244), ``out`` writes into an existing ``QuantizedTensor``
    (persistent KV-cache slot) instead of allocating.
    """
    if config is None:
        config = QuantizationConfig()
    if config.backend not in (None, QuantizeBackend.cuda):
        raise ValueError(f"Backend {config.backend} does not support the given parameters")
    if not _supported(x, config):
        if config.backend is None:
            raise ValueError("No backend found that supports the given parameters")
        raise ValueError(f"Backend {config.backend} does not support the given parameters")
    # fp16 input, which the reference's CUDA backend takes beside bf16 (quantize/cuda/backend.py:45-51), goes through
    # llnv_quantize_nvfp4_f16: same result layout, the reference's fp32 arithmetic block by block (ops.quantize_nvfp4).
    rows, cols = x.shape
    if cols % 64 != 0:
        x = F.pad(x, (0, (-cols) % 64))
    if out is not None:
        if amax is not None:
            out.amax.copy_(amax.reshape(out.amax.shape))
        ops.quantize_nvfp4(x, config.scale_rule.cuda_id(), out.amax, out.values, out.scale_factors,
                           amax_given=amax is not None)
        return out
    codes, sf, amax_t = ops.quantize_nvfp4(x, config.scale_rule.cuda_id(), amax)
    return QuantizedTensor(codes, sf, amax_t, config.dtype, (rows, cols), config.scale_rule,
                           (codes.shape[0], codes.shape[1] * 2))
