"""NVFP4 ``Linear`` and model conversion with the reference's API
(fouroversix/src/fouroversix/model/modules/linear.py:153-355, model/quantize.py:13-127,
model/config.py:16-194): ``FourOverSixLinear`` quantizes its input, runs the W4A4 GEMM and adds
the bias - here in one fused epilogue - against a weight that was quantized once."""
from __future__ import annotations

import hashlib
import json
from dataclasses import dataclass, field
from typing import Any, Callable, ClassVar

import torch
import torch.nn as nn

from .enums import DataType, MatmulBackend, QuantizeBackend, RoundStyle, ScaleRule
from .matmul import fp4_matmul
from .quantize import QuantizationConfig, QuantizedTensor, quantize_to_fp4


def _enum(cls, v):
    return cls(v) if isinstance(v, str) else v


@dataclass
class ModuleQuantizationConfig:
    activation_scale_rule: ScaleRule | None = None
    dtype: DataType = DataType.nvfp4
    gradient_round_style: RoundStyle = RoundStyle.stochastic
    gradient_scale_rule: ScaleRule | None = None
    keep_master_weights: bool = False
    matmul_backend: MatmulBackend | None = None
    output_dtype: DataType = DataType.bfloat16
    quantize_backend: QuantizeBackend | None = None
    scale_rule: ScaleRule = ScaleRule.mse
    weight_scale_2d: bool = False
    weight_scale_rule: ScaleRule | None = None
    activation_chunk_size: int | None = None

    def __post_init__(self) -> None:
        for name, cls in (("activation_scale_rule", ScaleRule), ("dtype", DataType), ("gradient_round_style", RoundStyle),
                          ("gradient_scale_rule", ScaleRule), ("matmul_backend", MatmulBackend), ("output_dtype", DataType),
                          ("quantize_backend", QuantizeBackend), ("scale_rule", ScaleRule), ("weight_scale_rule", ScaleRule)):
            setattr(self, name, _enum(cls, getattr(self, name)))
        self.activation_scale_rule = self.activation_scale_rule or self.scale_rule
        self.gradient_scale_rule = self.gradient_scale_rule or self.scale_rule
        self.weight_scale_rule = self.weight_scale_rule or self.scale_rule

    def get_activation_config(self, **kw: Any) -> QuantizationConfig:
        return QuantizationConfig(backend=self.quantize_backend, dtype=self.dtype, scale_rule=self.activation_scale_rule, **kw)

    def get_gradient_config(self, **kw: Any) -> QuantizationConfig:
        return QuantizationConfig(backend=self.quantize_backend, dtype=self.dtype, round_style=self.gradient_round_style,
                                  scale_rule=self.gradient_scale_rule, **kw)

    def get_weight_config(self, **kw: Any) -> QuantizationConfig:
        return QuantizationConfig(backend=self.quantize_backend, block_scale_2d=self.weight_scale_2d, dtype=self.dtype,
                                  scale_rule=self.weight_scale_rule, **kw)


@dataclass
class ModelQuantizationConfig(ModuleQuantizationConfig):
    module_config_overrides: dict[str, ModuleQuantizationConfig] = field(default_factory=dict)
    modules_to_not_convert: list[str] = field(default_factory=lambda: ["lm_head"])

    def __post_init__(self) -> None:
        super().__post_init__()
        for name, cfg in list((self.module_config_overrides or {}).items()):
            if isinstance(cfg, dict):
                self.module_config_overrides[name] = ModuleQuantizationConfig(**cfg)

    def get_module_config(self, module_name: str) -> ModuleQuantizationConfig:
        return (self.module_config_overrides or {}).get(module_name, self)

    def __hash__(self):
        return hashlib.sha256(json.dumps(self.__dict__, sort_keys=True, default=str).encode()).hexdigest()


class QuantizedModule:
    """Registry high-precision module type -> quantized module type."""

    _registry: ClassVar[dict[type, type]] = {}
    _replace_in_model: ClassVar[dict[type, bool]] = {}

    @classmethod
    def is_quantized_module_type(cls, module_type: type) -> bool:
        return module_type in cls._registry.values()

    @classmethod
    def get_cls(cls, high_precision_cls: type):
        return cls._registry.get(high_precision_cls)

    @classmethod
    def should_replace_existing_modules_in_model(cls, module_type: type) -> bool:
        return cls._replace_in_model.get(module_type, False)

    @classmethod
    def register(cls, high_precision_cls: type, *, replace_existing_modules_in_registry: bool = False,
                 replace_existing_modules_in_model: bool = True) -> Callable[[type], type]:
        if high_precision_cls in cls._registry and not replace_existing_modules_in_registry:
            raise ValueError(f"High-precision module {high_precision_cls} is already registered.")
        for known in list(cls._registry):
            if issubclass(high_precision_cls, known) and known is not high_precision_cls:
                if not replace_existing_modules_in_registry:
                    raise TypeError(f"High-precision module {high_precision_cls} is a subclass of {known}, "
                                    "which is already registered.")
                del cls._registry[known]

        def deco(wrapped: type) -> type:
            cls._registry[high_precision_cls] = wrapped
            cls._replace_in_model[high_precision_cls] = replace_existing_modules_in_model
            return wrapped

        return deco


@QuantizedModule.register(nn.Linear)
class FourOverSixLinear(nn.Linear):
    """Drop-in ``nn.Linear`` whose forward is NVFP4 W4A4 (inference only)."""

    _BUFFERS = ("values", "scale_factors", "amax", "metadata")

    def __init__(self, module: nn.Linear, config: ModuleQuantizationConfig) -> None:
        super().__init__(module.in_features, module.out_features, module.bias is not None,
                         device="meta", dtype=module.weight.dtype)
        self.weight = module.weight
        self.bias = module.bias
        self.config = config
        if not config.keep_master_weights:
            dev = module.weight.device
            bs = config.dtype.block_size()
            self.register_buffer("quantized_weight_values",
                                 torch.zeros(self.out_features, self.in_features // 2, dtype=torch.uint8, device=dev))
            self.register_buffer("quantized_weight_scale_factors",
                                 torch.zeros(self.out_features * self.in_features // bs, dtype=config.dtype.scale_dtype(), device=dev))
            self.register_buffer("quantized_weight_amax", torch.zeros(1, dtype=torch.float32, device=dev))
            self.register_buffer("quantized_weight_metadata", torch.zeros(4, dtype=torch.int32, device=dev))

    @property
    def parameters_to_quantize(self) -> tuple[str, ...]:
        return ("weight",)

    def get_element_size(self, parameter_name: str) -> float:
        sizes = {"quantized_weight_values": 0.5, "weight": 9 / 16}
        if parameter_name in sizes:
            return sizes[parameter_name]
        return getattr(self, parameter_name).element_size()

    def get_quantized_parameters(self, parameter_name: str, parameter: torch.Tensor,
                                 include_transposed: bool = False) -> dict[str, Any]:
        if parameter_name != "weight":
            raise ValueError(f"Unsupported high-precision parameter: {parameter_name}")
        if include_transposed:
            raise ValueError("transposed weight copies (training) are not supported by the inference path")
        q = quantize_to_fp4(parameter, self.config.get_weight_config())
        return self._serialize_quantized_weight("quantized_weight", q)

    @staticmethod
    def _serialize_quantized_weight(prefix: str, q: QuantizedTensor) -> dict[str, torch.Tensor]:
        meta = torch.tensor([*q.original_shape, *q.padded_shape], dtype=torch.int32)
        return {f"{prefix}_values": q.values, f"{prefix}_scale_factors": q.scale_factors,
                f"{prefix}_amax": q.amax, f"{prefix}_metadata": meta}

    def materialize(self) -> None:
        """Quantize the master weight once, keep only the NVFP4 copy."""
        params = self.get_quantized_parameters("weight", self.weight.data)
        for key, value in params.items():
            setattr(self, key, value.to(self.weight.device))
        self.weight = None
        self.__dict__.pop("_quantized_weight", None)

    def _build_quantized_weight(self, prefix: str):
        parts = [getattr(self, f"{prefix}_{b}", None) for b in self._BUFFERS]
        if any(p is None for p in parts):
            return None
        values, sf, amax, meta = parts
        m = meta.tolist()
        return QuantizedTensor(values, sf, amax, self.config.dtype, tuple(m[:2]), self.config.weight_scale_rule, tuple(m[2:]))

    def quantized_weight(self):
        if "_quantized_weight" not in self.__dict__:
            if self.config.keep_master_weights:
                return self.weight
            self.__dict__["_quantized_weight"] = self._build_quantized_weight("quantized_weight")
        return self.__dict__["_quantized_weight"]

    def quantized_weight_transposed(self):
        return None

    def forward(self, input: torch.Tensor) -> torch.Tensor:
        w = self.quantized_weight()
        if not isinstance(w, QuantizedTensor):
            w = quantize_to_fp4(w.data, self.config.get_weight_config())
        x2d = input.reshape(-1, input.shape[-1])
        xq = quantize_to_fp4(x2d, self.config.get_activation_config())
        out = fp4_matmul(xq, w, backend=self.config.matmul_backend, out_dtype=self.config.output_dtype, bias=self.bias)
        return out.reshape(*input.shape[:-1], w.original_shape[0])


def quantize_model(model: nn.Module, config: ModelQuantizationConfig, **kwargs: Any) -> None:
    """Swap every registered module type (``nn.Linear``) for its NVFP4 counterpart, in place."""
    skip = set(config.modules_to_not_convert or [])
    for name, module in list(model.named_modules()):
        if not name or name in skip:
            continue
        qcls = QuantizedModule.get_cls(type(module))
        if qcls is None or not QuantizedModule.should_replace_existing_modules_in_model(type(module)):
            continue
        model.set_submodule(name, qcls(module, config.get_module_config(name), **kwargs))
