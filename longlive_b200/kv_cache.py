"""LongLive-side quantization glue with the reference's names (utils/quant.py:74-88, 585-798):
filtered model conversion, weight materialization, and the NVFP4 KV-cache helpers."""
from __future__ import annotations

import re
from copy import deepcopy
from dataclasses import dataclass

import torch
import torch.nn as nn

from . import ops
from .linear import FourOverSixLinear, ModelQuantizationConfig, quantize_model
from .quantize import QuantizationConfig, QuantizedTensor

QUANTIZATION_TYPE = {"weight": "weight", "activation": "activation", "kv": "kv"}

DEFAULT_GENERATOR_FILTERED_MODULES = [
    "text_embedding.0", "text_embedding.2", "patch_embedding", "time_projection.1", "time_embedding.0",
    "time_embedding.2", "head.head", "head.modulation", "re:.*norm_k$", "re:.*norm_q$", "re:.*norm1$",
    "re:.*norm2$", "re:.*norm3$",
]
FILTER_PROFILE_ALIASES = {"generator": "generator", "student": "generator", "real_score": "real_score",
                          "teacher": "real_score", "fake_score": "fake_score", "critic": "fake_score"}


@dataclass
class LongLiveQuantizationConfig(QuantizationConfig):
    type: str = "weight"

    def __post_init__(self) -> None:
        super().__post_init__()
        if not isinstance(self.type, str):
            raise TypeError("Quantization type must be a string.")
        if self.type not in QUANTIZATION_TYPE:
            raise ValueError(f"Unknown quantization type '{self.type}'. Expected one of: {', '.join(QUANTIZATION_TYPE)}.")


def _resolve_modules_to_not_convert(model: nn.Module, patterns) -> list[str]:
    if not patterns:
        return []
    exact, regexes = set(), []
    for pat in patterns:
        if not isinstance(pat, str):
            raise TypeError("Each filtered module pattern must be a string.")
        if pat.startswith("re:"):
            regexes.append(re.compile(pat[3:]))
        else:
            exact.add(pat)
    names = [n for n, _ in model.named_modules() if n and (n in exact or any(r.search(n) for r in regexes))]
    return sorted(set(names))


def _materialize_quantized_weights_for_inference(model: nn.Module, target_device=None, cache_transposed_weights: bool = False):
    """Quantize every NVFP4 Linear's master weight once and drop the bf16 copy.

    Returns (module names, master bytes, quantized bytes) like utils/quant.py:477-582.
    """
    if cache_transposed_weights:
        raise ValueError("transposed weight caches are a training feature and are not supported")
    names, master, quant = [], 0, 0
    for name, mod in model.named_modules():
        if not isinstance(mod, FourOverSixLinear) or mod.weight is None or mod.config.keep_master_weights:
            continue
        if target_device is not None and mod.weight.device != torch.device(target_device):
            mod.weight.data = mod.weight.data.to(target_device)
            if mod.bias is not None:
                mod.bias.data = mod.bias.data.to(target_device)
        master += mod.weight.numel() * mod.weight.element_size()
        mod.materialize()
        quant += mod.quantized_weight_values.numel() + mod.quantized_weight_scale_factors.numel() + 4
        names.append(name)
    return names, master, quant


def quantize_model_with_filter(model: nn.Module, quant_config=None, filtered_modules=None, filter_profile=None,
                               use_default_filtered_modules: bool = False, cast_model_to_bf16: bool = True,
                               materialize_for_inference: bool = False, materialize_target_device=None,
                               use_transformer_engine: bool = False, te_inference_only: bool = False,
                               te_low_precision_weights=None, te_recipe_kwargs=None, te_module_kwargs=None,
                               te_fallback_to_fouroversix: bool = False, verbose: bool = True, **kwargs):
    """Convert a model's Linear layers to NVFP4, skipping names / ``re:`` patterns (utils/quant.py:585-689).
    The ``te_*`` parameters belong to the reference's TransformerEngine path and are accepted for call
    compatibility; asking for that path (``use_transformer_engine=True``) raises."""
    if use_transformer_engine:
        raise ValueError("the TransformerEngine linear path is not part of this package")
    if quant_config is None:
        cfg = ModelQuantizationConfig()
    elif isinstance(quant_config, dict):
        cfg = ModelQuantizationConfig(**quant_config)
    elif isinstance(quant_config, ModelQuantizationConfig):
        cfg = deepcopy(quant_config)
    else:
        raise TypeError("quant_config must be ModelQuantizationConfig, dict, or None.")
    patterns = list(filtered_modules or [])
    if use_default_filtered_modules:
        patterns = list(DEFAULT_GENERATOR_FILTERED_MODULES) + patterns
    matched = _resolve_modules_to_not_convert(model, patterns)
    cfg.modules_to_not_convert = sorted(set(cfg.modules_to_not_convert or []) | set(matched))
    if cast_model_to_bf16:
        model.to(torch.bfloat16)
    quantize_model(model, cfg)
    if materialize_for_inference:
        names, master, quant = _materialize_quantized_weights_for_inference(model, materialize_target_device)
        if verbose:
            print(f"[quantize_model_with_filter] materialized_modules={len(names)}, "
                  f"master_weight={master / 2**30:.3f} GiB, quantized_weight={quant / 2**30:.3f} GiB")
    if verbose:
        print(f"[quantize_model_with_filter] profile={filter_profile or 'default'}, matched={len(matched)}, "
              f"total_excluded={len(cfg.modules_to_not_convert)}")
    return model, matched


def dequantize_kv_cache(kv_list, max_blocks, num_heads, block_token_size, dtype, device, out=None):
    """``max_blocks`` QuantizedTensors [T*H, 128] -> [1, max_blocks*T, H, 128] in one launch.

    Same signature and rounding as the fused path of utils/quant.py:731-768."""
    blocks = kv_list[:max_blocks]
    rule = blocks[0].scale_rule
    return ops.kv_dequant([b.values for b in blocks], [b.scale_factors for b in blocks], [b.amax for b in blocks],
                          num_heads, block_token_size, dtype, rule.max_allowed_e2m1_value(),
                          rule.max_allowed_e4m3_value(), ops.DEQ_FUSED, out)


def clone_quantized_tensor(qt: QuantizedTensor) -> QuantizedTensor:
    return QuantizedTensor(qt.values.clone(), qt.scale_factors.clone(), qt.amax.clone() if qt.amax is not None else None,
                           qt.dtype, qt.original_shape, qt.scale_rule, qt.padded_shape)


def copy_quantized_into(slot: QuantizedTensor, src: QuantizedTensor) -> None:
    """Copy into a persistent slot without changing the slot's buffer addresses (utils/quant.py:783-794)."""
    slot.values.copy_(src.values)
    slot.scale_factors.copy_(src.scale_factors)
    if src.amax is not None and slot.amax is not None:
        slot.amax.copy_(src.amax.reshape(slot.amax.shape))


def k_smooth(k: torch.Tensor) -> torch.Tensor:
    """``k - mean(k, -1)`` (utils/quant.py:797-798)."""
    return k - k.mean(dim=-1, keepdim=True)
