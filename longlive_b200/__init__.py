"""B200 (sm_100a) NVFP4 inference path for a LongLive-2.0-shaped causal DiT.

The public names are those of the reference's quantization API (``fouroversix`` package and
``utils/quant.py``), so its model and pipeline code can import them from here unchanged.
Everything computes through ``libllnvfp4.so`` (hand-written CUDA behind a C ABI); importing a
compute function without the built library raises.
"""
from .enums import DataType, MatmulBackend, QuantizeBackend, RoundStyle, ScaleRule
from .kv_cache import (LongLiveQuantizationConfig, clone_quantized_tensor, copy_quantized_into, dequantize_kv_cache,
                       k_smooth, quantize_model_with_filter, _materialize_quantized_weights_for_inference)
from .linear import (FourOverSixLinear, ModelQuantizationConfig, ModuleQuantizationConfig, QuantizedModule,
                     quantize_model)
from .matmul import fp4_matmul
from .quantize import QuantizationConfig, QuantizedTensor, from_blocked, quantize_to_fp4, to_blocked

__version__ = "0.1.0"

__all__ = [
    "DataType", "FourOverSixLinear", "LongLiveQuantizationConfig", "MatmulBackend", "ModelQuantizationConfig",
    "ModuleQuantizationConfig", "QuantizationConfig", "QuantizeBackend", "QuantizedModule", "QuantizedTensor",
    "RoundStyle", "ScaleRule", "clone_quantized_tensor", "copy_quantized_into", "dequantize_kv_cache", "fp4_matmul",
    "from_blocked", "k_smooth", "quantize_model", "quantize_model_with_filter", "quantize_to_fp4", "to_blocked",
]
