"""The three operator seams of the hot path as ``torch.library`` custom ops with fake (meta) implementations.

The reference's model may run under ``torch.compile``, so its extension registers its kernels as custom ops
with fake implementations (fouroversix/src/fouroversix/quantize/cuda/ops.py:4-46,
fouroversix/src/fouroversix/matmul/cutlass/ops.py:66-92, utils/kernel/kv_dequant.py:53-82 with the schema of
utils/kernel/kv_dequant.cpp:14).  The ops below take and return what those ops take and return and call the
C-ABI kernels of this package, so a traced graph contains one opaque node per kernel instead of a graph break:

    torch.ops.llnvfp4.quantize_to_fp4(x, is_nvfp4, is_rtn, is_rht, is_2d, is_transpose, selection_rule, rbits)
        -> (values uint8 [Mp, K/2], scale_factors e4m3 [Mp*K/16] swizzled, amax f32 [1])
    torch.ops.llnvfp4.gemm_nvfp4nvfp4_accum_fp32_out_bf16_tnt(a, b, a_sf, b_sf, alpha) -> bf16 [Mp, N]
    torch.ops.llnvfp4.dequantize_kv_cache_fp4(values[], scale_factors[], amax[], num_heads, block_token_size,
                                              dtype_code, e2m1_max, e4m3_max) -> [1, blocks*T, H, 128]

``install_reference_aliases()`` additionally defines the reference's own op names
(``fouroversix::...``, ``longlive_kernels::...``) on top of the same functions, for a process in which the
reference's extension is not loaded; it refuses to shadow ops that already exist.
"""
from __future__ import annotations

import torch

from . import ops

_DTYPES = {0: torch.bfloat16, 1: torch.float16, 2: torch.float32}


def _padded(m: int) -> int:
    return (m + 127) // 128 * 128


@torch.library.custom_op("llnvfp4::quantize_to_fp4", mutates_args=())
def quantize_to_fp4(x: torch.Tensor, is_nvfp4: bool, is_rtn: bool, is_rht: bool, is_2d: bool, is_transpose: bool,
                    selection_rule: int, rbits: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    if not is_nvfp4 or not is_rtn or is_rht or is_2d or is_transpose:
        raise RuntimeError("llnvfp4::quantize_to_fp4 supports NVFP4 with round-to-nearest, 1-D block scales, no RHT, no transpose")
    if x.dim() != 2 or x.dtype not in (torch.bfloat16, torch.float16) or x.shape[1] % 64 != 0:
        raise RuntimeError("llnvfp4::quantize_to_fp4 expects a 2-D bfloat16 or float16 tensor whose column count is a multiple of 64")
    codes, sf, amax = ops.quantize_nvfp4(x.contiguous(), int(selection_rule))
    return codes, sf, amax


@quantize_to_fp4.register_fake
def _(x, is_nvfp4, is_rtn, is_rht, is_2d, is_transpose, selection_rule, rbits):
    mp = _padded(x.shape[0])
    return (torch.empty(mp, x.shape[1] // 2, dtype=torch.uint8, device=x.device),
            torch.empty(mp * x.shape[1] // 16, dtype=torch.float8_e4m3fn, device=x.device),
            torch.empty(1, dtype=torch.float32, device=x.device))


@torch.library.custom_op("llnvfp4::gemm_nvfp4nvfp4_accum_fp32_out_bf16_tnt", mutates_args=())
def gemm_nvfp4nvfp4_accum_fp32_out_bf16_tnt(a: torch.Tensor, b: torch.Tensor, a_sf: torch.Tensor, b_sf: torch.Tensor,
                                            alpha: torch.Tensor) -> torch.Tensor:
    m, n, k = a.shape[0], b.shape[0], a.shape[1] * 2
    if a.dtype != torch.uint8 or b.dtype != torch.uint8 or b.shape[1] * 2 != k or alpha.dtype != torch.float32:
        raise RuntimeError("llnvfp4::gemm expects uint8 code matrices [M, K/2], [N, K/2] and a float32 alpha")
    return ops.gemm_nvfp4(a, a_sf, None, 3, b, b_sf, None, 3, m, n, k, alpha=alpha.reshape(-1))


@gemm_nvfp4nvfp4_accum_fp32_out_bf16_tnt.register_fake
def _(a, b, a_sf, b_sf, alpha):
    return torch.empty(a.shape[0], b.shape[0], dtype=torch.bfloat16, device=a.device)


@torch.library.custom_op("llnvfp4::dequantize_kv_cache_fp4", mutates_args=())
def dequantize_kv_cache_fp4(values: list[torch.Tensor], scale_factors: list[torch.Tensor], amax: list[torch.Tensor],
                            num_heads: int, block_token_size: int, dtype_code: int, e2m1_max: float,
                            e4m3_max: float) -> torch.Tensor:
    if dtype_code not in _DTYPES:
        raise RuntimeError(f"Unsupported fused KV dequant dtype code: {dtype_code}")
    return ops.kv_dequant(list(values), list(scale_factors), list(amax), num_heads, block_token_size, _DTYPES[dtype_code],
                          e2m1_max, e4m3_max, ops.DEQ_FUSED)


@dequantize_kv_cache_fp4.register_fake
def _(values, scale_factors, amax, num_heads, block_token_size, dtype_code, e2m1_max, e4m3_max):
    return torch.empty(1, len(values) * block_token_size, num_heads, 128, dtype=_DTYPES[dtype_code], device=values[0].device)


_ALIASES = (
    ("fouroversix", "quantize_to_fp4",
     "(Tensor x, bool is_nvfp4, bool is_rtn, bool is_rht, bool is_2d, bool is_transpose, int selection_rule, int rbits) -> (Tensor, Tensor, Tensor)",
     quantize_to_fp4),
    ("fouroversix", "gemm_nvfp4nvfp4_accum_fp32_out_bf16_tnt", "(Tensor A, Tensor B, Tensor A_sf, Tensor B_sf, Tensor alpha) -> Tensor",
     gemm_nvfp4nvfp4_accum_fp32_out_bf16_tnt),
    ("longlive_kernels", "dequantize_kv_cache_fp4",
     "(Tensor[] values, Tensor[] scale_factors, Tensor[] amax, int num_heads, int block_token_size, int dtype_code, float e2m1_max, float e4m3_max) -> Tensor",
     dequantize_kv_cache_fp4),
)
_alias_libs: list = []


def install_reference_aliases() -> list[str]:
    """Define the reference's op names on top of this package's kernels.  Returns the qualified names installed;
    an op that already exists (the reference's own extension is loaded) is left alone."""
    done = []
    for ns, name, schema, fn in _ALIASES:
        if hasattr(getattr(torch.ops, ns), name):
            continue
        lib = torch.library.Library(ns, "FRAGMENT")
        lib.define(name + schema)
        lib.impl(name, fn._opoverload, "CompositeExplicitAutograd")
        _alias_libs.append(lib)
        done.append(f"{ns}::{name}")
    return done
