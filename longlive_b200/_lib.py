"""ctypes binding of ``libllnvfp4.so``.  There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libllnvfp4.so")

# names declared in include/llnvfp4.h
EXPORTS = [
    "llnv_version", "llnv_last_error", "llnv_check_status", "llnv_amax_bf16", "llnv_quantize_nvfp4",
    "llnv_kv_dequant", "llnv_dequantize_nvfp4", "llnv_gemm_nvfp4", "llnv_gemm_nvfp4_grouped", "llnv_adaln_quantize_nvfp4",
    "llnv_layernorm_quantize_nvfp4", "llnv_gemm_nvfp4_ex", "llnv_attention_nvfp4kv", "llnv_init_device", "llnv_launch_count", "llnv_set_peer_poll_limit", "llnv_selftest_div_const", "llnv_fp4_mma_rate", "llnv_set_amax_accumulate", "llnv_quantize_nvfp4_f16", "llnv_quantize_nvfp4_group", "llnv_adaln_quantize_nvfp4_group", "llnv_layernorm_quantize_nvfp4_group",
    "llnv_adaln_quantize_nvfp4_static", "llnv_static_max_rows", "llnv_rmsnorm_rope", "llnv_attention_bf16", "llnv_attention_bf16_ex", "llnv_quantize_nvfp4_ex", "llnv_quantize_nvfp4_pair", "llnv_rmsnorm_rope_ex", "llnv_rmsnorm_rope_scatter", "llnv_rmsnorm_rope_qk", "llnv_scatter_2d", "llnv_peer_barrier", "llnv_peer_allreduce_max", "llnv_attention_key_splits", "llnv_attention_workspace_bytes", "llnv_adaln_quantize_nvfp4_ex", "llnv_layernorm_quantize_nvfp4_ex", "llnv_unipc_step", "llnv_set_pdl", "llnv_linear_bf16", "llnv_patchify", "llnv_unpatchify",
]


class Epilogue(C.Structure):
    """Mirror of ``llnv_epilogue_t``."""
    _fields_ = [
        ("alpha", C.c_void_p), ("bias", C.c_void_p), ("act", C.c_int32), ("residual", C.c_void_p),
        ("ldr", C.c_int64), ("gate", C.c_void_p), ("gate_stride", C.c_int64), ("frame_rows", C.c_int32),
        ("out_amax", C.c_void_p), ("row_offset", C.c_int32), ("q_codes", C.c_void_p), ("q_sf", C.c_void_p),
        ("q_amax", C.c_void_p), ("q_rule", C.c_int32),
    ]


class UniPCCoef(C.Structure):
    """Mirror of ``llnv_unipc_coef``."""
    _fields_ = [
        ("sigma", C.c_float), ("use_corrector", C.c_int32), ("corrector_order", C.c_int32), ("cc1", C.c_float), ("cc2", C.c_float),
        ("cc3", C.c_float), ("c_inv_rk", C.c_float), ("c_rho0", C.c_float), ("c_rho1", C.c_float), ("predictor_order", C.c_int32),
        ("pc1", C.c_float), ("pc2", C.c_float), ("pc3", C.c_float), ("p_inv_rk", C.c_float), ("p_zero", C.c_float),
    ]


class LibraryMissing(RuntimeError):
    pass


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise LibraryMissing(
                f"{LIB_PATH} is missing: build it with `python -m longlive_b200.build` "
                "(there is no CPU or PyTorch fallback for the NVFP4 kernels)")
        l = C.CDLL(LIB_PATH)
        l.llnv_last_error.restype = C.c_char_p
        p, i64, i32, f32 = C.c_void_p, C.c_int64, C.c_int, C.c_float
        l.llnv_check_status.argtypes = [p]
        l.llnv_amax_bf16.argtypes = [p, i64, i64, i64, p, p]
        l.llnv_quantize_nvfp4.argtypes = [p, i64, i64, i64, i32, p, p, p, i32, p]
        l.llnv_kv_dequant.argtypes = [p, p, p, i32, i32, i32, i32, f32, f32, i32, p, p]
        l.llnv_dequantize_nvfp4.argtypes = [p, p, p, i64, i64, i64, i32, f32, f32, i32, p, i64, p]
        l.llnv_gemm_nvfp4.argtypes = [p, p, p, i32, p, p, p, i32, i64, i64, i64, p, p, i64, p]
        l.llnv_adaln_quantize_nvfp4.argtypes = [p, i64, i64, i64, p, p, i64, i32, f32, i32, i32, p, p, p, p, i64, p, p]
        l.llnv_layernorm_quantize_nvfp4.argtypes = [p, i64, i64, i64, p, p, f32, i32, p, p, p, p, i64, p, p]
        l.llnv_fp4_mma_rate.argtypes = [i32, p, p]
        l.llnv_set_amax_accumulate.argtypes = [i32]
        l.llnv_quantize_nvfp4_f16.argtypes = [p, i64, i64, i64, i32, p, p, p, i32, p]
        l.llnv_quantize_nvfp4_group.argtypes = [p, i64, i64, i64, i32, p, p, p, i32, p, p, i32, i32, p, p]
        l.llnv_adaln_quantize_nvfp4_group.argtypes = [p, i64, i64, i64, p, p, i64, i32, f32, i32, i32, p, p, p, p, i64, p, p, i32, i32, p, p]
        l.llnv_layernorm_quantize_nvfp4_group.argtypes = [p, i64, i64, i64, p, p, f32, i32, p, p, p, p, p, p, i32, i32, p, p]
        l.llnv_gemm_nvfp4_ex.argtypes = [p, p, p, i32, p, p, p, i32, i64, i64, i64, p, p, i64, i32, p]
        l.llnv_selftest_div_const.argtypes = [i32, C.c_uint32, C.c_uint64, p, p]
        l.llnv_adaln_quantize_nvfp4_static.argtypes = [p, i64, i64, i64, p, p, i64, i32, f32, i32, i32, p, p, p, p, i64, p]
        l.llnv_static_max_rows.restype = C.c_int64
        l.llnv_attention_bf16.argtypes = [p, i64, i64, p, p, i64, i64, i64, i32, f32, p, i64, p]
        l.llnv_attention_bf16_ex.argtypes = [p, i64, i64, p, p, i64, i64, i64, i32, f32, p, i64, i32, p, i64, p, p]
        l.llnv_attention_nvfp4kv.argtypes = [p, i64, i64, p, p, p, p, p, p, i32, i32, f32, f32, p, p, i64, i64, i64, i32, f32, p, i64, i32, p,
                                             i64, p, p]
        l.llnv_attention_key_splits.argtypes = [i64, i64, i32]
        l.llnv_attention_workspace_bytes.argtypes = [i64, i32, i32]
        l.llnv_attention_workspace_bytes.restype = C.c_int64
        l.llnv_adaln_quantize_nvfp4_ex.argtypes = [p, i64, i64, i64, p, p, i64, i32, f32, i32, i32, p, p, p, p, i64, p, i64, i32, p]
        l.llnv_layernorm_quantize_nvfp4_ex.argtypes = [p, i64, i64, i64, p, p, f32, i32, p, p, p, p, i64, p, i32, p]
        l.llnv_rmsnorm_rope.argtypes = [p, i64, i64, i64, p, f32, p, p, p, i64, p, i64, p, p]
        l.llnv_rmsnorm_rope_ex.argtypes = [p, i64, i64, i64, p, f32, p, p, p, i64, p, i64, p, i32, p]
        l.llnv_quantize_nvfp4_ex.argtypes = [p, i64, i64, i64, i32, p, p, p, i32, i32, p]
        l.llnv_rmsnorm_rope_scatter.argtypes = [p, i64, i64, i64, p, f32, p, p, p, i64, p, i64, p, i32, p]
        l.llnv_quantize_nvfp4_pair.argtypes = [p, p, i64, i64, i64, i32, p, p, p, p, p, p, i32, p]
        l.llnv_gemm_nvfp4_grouped.argtypes = [p, p, p, i32, p, p, p, i32, i64, i64, i64, i32, p, p, p, p, p]
        l.llnv_rmsnorm_rope_qk.argtypes = [p, i64, p, p, i64, p, i64, p, p, i64, p, i64, p, i64, i64, f32, p, p, i32, p]
        l.llnv_scatter_2d.argtypes = [p, i64, i64, p, i64, i64, i64, i32, p]
        l.llnv_peer_barrier.argtypes = [p, i32, i32, p, p]
        l.llnv_peer_allreduce_max.argtypes = [p, i32, p, p, i32, i32, p, p]
        l.llnv_set_pdl.argtypes = [i32]
        l.llnv_set_peer_poll_limit.argtypes = [C.c_uint32]
        l.llnv_init_device.argtypes = []
        l.llnv_launch_count.argtypes = []
        l.llnv_launch_count.restype = C.c_uint64
        l.llnv_patchify.argtypes = [p, i64, i64, p, i64, i32, i32, i32, i32, p]
        l.llnv_unpatchify.argtypes = [p, i64, p, i64, i64, i32, i32, i32, i32, p]
        l.llnv_linear_bf16.argtypes = [p, i64, p, i64, p, i32, i64, i64, i64, p, i64, p]
        l.llnv_unipc_step.argtypes = [p, p, p, p, p, p, p, p, i64, i32, p, p]
        for name in EXPORTS:
            getattr(l, name)
        _lib = l
    return _lib


_ready_devices: set = set()


def init_device(index: int) -> None:
    """One-time library set-up on CUDA device ``index`` (``llnv_init_device``): done on the first use of a
    device from Python, so that the library never has to allocate inside a later stream capture."""
    if index in _ready_devices:
        return
    import torch
    with torch.cuda.device(index):
        check(lib().llnv_init_device())
    _ready_devices.add(index)


def check(rc: int, exc=RuntimeError) -> None:
    if rc != 0:
        msg = lib().llnv_last_error().decode("utf-8", "replace")
        if rc == -1:
            raise ValueError(msg) if exc is RuntimeError else exc(msg)
        raise exc(f"llnvfp4 error {rc}: {msg}")
