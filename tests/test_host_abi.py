"""CPU-only checks: the C-ABI library builds, loads and exports every declared symbol; the host
side of the Python API validates arguments like the reference's frontend."""
import ctypes
import os
import re

import pytest
import torch

import longlive_b200 as L
from longlive_b200 import _lib, build

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def libpath():
    return build.build()


def test_library_exports_every_declared_symbol(libpath):
    header = open(os.path.join(ROOT, "include", "llnvfp4.h")).read()
    declared = set(re.findall(r"\b(llnv_[a-z0-9_]+)\s*\(", header))
    declared.discard("llnv_epilogue_t")
    assert declared, "no declarations found"
    lib = ctypes.CDLL(libpath)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} declared in include/llnvfp4.h but not exported"
    assert set(_lib.EXPORTS) <= declared
    assert lib.llnv_version() >= 1


def test_loader_has_no_fallback(monkeypatch, tmp_path):
    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "missing.so"))
    with pytest.raises(_lib.LibraryMissing):
        _lib.lib()


def test_enums_and_config_match_reference_values():
    assert [L.ScaleRule(r).cuda_id() for r in ("static_6", "static_4", "mae", "mse", "abs_max")] == [0, 1, 2, 3, 4]
    assert L.ScaleRule.mse.max_allowed_e4m3_value() == 256 and L.ScaleRule.static_6.max_allowed_e4m3_value() == 448
    assert L.ScaleRule.static_4.max_allowed_e2m1_value() == 4
    cfg = L.QuantizationConfig(backend="cuda", scale_rule="abs_max")
    assert cfg.backend is L.QuantizeBackend.cuda and cfg.scale_rule is L.ScaleRule.abs_max
    assert L.DataType.nvfp4.block_size() == 16 and L.DataType.nvfp4.scale_dtype() == torch.float8_e4m3fn
    kv = L.LongLiveQuantizationConfig(scale_rule="mse", backend="cuda", type="kv")
    assert kv.type == "kv"
    with pytest.raises(ValueError):
        L.LongLiveQuantizationConfig(type="nope")


def test_quantize_rejects_unsupported_requests():
    x = torch.zeros(128, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError):                       # CPU tensor: no backend supports it
        L.quantize_to_fp4(x)
    with pytest.raises(ValueError):
        L.quantize_to_fp4(x, L.QuantizationConfig(backend="pytorch"))
    with pytest.raises(ValueError):
        L.quantize_to_fp4(x, L.QuantizationConfig(dtype="mxfp4", scale_rule="mse"))


def test_swizzle_roundtrip_matches_oracle():
    import numpy as np
    from oracle import nvfp4_oracle as O
    sf = torch.arange(256 * 8, dtype=torch.int32).remainder(251).to(torch.uint8).reshape(256, 8)
    flat = L.to_blocked(sf)
    assert np.array_equal(flat.numpy(), O.to_blocked(sf.numpy()))
    assert torch.equal(L.from_blocked(flat, (256, 8)), sf)


def test_quantize_model_filter_and_registry():
    import torch.nn as nn

    class Blk(nn.Module):
        def __init__(self):
            super().__init__()
            self.q = nn.Linear(64, 64)
            self.norm1 = nn.LayerNorm(64)
            self.head = nn.Sequential(nn.Linear(64, 64))

    m = nn.ModuleDict({"blocks": nn.ModuleList([Blk(), Blk()])})
    model, matched = L.quantize_model_with_filter(m, {"scale_rule": "mse"}, filtered_modules=["re:.*head\\.0$"],
                                                  use_default_filtered_modules=True, verbose=False)
    assert matched == ["blocks.0.head.0", "blocks.0.norm1", "blocks.1.head.0", "blocks.1.norm1"]
    assert isinstance(model["blocks"][0].q, L.FourOverSixLinear)
    assert type(model["blocks"][0].head[0]) is nn.Linear
    assert model["blocks"][0].q.weight.dtype == torch.bfloat16
    assert model["blocks"][0].q.quantized_weight_values.shape == (64, 32)
    with pytest.raises(ValueError):
        L.QuantizedModule.register(nn.Linear)(object)


def test_documented_python_seam_names_exist():
    """Every name the integration notes rebind on the reference's utils.quant (and the scheduler class) is importable from
    this package, so the documented aliasing snippet cannot rot."""
    import longlive_b200
    import longlive_b200.kv_cache
    import longlive_b200.scheduler
    for name in ("quantize_to_fp4", "dequantize_kv_cache", "copy_quantized_into", "clone_quantized_tensor", "k_smooth",
                 "quantize_model_with_filter", "_materialize_quantized_weights_for_inference", "LongLiveQuantizationConfig"):
        obj = getattr(longlive_b200, name, None) or getattr(longlive_b200.kv_cache, name, None)
        assert obj is not None, name
    for name in ("DataType", "ModelQuantizationConfig", "QuantizationConfig", "QuantizedTensor", "RoundStyle", "ScaleRule",
                 "quantize_model", "quantize_to_fp4", "fp4_matmul", "FourOverSixLinear"):
        assert hasattr(longlive_b200, name), name
    sched = longlive_b200.scheduler.FlowUniPCMultistepScheduler
    assert all(hasattr(sched, m) for m in ("set_timesteps", "step"))
