"""Checkpoint format helpers (host logic, no GPU): layouts the reference writes are unwrapped the
way utils/nvfp4_checkpoint.py does, and the key names follow the causal Wan model's module tree."""
import os

import numpy as np
import torch

from longlive_b200 import checkpoint as ck
from longlive_b200.dit import DiTConfig
from oracle import nvfp4_oracle as O

FIXTURE = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "nvfp4_state_dict.pt")


def test_state_dict_written_by_the_reference_exporter():
    """``tests/golden/nvfp4_state_dict.pt`` holds the entries the reference's FourOverSixLinear.get_quantized_parameters
    (fouroversix/src/fouroversix/model/modules/linear.py:233-289) wrote for two Linears, in the exporter's outer layout,
    plus their bf16 master weights.  The file loads with weights_only=True, is recognised, carries the key names and
    the metadata layout this package reads, and its codes, scales and amax are what the oracle's quantizer gives for
    the master weights, bit for bit."""
    ckpt = torch.load(FIXTURE, map_location="cpu", weights_only=True)
    assert ckpt["checkpoint_format"] == ck.NVFP4_CHECKPOINT_FORMAT and ckpt["checkpoint_version"] == ck.NVFP4_CHECKPOINT_VERSION
    sd = ck.unwrap_generator_state_dict(ckpt)
    assert ck.is_nvfp4_state_dict(sd)
    assert ckpt["quantization"]["scale_rule"] == "mse"
    wanted = {k[len("model."):] for k in ck.expected_keys(DiTConfig(layers=1))}
    assert set(sd) <= wanted, set(sd) - wanted
    for name, (o, i) in {"blocks.0.self_attn.q": (256, 256), "blocks.0.ffn.0": (512, 256)}.items():
        meta = sd[f"{name}.quantized_weight_metadata"]
        assert meta.dtype == torch.int32 and meta.tolist() == [o, i, o, i]          # original rows, cols, padded rows, cols
        codes, sf, amax = O.quantize_nvfp4(ckpt["masters"][f"{name}.weight"].float().numpy(), "mse")
        assert np.array_equal(sd[f"{name}.quantized_weight_values"].numpy(), codes)
        assert np.array_equal(sd[f"{name}.quantized_weight_scale_factors"].view(torch.uint8).numpy(), sf)
        assert np.float32(sd[f"{name}.quantized_weight_amax"].item()) == amax
        assert sd[f"{name}.bias"].dtype == torch.bfloat16 and sd[f"{name}.bias"].numel() == o


def test_unwrap_and_detect():
    sd = {"model.blocks.0.self_attn.q.quantized_weight_values": torch.zeros(1, dtype=torch.uint8)}
    assert ck.is_nvfp4_state_dict(sd) and not ck.is_nvfp4_state_dict({"model.blocks.0.self_attn.q.weight": 1})
    assert not ck.is_nvfp4_state_dict([1, 2])
    assert ck.unwrap_generator_state_dict({"generator": sd, "generator_ema": {"e": 1}}) is sd
    assert ck.unwrap_generator_state_dict({"generator": sd, "generator_ema": {"e": 1}}, use_ema=True) == {"e": 1}
    assert ck.unwrap_generator_state_dict({"generator": sd}, use_ema=True) is sd
    assert ck.unwrap_generator_state_dict({"model": sd}) is sd
    assert ck.unwrap_generator_state_dict(sd) is sd
    assert ck.unwrap_generator_state_dict(7) == 7
    assert ck.clean_fsdp_state_dict_keys({"model._fsdp_wrapped_module.blocks.0.modulation": 3}) == {"model.blocks.0.modulation": 3}


def test_expected_keys_follow_the_reference_module_tree():
    cfg = DiTConfig(layers=2)
    keys = ck.expected_keys(cfg)
    assert len(keys) == len(set(keys))
    for k in ("model.blocks.1.self_attn.q.quantized_weight_values", "model.blocks.0.cross_attn.o.quantized_weight_metadata",
              "model.blocks.1.ffn.2.bias", "model.blocks.0.self_attn.norm_k.weight", "model.blocks.0.norm3.bias",
              "model.blocks.1.modulation", "model.patch_embedding.weight", "model.time_projection.1.weight",
              "model.text_embedding.2.bias", "model.head.head.weight", "model.head.modulation"):
        assert k in keys, k
    per_block = 10 * 5 + 7
    assert len(keys) == 2 * per_block + 3 + 6 * 2
    bf16 = ck.expected_keys(cfg, quantized=False)
    assert "model.blocks.0.ffn.0.weight" in bf16 and not any("quantized_weight" in k for k in bf16)


def test_head_row_order_folds_unpatchify_and_patchify():
    """A head with permuted rows emits, per token, what the reference's head + unpatchify + patchify
    (Conv3d feature order) would: (kh, kw, channel) -> [C, F, H, W] -> (channel, kh, kw)."""
    C, f, h, w = 5, 2, 3, 4
    g = torch.Generator().manual_seed(0)
    u = torch.randn(f * h * w, 4 * C, generator=g)                        # reference head output, features (kh, kw, c)
    lat = torch.einsum("fhwpqrc->cfphqwr", u.view(f, h, w, 1, 2, 2, C)).reshape(C, f, 2 * h, 2 * w)   # unpatchify
    # patchify as the Conv3d with kernel (1, 2, 2) sees it: token (f, hh, ww), features (c, kh, kw)
    tok = lat.view(C, f, h, 2, w, 2).permute(1, 2, 4, 0, 3, 5).reshape(f * h * w, 4 * C)
    assert torch.equal(u[:, ck.head_row_order(C)], tok)
    inv = torch.argsort(ck.head_row_order(C))
    assert torch.equal(tok[:, inv], u)
