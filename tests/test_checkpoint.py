"""Checkpoint format helpers (host logic, no GPU): layouts the reference writes are unwrapped the
way utils/nvfp4_checkpoint.py does, and the key names follow the causal Wan model's module tree."""
import torch

from longlive_b200 import checkpoint as ck
from longlive_b200.dit import DiTConfig


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
