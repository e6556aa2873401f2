"""Reading and writing generator checkpoints in the reference's NVFP4 format.

The reference stores a generator whose Linear layers were replaced by its NVFP4 module as a
``torch.save``d mapping ``{"generator": state_dict, "checkpoint_format":
"longlive_generator_nvfp4", "checkpoint_version": 1, ...}`` (scripts/save_merged_nvfp4_generator.py:
98-135, 226-236; utils/nvfp4_checkpoint.py:18-47).  Every quantized Linear contributes the buffers
``<name>.quantized_weight_values`` (uint8 codes [N_pad, K/2]), ``..._scale_factors`` (e4m3, 128x4
swizzled), ``..._amax`` (fp32 [1]) and ``..._metadata`` (int32: original rows, cols, padded rows,
cols) plus ``<name>.bias`` (fouroversix/src/fouroversix/model/modules/linear.py:270-307); layers
that were left in bf16 keep ``<name>.weight``.  Module names are those of the causal Wan model
(wan_5b/modules/causal_model.py:320-325, 816-827, 945-948, 1052-1071), under the ``model.`` prefix
of the generator wrapper.

``state_dict_of`` / ``load_state_dict_into`` map those names onto the tensors of
``longlive_b200.dit.CausalDiT``; a block Linear found as bf16 ``weight`` is quantized on load (the
same thing the reference's ``quantize_model_with_filter`` does after loading a bf16 checkpoint).
The patch embedding is stored as the Conv3d weight [dim, C_in, 1, 2, 2]; flattened it is the
[dim, C_in * 4] matrix applied to tokens whose features are ordered (channel, kh, kw).
The reference's head emits the features of a token in the order (kh, kw, channel), which its
``unpatchify`` turns back into a latent (wan_5b/modules/causal_model.py:1851-1857); the model here
keeps latents patchified between the forwards of a chunk, so the rows of ``head.head`` are
permuted on load into the input order (channel, kh, kw) -- the head then writes the flow
prediction in the layout of its input and the scheduler step needs no unpatchify / patchify pair --
and permuted back on save.
"""
from __future__ import annotations

from collections.abc import Mapping

import torch

from .enums import ScaleRule
from .quantize import QuantizationConfig, QuantizedTensor, quantize_to_fp4

NVFP4_CHECKPOINT_FORMAT = "longlive_generator_nvfp4"
NVFP4_CHECKPOINT_VERSION = 1

# (attribute of dit.Block, module path inside a reference block)
BLOCK_LINEARS = (("q", "self_attn.q"), ("k", "self_attn.k"), ("v", "self_attn.v"), ("o", "self_attn.o"),
                 ("cq", "cross_attn.q"), ("ck", "cross_attn.k"), ("cv", "cross_attn.v"), ("co", "cross_attn.o"),
                 ("ffn0", "ffn.0"), ("ffn2", "ffn.2"))
BLOCK_VECTORS = (("norm_q", "self_attn.norm_q.weight"), ("norm_k", "self_attn.norm_k.weight"),
                 ("cnorm_q", "cross_attn.norm_q.weight"), ("cnorm_k", "cross_attn.norm_k.weight"),
                 ("norm3_w", "norm3.weight"), ("norm3_b", "norm3.bias"), ("modulation", "modulation"))
# (weight attribute, bias attribute of dit.CausalDiT, module path); these stay bf16 in the reference too
EDGE_LINEARS = (("time_w0", "time_b0", "time_embedding.0"), ("time_w1", "time_b1", "time_embedding.2"),
                ("tproj_w", "tproj_b", "time_projection.1"), ("text_w0", "text_b0", "text_embedding.0"),
                ("text_w1", "text_b1", "text_embedding.2"), ("head_w", "head_b", "head.head"))


def head_row_order(in_channels: int, patch: int = 4) -> torch.Tensor:
    """Index array p with ``w_model = w_reference[p]``: model row c * patch + k is the reference's row k * C + c."""
    return torch.arange(patch * in_channels).view(patch, in_channels).t().reshape(-1)


def is_nvfp4_state_dict(state_dict: object) -> bool:
    """True when the mapping holds materialized NVFP4 weight buffers (utils/nvfp4_checkpoint.py:23-27)."""
    return isinstance(state_dict, Mapping) and any(str(k).endswith("quantized_weight_values") for k in state_dict)


def unwrap_generator_state_dict(checkpoint: object, use_ema: bool = False) -> object:
    """The generator's state dict out of the checkpoint layouts the reference writes
    (utils/nvfp4_checkpoint.py:38-47): ``generator`` / ``generator_ema``, ``model``, or the mapping itself."""
    if not isinstance(checkpoint, Mapping):
        return checkpoint
    if "generator" in checkpoint or "generator_ema" in checkpoint:
        return checkpoint["generator_ema" if use_ema and "generator_ema" in checkpoint else "generator"]
    return checkpoint.get("model", checkpoint)


def clean_fsdp_state_dict_keys(state_dict: Mapping) -> dict:
    """Strip the FSDP wrapper infix some EMA checkpoints carry (utils/nvfp4_checkpoint.py:50-52)."""
    return {str(k).replace("_fsdp_wrapped_module.", ""): v for k, v in state_dict.items()}


def _serialize(prefix: str, q: QuantizedTensor) -> dict:
    return {f"{prefix}.quantized_weight_values": q.values, f"{prefix}.quantized_weight_scale_factors": q.scale_factors,
            f"{prefix}.quantized_weight_amax": q.amax,
            f"{prefix}.quantized_weight_metadata": torch.tensor([*q.original_shape, *q.padded_shape], dtype=torch.int32)}


def expected_keys(cfg, prefix: str = "model.", quantized: bool = True) -> list[str]:
    """Every key ``state_dict_of`` writes for a model of configuration ``cfg``."""
    keys = []
    for i in range(cfg.layers):
        for _, path in BLOCK_LINEARS:
            base = f"{prefix}blocks.{i}.{path}"
            keys += ([f"{base}.quantized_weight_{s}" for s in ("values", "scale_factors", "amax", "metadata")] if quantized
                     else [f"{base}.weight"]) + [f"{base}.bias"]
        keys += [f"{prefix}blocks.{i}.{path}" for _, path in BLOCK_VECTORS]
    keys += [f"{prefix}patch_embedding.weight", f"{prefix}patch_embedding.bias", f"{prefix}head.modulation"]
    for _, _, path in EDGE_LINEARS:
        keys += [f"{prefix}{path}.weight", f"{prefix}{path}.bias"]
    return keys


def state_dict_of(model, prefix: str = "model.") -> dict:
    """The model's tensors under the reference's names (NVFP4 buffers for the block Linears)."""
    cfg, sd = model.cfg, {}
    for i, blk in enumerate(model.blocks):
        for attr, path in BLOCK_LINEARS:
            lin = getattr(blk, attr)
            sd.update(_serialize(f"{prefix}blocks.{i}.{path}", lin.q))
            sd[f"{prefix}blocks.{i}.{path}.bias"] = lin.bias
        for attr, path in BLOCK_VECTORS:
            sd[f"{prefix}blocks.{i}.{path}"] = getattr(blk, attr)
    sd[f"{prefix}patch_embedding.weight"] = model.patch_w.view(cfg.dim, cfg.in_channels, 1, 2, 2)
    sd[f"{prefix}patch_embedding.bias"] = model.patch_b
    sd[f"{prefix}head.modulation"] = model.head_mod
    for w, b, path in EDGE_LINEARS:
        sd[f"{prefix}{path}.weight"] = getattr(model, w)
        sd[f"{prefix}{path}.bias"] = getattr(model, b)
    inv = torch.argsort(head_row_order(cfg.in_channels)).to(model.head_w.device)
    sd[f"{prefix}head.head.weight"] = model.head_w[inv]
    sd[f"{prefix}head.head.bias"] = model.head_b[inv]
    return sd


def save_checkpoint(model, path: str, weight_scale_rule: str = "mse", **extra) -> None:
    """Write ``{"generator": state_dict, checkpoint_format, checkpoint_version, quantization}`` with CPU tensors."""
    sd = {k: v.detach().cpu() for k, v in state_dict_of(model).items()}
    torch.save({"generator": sd, "checkpoint_format": NVFP4_CHECKPOINT_FORMAT, "checkpoint_version": NVFP4_CHECKPOINT_VERSION,
                "quantization": {"format": "nvfp4", "backend": "fouroversix", "materialized": True, "dtype": "bfloat16",
                                 "scale_rule": weight_scale_rule}, **extra}, path)


def _copy(dst: torch.Tensor, src: torch.Tensor, key: str) -> None:
    if dst.numel() != src.numel():
        raise RuntimeError(f"size mismatch for {key}: checkpoint {tuple(src.shape)} vs model {tuple(dst.shape)}")
    dst.copy_(src.reshape(dst.shape).to(device=dst.device, dtype=dst.dtype))


def load_state_dict_into(model, state_dict: Mapping, prefix: str = "model.", weight_scale_rule: str = "mse",
                         strict: bool = True) -> list[str]:
    """Load a generator state dict (NVFP4 buffers or bf16 weights) into ``model``.  Returns the keys
    of the mapping that were not used; with ``strict`` a missing model tensor raises ``KeyError``.
    ``weight_scale_rule`` is the rule the stored weight codes were produced with (the checkpoint's
    ``quantization.scale_rule``); it fixes the E4M3 range of the scales."""
    sd = clean_fsdp_state_dict_keys(state_dict)
    used = set()

    def take(key):
        if key not in sd:
            if strict:
                raise KeyError(f"checkpoint has no tensor {key!r}")
            return None
        used.add(key)
        return sd[key]

    rule = ScaleRule(weight_scale_rule) if not isinstance(weight_scale_rule, ScaleRule) else weight_scale_rule
    dev = model.device
    for i, blk in enumerate(model.blocks):
        for attr, path in BLOCK_LINEARS:
            lin, base = getattr(blk, attr), f"{prefix}blocks.{i}.{path}"
            if f"{base}.quantized_weight_values" in sd:
                values, sf = take(f"{base}.quantized_weight_values"), take(f"{base}.quantized_weight_scale_factors")
                amax, meta = take(f"{base}.quantized_weight_amax"), take(f"{base}.quantized_weight_metadata")
                orig, padded = tuple(int(v) for v in meta[:2]), tuple(int(v) for v in meta[2:])
                if orig != (lin.out_f, lin.in_f):
                    raise RuntimeError(f"size mismatch for {base}: checkpoint {orig} vs model {(lin.out_f, lin.in_f)}")
                lin.q = QuantizedTensor(values.to(dev).contiguous(), sf.to(dev).contiguous(),
                                        amax.to(device=dev, dtype=torch.float32).reshape(1), "nvfp4", orig, rule, padded)
            else:
                w = take(f"{base}.weight")
                if w is not None:
                    if tuple(w.shape) != (lin.out_f, lin.in_f):
                        raise RuntimeError(f"size mismatch for {base}.weight: {tuple(w.shape)} vs {(lin.out_f, lin.in_f)}")
                    lin.q = quantize_to_fp4(w.to(device=dev, dtype=torch.bfloat16).contiguous(), QuantizationConfig(scale_rule=rule.value))
            b = take(f"{base}.bias")
            if b is not None:
                _copy(lin.bias, b, f"{base}.bias")
        for attr, path in BLOCK_VECTORS:
            t = take(f"{prefix}blocks.{i}.{path}")
            if t is not None:
                _copy(getattr(blk, attr), t, f"{prefix}blocks.{i}.{path}")
    for attr, key in (("patch_w", "patch_embedding.weight"), ("patch_b", "patch_embedding.bias"), ("head_mod", "head.modulation")):
        t = take(prefix + key)
        if t is not None:
            _copy(getattr(model, attr), t, prefix + key)
    for w, b, path in EDGE_LINEARS:
        for attr, key in ((w, f"{prefix}{path}.weight"), (b, f"{prefix}{path}.bias")):
            t = take(key)
            if t is not None:
                _copy(getattr(model, attr), t, key)
    if f"{prefix}head.head.weight" in used:
        order = head_row_order(model.cfg.in_channels).to(model.head_w.device)
        model.head_w.copy_(model.head_w[order])
        if f"{prefix}head.head.bias" in used:
            model.head_b.copy_(model.head_b[order])
    for blk in model.blocks:
        blk.fuse_qkv()
    model.modulation_all = torch.stack([blk.modulation for blk in model.blocks], 0)
    model._prompts = []                        # cached text K/V belong to the old weights
    model._graphs.clear()                      # captured graphs hold the old weight addresses
    model._time_cache.clear()                  # cached time embeddings belong to the old weights
    return [k for k in sd if k not in used]


def load_checkpoint(model, path: str, use_ema: bool = False, strict: bool = True) -> list[str]:
    """``torch.load`` a checkpoint file and load its generator into ``model``.  The file is read with
    ``weights_only=True``: the format holds tensors and plain containers only, so nothing in it needs unpickling
    arbitrary objects (the reference's loader passes ``weights_only=False``)."""
    ckpt = torch.load(path, map_location="cpu", weights_only=True)
    rule = "mse"
    if isinstance(ckpt, Mapping) and isinstance(ckpt.get("quantization"), Mapping):
        rule = ckpt["quantization"].get("weight_scale_rule") or ckpt["quantization"].get("scale_rule") or rule
    return load_state_dict_into(model, unwrap_generator_state_dict(ckpt, use_ema), weight_scale_rule=rule, strict=strict)
