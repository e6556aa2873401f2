"""Generate ``dit_block.npz`` and ``nvfp4_state_dict.pt`` by running the REFERENCE's own code on CPU.

    python tests/golden/make_golden_block.py --reference /path/to/LongLive

dit_block.npz: the reference's ``CausalWanAttentionBlock`` (wan_5b/modules/causal_model.py:793-930)
on a reduced configuration (dim 256, 2 heads, FFN 512, 3 frames of 6 x 8 tokens per chunk, window of
3 chunk blocks, 1 sink block) with every Linear replaced by the reference's ``FourOverSixLinear``
(PyTorch quantize and matmul backends), the NVFP4 KV cache the pipeline builds
(pipeline/causal_diffusion_inference.py:767-856) and the reference's own cache update
(``CausalWanModel._apply_cache_updates``, causal_model.py:1371-1483), run for four consecutive chunks:
the fourth rolls the cache.  Stored: weights, per-chunk inputs and outputs, and the cache block each
chunk writes.  What is replaced to make the block run on CPU: FlashAttention by an fp32 SDPA (the
file's own fallback, wan_5b/modules/attention.py:291-306), the Triton RoPE / adaLN kernels by the eager
code the file selects with LLV2_TRITON_ROPE=0 / LLV2_TRITON_ADALN=0, and the fused CUDA KV dequantize by
``QuantizedTensor.dequantize`` per block (the PyTorch rounding, quantized_tensor.py:187-209).

nvfp4_state_dict.pt: state-dict entries written by the reference's
``FourOverSixLinear.get_quantized_parameters`` (model/modules/linear.py:233-289) for two small Linears,
together with their bf16 master weights, in the checkpoint layout of utils/nvfp4_checkpoint.py.
"""
from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from make_golden import _setup, bf16_bits, u8  # noqa: E402

CFG = dict(dim=256, ffn_dim=512, heads=2, text_len=128, grid_h=6, grid_w=8, frames=3, window_frames=9, sink_frames=3)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the NVlabs/LongLive checkout")
    args = ap.parse_args()
    _setup(args.reference)
    torch.set_grad_enabled(False)

    import torch.nn as nn
    import utils.quant as uq
    from fouroversix import QuantizationConfig, quantize_to_fp4
    from fouroversix.model.config import ModuleQuantizationConfig
    from fouroversix.model.modules.linear import FourOverSixLinear
    from wan_5b.modules import causal_model as cm
    from wan_5b.modules.model import rope_params

    # -- CPU stand-ins for the GPU-only pieces (see the module docstring)
    def sdpa(q, k, v, *a, **kw):
        return torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2).float(), k.transpose(1, 2).float(), v.transpose(1, 2).float()).transpose(1, 2).contiguous().to(q.dtype)

    cm.attention = sdpa
    cm.flash_attention = sdpa

    def dequantize_blocks(kv_list, max_blocks, num_heads, block_token_size, dtype, device):
        parts = [kv_list[i].dequantize(dtype).view(block_token_size, num_heads, -1) for i in range(max_blocks)]
        return torch.cat(parts, 0).unsqueeze(0)

    uq.dequantize_kv_cache = dequantize_blocks

    c = CFG
    dim, ffn, heads = c["dim"], c["ffn_dim"], c["heads"]
    ft = c["grid_h"] * c["grid_w"]
    S = c["frames"] * ft
    torch.manual_seed(20)
    blk = cm.CausalWanAttentionBlock(dim, ffn, heads, local_attn_size=c["window_frames"], sink_size=c["sink_frames"],
                                     qk_norm=True, cross_attn_norm=True, eps=1e-6)
    for name, p in blk.named_parameters():
        if name.endswith("weight") and p.dim() == 2:
            p.data = torch.randn_like(p) * 0.05
        elif name.endswith("bias"):
            p.data = torch.randn_like(p) * 0.02
        elif p.dim() == 1:                      # norm weights
            p.data = 1 + 0.05 * torch.randn_like(p)
    blk = blk.to(torch.bfloat16)
    mcfg = ModuleQuantizationConfig(quantize_backend="pytorch", matmul_backend="pytorch", scale_rule="mse", keep_master_weights=True)

    def swap(parent, attr):
        setattr(parent, attr, FourOverSixLinear(getattr(parent, attr), mcfg))

    for attr in ("q", "k", "v", "o"):
        swap(blk.self_attn, attr)
        swap(blk.cross_attn, attr)
    blk.ffn[0] = FourOverSixLinear(blk.ffn[0], mcfg)
    blk.ffn[2] = FourOverSixLinear(blk.ffn[2], mcfg)

    kvq = QuantizationConfig(backend="pytorch", scale_rule="mse")
    block_tokens = S
    max_blocks = c["window_frames"] // c["frames"]
    zero_qt = quantize_to_fp4(torch.zeros(block_tokens * heads, 128, dtype=torch.bfloat16), kvq)
    cache = {"k": [uq.clone_quantized_tensor(zero_qt) for _ in range(max_blocks)],
             "v": [uq.clone_quantized_tensor(zero_qt) for _ in range(max_blocks)],
             "quantized": True, "block_token_size": block_tokens, "max_blocks": max_blocks, "num_heads": heads,
             "num_filled_blocks": 0, "global_end_index": torch.tensor([0]), "local_end_index": torch.tensor([0]),
             "pinned_start": torch.tensor([-1]), "pinned_len": torch.tensor([0])}

    class ModelStub:                      # the one attribute _apply_cache_updates reads from the model
        kv_quant_config = kvq

    d = 128
    freqs = torch.cat([rope_params(1024, d - 4 * (d // 6)), rope_params(1024, 2 * (d // 6)), rope_params(1024, 2 * (d // 6))], dim=1)
    gen = torch.Generator().manual_seed(21)
    context = torch.randn(1, c["text_len"], dim, generator=gen).bfloat16()
    out = {"cfg": np.array([dim, ffn, heads, c["text_len"], c["grid_h"], c["grid_w"], c["frames"], c["window_frames"], c["sink_frames"]]),
           "context": bf16_bits(context[0])}
    names = {"q": blk.self_attn.q, "k": blk.self_attn.k, "v": blk.self_attn.v, "o": blk.self_attn.o, "cq": blk.cross_attn.q,
             "ck": blk.cross_attn.k, "cv": blk.cross_attn.v, "co": blk.cross_attn.o, "ffn0": blk.ffn[0], "ffn2": blk.ffn[2]}
    for n, lin in names.items():
        out[f"w_{n}"] = bf16_bits(lin.weight.data)
        out[f"b_{n}"] = bf16_bits(lin.bias.data)
    out["norm_q"] = bf16_bits(blk.self_attn.norm_q.weight.data)
    out["norm_k"] = bf16_bits(blk.self_attn.norm_k.weight.data)
    out["cnorm_q"] = bf16_bits(blk.cross_attn.norm_q.weight.data)
    out["cnorm_k"] = bf16_bits(blk.cross_attn.norm_k.weight.data)
    out["norm3_w"] = bf16_bits(blk.norm3.weight.data)
    out["norm3_b"] = bf16_bits(blk.norm3.bias.data)
    out["modulation"] = bf16_bits(blk.modulation.data)

    grid = torch.tensor([[c["frames"], c["grid_h"], c["grid_w"]]])
    seq_lens = torch.tensor([S])
    n_chunks = max_blocks + 1
    for chunk in range(n_chunks):
        x = (torch.randn(1, S, dim, generator=gen) * 1.5).bfloat16()
        e = (torch.randn(1, c["frames"], 6, dim, generator=gen) * 0.3).bfloat16()        # time projection; the block adds its modulation
        y, info = blk(x, e, seq_lens, grid, freqs, context, None, None, kv_cache=cache, current_start=chunk * S)
        cm.CausalWanModel._apply_cache_updates(ModelStub(), [cache], [(0, info)])
        action = info[2]["action"]
        slot = info[2]["local_start_index"] // block_tokens
        out[f"x{chunk}"] = bf16_bits(x[0])
        out[f"e{chunk}"] = bf16_bits(e[0])
        out[f"y{chunk}"] = bf16_bits(y[0])
        out[f"action{chunk}"] = np.array([0 if action == "direct_insert" else 1, slot])
        for side in ("k", "v"):
            qt = cache[side][slot]
            out[f"{side}_codes{chunk}"] = qt.values.numpy().copy()
            out[f"{side}_sf{chunk}"] = u8(qt.scale_factors).copy()
            out[f"{side}_amax{chunk}"] = np.float32(qt.amax.item())
        print(f"chunk {chunk}: {action}, block slot {slot}, |y| mean {y.float().abs().mean():.4f}")
    np.savez_compressed(os.path.join(HERE, "dit_block.npz"), **out)

    # ---- RoPE with a temporal scale and a multi-shot offset (utils/position_embedding_utils.py:56-105) ----------
    gen = torch.Generator().manual_seed(41)
    F_, Hh, Ww, nh = 3, 4, 6, 2
    xq = torch.randn(1, F_ * Hh * Ww, nh, d, generator=gen).bfloat16()
    ro = {"x": bf16_bits(xq), "grid": np.array([F_, Hh, Ww])}
    for tag, (start, ts, off) in {"a": (5, 0.5, 0.0), "b": (7, 1.0, 2.5), "c": (2, 0.75, 3.25)}.items():
        yy = cm.causal_rope_apply(xq, [(F_, Hh, Ww)], freqs, start_frame=start, t_scale=ts, temporal_offset=off).type_as(xq)
        ro[f"y_{tag}"] = bf16_bits(yy)
        ro[f"p_{tag}"] = np.array([start, ts, off], dtype=np.float64)
    np.savez_compressed(os.path.join(HERE, "rope_offset.npz"), **ro)

    # ---- NVFP4 state-dict entries as the reference's exporter writes them ---------------------------
    from utils.nvfp4_checkpoint import NVFP4_CHECKPOINT_FORMAT, NVFP4_CHECKPOINT_VERSION
    gen = torch.Generator().manual_seed(31)
    sd, masters = {}, {}
    qcfg = ModuleQuantizationConfig(quantize_backend="pytorch", matmul_backend="pytorch", scale_rule="mse")
    for name, (o, i) in {"blocks.0.self_attn.q": (256, 256), "blocks.0.ffn.0": (512, 256)}.items():
        lin = nn.Linear(i, o).to(torch.bfloat16)
        lin.weight.data = (torch.randn(o, i, generator=gen) * 0.05).bfloat16()
        lin.bias.data = (torch.randn(o, generator=gen) * 0.02).bfloat16()
        ql = FourOverSixLinear(lin, qcfg)
        for k, v in ql.get_quantized_parameters("weight", lin.weight.data).items():
            sd[f"{name}.{k}"] = v.clone()
        sd[f"{name}.bias"] = lin.bias.data.clone()
        masters[f"{name}.weight"] = lin.weight.data.clone()
    # outer layout of scripts/save_merged_nvfp4_generator.py:220-236 (plus the bf16 masters, for the tests)
    torch.save({"generator": sd, "checkpoint_format": NVFP4_CHECKPOINT_FORMAT, "checkpoint_version": NVFP4_CHECKPOINT_VERSION,
                "quantization": {"format": "nvfp4", "backend": "fouroversix", "materialized": True, "dtype": "bfloat16",
                                 "scale_rule": "mse"}, "masters": masters},
               os.path.join(HERE, "nvfp4_state_dict.pt"))
    print("written:", os.path.join(HERE, "dit_block.npz"), os.path.join(HERE, "nvfp4_state_dict.pt"))


if __name__ == "__main__":
    main()
