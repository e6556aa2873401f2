"""Generate the golden fixtures in this folder by running the REFERENCE's own CPU code.

Run from the repository root, in a container where the reference checkout is mounted:

    python tests/golden/make_golden.py --reference /path/to/LongLive

It imports the reference's PyTorch backends (quantizer, QuantizedTensor.dequantize, the
PyTorch matmul backend, utils.quant helpers, the eager RoPE / norm code of the causal DiT)
and stores small input/output vectors as ``.npz`` files.  The fixtures travel with the
repository; the reference itself does not, so nothing else reads the reference at run time.

bf16 tensors are stored as uint16 bit patterns, e4m3 scales as uint8 bit patterns.
``--only fp16`` writes just ``quantize_fp16.npz`` (the quantizer on an fp16 tensor, stored as uint16 bit patterns of
the halves) and leaves the other files as they are.
"""
from __future__ import annotations

import argparse
import hashlib
import importlib.metadata as md
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _setup(reference_root: str) -> None:
    sys.path.insert(0, os.path.join(reference_root, "fouroversix", "src"))
    sys.path.insert(0, reference_root)
    orig = md.version
    # fouroversix/__init__.py asks importlib.metadata for its own version; it is not
    # pip-installed here, so answer with the version its setup.py declares.
    md.version = lambda n: "1.1.0" if n == "fouroversix" else orig(n)
    os.environ["LLV2_TRITON_ROPE"] = "0"
    os.environ["LLV2_TRITON_ADALN"] = "0"
    import torch.nn as nn
    d = types.ModuleType("diffusers")
    cu = types.ModuleType("diffusers.configuration_utils")
    mo = types.ModuleType("diffusers.models")
    mu = types.ModuleType("diffusers.models.modeling_utils")

    class ConfigMixin:
        pass

    class ModelMixin(nn.Module):
        pass

    cu.ConfigMixin = ConfigMixin
    cu.register_to_config = lambda f: f
    mu.ModelMixin = ModelMixin
    for n, m in {"diffusers": d, "diffusers.configuration_utils": cu, "diffusers.models": mo,
                 "diffusers.models.modeling_utils": mu}.items():
        sys.modules[n] = m
    sys.modules["ftfy"] = types.ModuleType("ftfy")
    ed = types.ModuleType("easydict")
    ed.EasyDict = dict
    sys.modules["easydict"] = ed


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().to(torch.bfloat16).view(torch.int16).numpy().view(np.uint16)


def u8(t: torch.Tensor) -> np.ndarray:
    return t.detach().contiguous().view(torch.uint8).numpy()


def sha(a: np.ndarray) -> str:
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def edge_case_tensor(gen: torch.Generator) -> torch.Tensor:
    """[200, 192] bf16 with outliers, an all-zero row, tiny blocks, negative zeros, ties."""
    x = torch.randn(200, 192, generator=gen)
    mask = torch.rand(200, 192, generator=gen) < 0.01
    x = torch.where(mask, x * 20, x)
    x[3] = 0.0                                  # all-zero row
    x[5, 16:32] = 1e-6                          # block whose scale underflows to 0
    x[6, 0:16] = 3e-4                           # block with a subnormal e4m3 scale
    x[7, 32:48] = torch.linspace(-2e-3, 2e-3, 16)
    x[8, 0:16] = torch.tensor([0.0, -0.0, 0.25, -0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -5.0, 6.0,
                               -6.0, 0.5, -0.5, 1.0])
    x[9, 48:64] = 7e-4
    x[10, 0:16] = torch.tensor([1.1e-3] + [2e-4] * 15)
    x[11, 16:32] = torch.tensor([-9e-4] + [1e-4] * 7 + [8.9e-4] + [0.0] * 7)
    for r in range(12, 44):                     # a ladder of tiny block maxima around the
        x[r, 64:80] = (2.0 ** -(4 + 0.25 * (r - 12))) * torch.sign(torch.randn(16, generator=gen))
        x[r, 80:96] = (2.0 ** -(8 + 0.25 * (r - 12))) * torch.randn(16, generator=gen)
    return x.bfloat16()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the NVlabs/LongLive checkout")
    ap.add_argument("--only", default="all", choices=["all", "fp16"], help="fp16: write quantize_fp16.npz and nothing else")
    args = ap.parse_args()
    _setup(args.reference)

    from fouroversix import QuantizationConfig, fp4_matmul, quantize_to_fp4
    from fouroversix.quantize.quantized_tensor import from_blocked

    rules = ["static_6", "static_4", "mae", "mse", "abs_max"]

    # ---- 0. quantizer on fp16 input (the reference widens to fp32; 11-bit significands, fp16 subnormals) ----------
    gen16 = torch.Generator().manual_seed(4321)
    x16 = (torch.randn(200, 192, generator=gen16) * 2).half()
    x16[3] = 0
    x16[5, 0:16] = torch.tensor([6.1e-5, -3.0e-5, 5.96e-8, 0.0] * 4).half()          # around the smallest normal / subnormal halves
    x16[7, 16:32] = torch.tensor([60000.0, -65504.0] + [1.0] * 14).half()            # the largest halves set the tensor amax
    x16[9, 32:48] = -0.0
    out16 = {"x": x16.view(torch.int16).numpy().view(np.uint16)}
    for rule in rules:
        q = quantize_to_fp4(x16, QuantizationConfig(backend="pytorch", scale_rule=rule))
        out16[f"{rule}_codes"] = q.values.numpy()
        out16[f"{rule}_sf"] = u8(q.scale_factors)
        out16[f"{rule}_amax"] = np.float32(q.amax.item())
    np.savez_compressed(os.path.join(HERE, "quantize_fp16.npz"), **out16)
    if args.only == "fp16":
        return

    # ---- 1. quantizer, all rules, edge-case tensor + plain randn + all-zero ----------
    gen = torch.Generator().manual_seed(1234)
    cases = {
        "edge": edge_case_tensor(gen),
        "randn": torch.randn(256, 128, generator=gen).bfloat16(),
        "zeros": torch.zeros(128, 64).bfloat16(),
        "ragged": (torch.randn(130, 320, generator=gen) * 3).bfloat16(),
    }
    out = {}
    for cname, x in cases.items():
        out[f"{cname}_x"] = bf16_bits(x)
        for rule in rules:
            q = quantize_to_fp4(x, QuantizationConfig(backend="pytorch", scale_rule=rule))
            out[f"{cname}_{rule}_codes"] = q.values.numpy()
            out[f"{cname}_{rule}_sf"] = u8(q.scale_factors)
            out[f"{cname}_{rule}_amax"] = np.float32(q.amax.item())
            out[f"{cname}_{rule}_padded"] = np.array(q.padded_shape, dtype=np.int64)
            deq32 = q.dequantize(torch.float32)
            deq16 = q.dequantize(torch.bfloat16)
            out[f"{cname}_{rule}_deq_f32"] = deq32.numpy()
            out[f"{cname}_{rule}_deq_bf16"] = bf16_bits(deq16)
    np.savez_compressed(os.path.join(HERE, "quantize_small.npz"), **out)

    # ---- 2. config-1 linear: digests of the full tensors + an output slice ------------
    torch.manual_seed(0)
    M, K, N = 2640, 3072, 3072
    x = torch.randn(M, K)
    x = torch.where(torch.rand(M, K) < 0.001, x * 20, x).bfloat16()
    w = (torch.randn(N, K) * 0.02).bfloat16()
    cfg = QuantizationConfig(backend="pytorch", scale_rule="mse")
    xq = quantize_to_fp4(x, cfg)
    wq = quantize_to_fp4(w, cfg)
    y = fp4_matmul(xq, wq, backend="pytorch")
    rows = np.r_[0:16, 1311:1327, 2624:2640]
    np.savez_compressed(
        os.path.join(HERE, "config1_linear.npz"),
        x_sha=sha(bf16_bits(x)), w_sha=sha(bf16_bits(w)),
        x_codes_sha=sha(xq.values.numpy()), x_sf_sha=sha(u8(xq.scale_factors)),
        x_amax=np.float32(xq.amax.item()),
        w_codes_sha=sha(wq.values.numpy()), w_sf_sha=sha(u8(wq.scale_factors)),
        w_amax=np.float32(wq.amax.item()),
        x_codes_rows=xq.values.numpy()[rows], rows=rows,
        y_rows=bf16_bits(y[rows]),
        y_abs_mean=np.float32(y.float().abs().mean().item()),
    )

    # ---- 3. small matmul incl. mixed rules ---------------------------------------------
    gen = torch.Generator().manual_seed(7)
    a = torch.randn(200, 256, generator=gen).bfloat16()
    b = (torch.randn(136, 256, generator=gen) * 0.05).bfloat16()
    mm = {"a": bf16_bits(a), "b": bf16_bits(b)}
    for ra, rb in [("mse", "mse"), ("static_6", "static_6"), ("mse", "static_6"), ("abs_max", "mae")]:
        yy = fp4_matmul(a, b, backend="pytorch",
                        input_config=QuantizationConfig(backend="pytorch", scale_rule=ra),
                        other_config=QuantizationConfig(backend="pytorch", scale_rule=rb))
        mm[f"y_{ra}_{rb}"] = bf16_bits(yy)
    np.savez_compressed(os.path.join(HERE, "matmul_small.npz"), **mm)

    # ---- 4. KV helpers: k_smooth, block quantize layout, per-block dequantize ----------
    import utils.quant as uq
    gen = torch.Generator().manual_seed(11)
    H, T = 4, 48
    k = torch.randn(1, T, H, 128, generator=gen).bfloat16()
    ks = uq.k_smooth(k)
    kvq = quantize_to_fp4(k[0].reshape(-1, 128).contiguous(), QuantizationConfig(backend="pytorch", scale_rule="mse"))
    deq = kvq.dequantize(torch.bfloat16).view(T, H, 128)
    np.savez_compressed(
        os.path.join(HERE, "kv_small.npz"),
        k=bf16_bits(k), k_smooth=bf16_bits(ks),
        codes=kvq.values.numpy(), sf=u8(kvq.scale_factors), amax=np.float32(kvq.amax.item()),
        deq_bf16=bf16_bits(deq),
        sf_unswizzled=u8(from_blocked(kvq.scale_factors, (kvq.padded_shape[0], 8))),
    )

    # ---- 5. RoPE (eager fp64 path), RMSNorm, LayerNorm+modulate (eager), SDPA ----------
    from wan_5b.modules import causal_model as cm
    from wan_5b.modules.model import WanLayerNorm, WanRMSNorm, rope_params
    gen = torch.Generator().manual_seed(21)
    d = 128
    freqs = torch.cat([rope_params(1024, d - 4 * (d // 6)), rope_params(1024, 2 * (d // 6)),
                       rope_params(1024, 2 * (d // 6))], dim=1)
    F_, Hh, Ww, heads = 2, 4, 6, 3
    q = torch.randn(1, F_ * Hh * Ww, heads, d, generator=gen).bfloat16()
    roped = cm.causal_rope_apply(q, [(F_, Hh, Ww)], freqs, start_frame=5).type_as(q)

    C = 384
    xin = (torch.randn(1, F_ * Hh * Ww, C, generator=gen) * 2 + 0.3).bfloat16()
    wn = (1 + 0.1 * torch.randn(C, generator=gen)).bfloat16()
    rms = WanRMSNorm(C, eps=1e-6)
    rms.weight.data = wn.clone()
    rms = rms.to(torch.bfloat16)
    y_rms = rms(xin)
    ln = WanLayerNorm(C, eps=1e-6)
    e_scale = (torch.randn(1, F_, 1, C, generator=gen) * 0.1).bfloat16()
    e_shift = (torch.randn(1, F_, 1, C, generator=gen) * 0.1).bfloat16()
    # the eager form of the modulated norm, wan_5b/modules/causal_model.py:875
    y_ada = (ln(xin).unflatten(1, (F_, Hh * Ww)) * (1 + e_scale) + e_shift).flatten(1, 2)

    lq, lk = 24, 72
    aq = torch.randn(1, lq, heads, d, generator=gen).bfloat16()
    ak = torch.randn(1, lk, heads, d, generator=gen).bfloat16()
    av = torch.randn(1, lk, heads, d, generator=gen).bfloat16()
    att = torch.nn.functional.scaled_dot_product_attention(
        aq.transpose(1, 2).float(), ak.transpose(1, 2).float(), av.transpose(1, 2).float()
    ).transpose(1, 2).contiguous().bfloat16()
    np.savez_compressed(
        os.path.join(HERE, "elementwise_small.npz"),
        rope_x=bf16_bits(q), rope_y=bf16_bits(roped), rope_grid=np.array([F_, Hh, Ww, 5]),
        norm_x=bf16_bits(xin), rms_w=bf16_bits(wn), rms_y=bf16_bits(y_rms),
        ada_scale=bf16_bits(e_scale), ada_shift=bf16_bits(e_shift), ada_y=bf16_bits(y_ada),
        att_q=bf16_bits(aq), att_k=bf16_bits(ak), att_v=bf16_bits(av), att_y=bf16_bits(att),
    )
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
