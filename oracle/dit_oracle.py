"""CPU restatement (numpy) of one causal DiT block forward with the NVFP4 path.  TEST INFRASTRUCTURE ONLY.

Composes the functions of ``nvfp4_oracle`` in the order of the reference's block
(wan_5b/modules/causal_model.py:829-930; self-attention :327-791 with the quantized-cache branch
:628-652; cross-attention :197-295; cache update :1371-1483).  Parity status: the individual
steps are pinned by the fixtures of ``tests/golden`` (see ``nvfp4_oracle``), and the composition is
pinned by ``tests/golden/dit_block.npz``: inputs, weights, outputs and cache blocks of the reference's own
``CausalWanAttentionBlock`` run on CPU for four consecutive chunks (``tests/golden/make_golden_block.py``;
checked by ``tests/test_dit_oracle_golden.py``).
"""
from __future__ import annotations

import numpy as np

from . import nvfp4_oracle as O

f32 = np.float32


def gelu_tanh(x):
    x = x.astype(f32)
    return O.bf16_round((0.5 * x * (1.0 + np.tanh(0.7978845608028654 * (x + 0.044715 * x ** 3)))).astype(f32))


def linear(x, w_q, w_shape, bias):
    """FourOverSixLinear forward: quantize(x, mse) @ Wq^T (fp32) -> bf16 -> + bias -> bf16."""
    return O.linear_forward(x, w_q, w_shape, bias, "mse", "mse")


def block_forward(x, e, p, ctx_kn, ctx_v, cos, sin, past_k, past_v, heads, frame_tokens, chunk_tokens, eps=1e-6,
                  deq_mode=O.DEQ_FUSED_CUDA):
    """x: [S, C]; e: [F, 6, C]; p: dict of weights (quantized triples + shapes, biases, norm weights);
    past_k / past_v: lists of quantized cache blocks; deq_mode: which of the reference's dequantize roundings
    the cached blocks take (its fused CUDA kernel by default, DEQ_PYTORCH for its CPU path).
    Returns (x_out, new_k_block, new_v_block)."""
    s, c = x.shape
    frame = np.arange(s) // frame_tokens
    y = O.adaln_modulate(x, e[:, 1], e[:, 0], frame_tokens, eps)
    q = linear(y, p["q"], (c, c), p["q_b"])
    k = linear(y, p["k"], (c, c), p["k_b"])
    v = linear(y, p["v"], (c, c), p["v_b"])
    qn = O.rms_norm(q, p["norm_q"], eps)
    kn = O.rms_norm(k, p["norm_k"], eps)
    qr = O.rope_apply(qn.reshape(s, heads, 128), cos, sin)
    kr = O.rope_apply(kn.reshape(s, heads, 128), cos, sin)
    attn = O.window_attention(qr, kr, v.reshape(s, heads, 128), past_k, past_v, heads, chunk_tokens, mode=deq_mode)
    new_k = O.quantize_nvfp4(kr.reshape(s * heads, 128), "mse")
    new_v = O.quantize_nvfp4(v.reshape(s * heads, 128), "mse")
    o = linear(attn.reshape(s, c), p["o"], (c, c), p["o_b"])
    x1 = O.bf16_round(x + O.bf16_round(o * e[frame, 2]))
    cn = O.layer_norm_affine(x1, p["norm3_w"], p["norm3_b"], eps)
    cq = O.rms_norm(linear(cn, p["cq"], (c, c), p["cq_b"]), p["cnorm_q"], eps)
    ca = O.attention(cq.reshape(s, heads, 128), ctx_kn, ctx_v)
    x2 = O.bf16_round(x1 + linear(ca.reshape(s, c), p["co"], (c, c), p["co_b"]))
    f = O.adaln_modulate(x2, e[:, 4], e[:, 3], frame_tokens, eps)
    ffn = p["ffn_dim"]
    h = gelu_tanh(linear(f, p["ffn0"], (ffn, c), p["ffn0_b"]))
    y2 = linear(h, p["ffn2"], (c, ffn), p["ffn2_b"])
    x3 = O.bf16_round(x2 + O.bf16_round(y2 * e[frame, 5]))
    return x3, new_k, new_v


def text_kv(ctx, p, heads, eps=1e-6):
    """Cross-attention keys (RMS-normed) and values of the text context, [L, heads, 128] each."""
    c = ctx.shape[1]
    k = O.rms_norm(linear(ctx, p["ck"], (c, c), p["ck_b"]), p["cnorm_k"], eps)
    v = linear(ctx, p["cv"], (c, c), p["cv_b"])
    return k.reshape(-1, heads, 128), v.reshape(-1, heads, 128)
