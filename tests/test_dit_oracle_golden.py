"""The block-composition oracle (``oracle/dit_oracle.py``) against the reference's own block.

``tests/golden/dit_block.npz`` holds inputs, weights, outputs and written cache blocks of the reference's
``CausalWanAttentionBlock`` (wan_5b/modules/causal_model.py:793-930) run on CPU with its PyTorch NVFP4
backends and its own cache update for four consecutive chunks (written by
``tests/golden/make_golden_block.py``).  The oracle composes the pinned step functions of
``nvfp4_oracle`` in the same order; this pins the order itself: which tensor is smoothed, what goes into
the cache, where the gates round, how a roll selects the window.

Tolerance.  Every step matches the reference bit for bit except the fp32 matmuls, whose summation order
depends on the BLAS build (<= 1 bf16 ulp after rounding).  One such ulp ahead of a quantizer can flip an
E2M1 code (or a block's 4-vs-6 choice), a change of up to ~25 % of that element of that GEMM operand.  Block
outputs are therefore compared with: relative Frobenius error <= 5e-3, at least 98 % of the elements
bit-identical, and at most 0.1 % of the elements further than 2^-4 |ref| + 2^-5 mean|ref| from the reference."""
import numpy as np

from oracle import dit_oracle as DO
from oracle import nvfp4_oracle as O


def _params(g):
    dim, ffn = int(g["cfg"][0]), int(g["cfg"][1])
    p = {"ffn_dim": ffn}
    for n in ("q", "k", "v", "o", "cq", "ck", "cv", "co", "ffn0", "ffn2"):
        p[n] = O.quantize_nvfp4(O.bf16_from_bits(g[f"w_{n}"]), "mse")
        p[n + "_b"] = O.bf16_from_bits(g[f"b_{n}"])
    for n in ("norm_q", "norm_k", "cnorm_q", "cnorm_k", "norm3_w", "norm3_b"):
        p[n] = O.bf16_from_bits(g[n])
    return p, dim


def test_block_oracle_reproduces_reference_block(golden):
    g = golden("dit_block.npz")
    dim, ffn, heads, text_len, gh, gw, frames, window_frames, sink_frames = (int(v) for v in g["cfg"])
    p, _ = _params(g)
    ft, S = gh * gw, frames * gh * gw
    max_blocks = window_frames // frames
    ctx = O.bf16_from_bits(g["context"])
    ctx_kn, ctx_v = DO.text_kv(ctx, p, heads)
    mod = O.bf16_from_bits(g["modulation"])                       # [1, 6, C]
    past_k, past_v = [], []
    actions = []
    for chunk in range(max_blocks + 1):
        x = O.bf16_from_bits(g[f"x{chunk}"])
        e = O.bf16_round(mod + O.bf16_from_bits(g[f"e{chunk}"]))   # causal_model.py:863, a bf16 add
        cos, sin = O.rope_tables(chunk * frames, frames, gh, gw)
        y, nk, nv = DO.block_forward(x, e, p, ctx_kn, ctx_v, cos, sin, past_k, past_v, heads, ft, S, deq_mode=O.DEQ_PYTORCH)
        ref = O.bf16_from_bits(g[f"y{chunk}"])
        rel = np.linalg.norm(y - ref) / np.linalg.norm(ref)
        same = (O.bf16_bits(y) == g[f"y{chunk}"]).mean()
        far = (np.abs(y - ref) > np.abs(ref) * 2.0 ** -4 + 2.0 ** -5 * np.abs(ref).mean()).mean()
        assert rel <= 5e-3 and same >= 0.98 and far <= 1e-3, (chunk, rel, same, far)
        # the cache block the reference wrote: same amax, and codes / scales equal up to the few flips explained above
        for side, blk in (("k", nk), ("v", nv)):
            assert np.float32(blk[2]) == g[f"{side}_amax{chunk}"], (chunk, side)
            assert (blk[0] != g[f"{side}_codes{chunk}"]).mean() <= 0.02, (chunk, side)
            assert (blk[1] != g[f"{side}_sf{chunk}"]).mean() <= 0.01, (chunk, side)
        actions.append(tuple(int(v) for v in g[f"action{chunk}"]))
        past_k.append(nk)
        past_v.append(nv)
        if len(past_k) > max_blocks - 1:          # the roll keeps the sink block and evicts the oldest block behind it
            del past_k[1], past_v[1]
    # the reference inserted directly while the cache filled and rolled on the chunk after it was full
    assert actions == [(0, 0), (0, 1), (0, 2), (1, 2)]
