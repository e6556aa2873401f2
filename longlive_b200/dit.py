"""Causal DiT block stack on the NVFP4 kernels: the caller side of the hot path.

Mirrors the inference forward of the reference's causal Wan2.2-5B-shaped DiT block
(wan_5b/modules/causal_model.py:829-930 block, :327-791 self-attention with the rolling NVFP4 KV
cache, :197-295 cross-attention, :1371-1483 cache update) as a sequence of C-ABI calls on
persistent buffers: no per-call allocation, no host synchronisation, cache roll by permuting a
block table instead of copying slots.  Random-init weights of the reference's shapes; patch
embedding, time/text MLPs and the head are plain bf16 torch ops (outside the hot path).

Per block and forward (S tokens of the chunk, window = cached blocks + current chunk):
  adaLN(e0,e1)+quantize -> q,k,v GEMMs(+bias; v also emits its amax)
  -> RMSNorm+RoPE (q) / RMSNorm+RoPE+k_smooth+amax (k)
  -> attention over [NVFP4 cache blocks, decoded inside the kernel | current chunk] -> quantize -> o GEMM(+bias,
  gate e2, residual) -> LayerNorm+quantize -> cross q GEMM -> RMSNorm -> attention over the text
  K/V -> quantize -> o GEMM(+bias, residual) -> adaLN(e3,e4)+quantize -> FFN GEMM(+bias, GELU, amax)
  -> quantize (amax given) -> FFN GEMM(+bias, gate e5, residual); then the rotated keys and the
  values of the chunk are quantized straight into the current cache block.

Sequence parallelism (``sp_group``): tokens are sharded for everything except self-attention,
where heads are sharded; see ``longlive_b200/sp.py``.  With ``sync_amax`` every per-tensor amax is
MAX-reduced over the group so that codes and scales equal the single-GPU run bit for bit.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from . import _lib, ops, sp
from .enums import ScaleRule
from .quantize import QuantizationConfig, QuantizedTensor, quantize_to_fp4
from .scheduler import FlowUniPCMultistepScheduler

MSE = ScaleRule.mse.cuda_id()


@dataclass
class DiTConfig:
    dim: int = 3072
    ffn_dim: int = 14336
    heads: int = 24
    layers: int = 30
    text_len: int = 512
    text_dim: int = 4096
    freq_dim: int = 256
    grid_h: int = 22                 # post-patch latent grid (44 x 80 latent, patch 1x2x2)
    grid_w: int = 40
    frames_per_chunk: int = 3
    window_frames: int = 15          # sink + local window, current chunk included
    sink_frames: int = 3
    global_sink_frames: int = 0      # frames anchored for the whole video (the reference's global_sink_size)
    in_channels: int = 48
    eps: float = 1e-6

    @property
    def frame_tokens(self) -> int:
        return self.grid_h * self.grid_w

    @property
    def chunk_tokens(self) -> int:
        return self.frames_per_chunk * self.frame_tokens

    @property
    def max_blocks(self) -> int:
        return self.window_frames // self.frames_per_chunk

    @property
    def patch_dim(self) -> int:
        return self.in_channels * 4


def rope_tables(cfg: DiTConfig, start_frame: int, device, t_scale: float = 1.0,
                temporal_offset: float = 0.0) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin fp32 [chunk_tokens, 64] for frames start_frame.., tokens in (f, h, w) order
    (wan_5b/modules/model.py:29-36, wan_5b/modules/causal_model.py:156-165, 1075-1081).  The temporal position of
    frame f is (start_frame + f + temporal_offset) * t_scale: ``t_scale`` < 1 compresses time, ``temporal_offset``
    is the multi-shot offset (shot index times phi) of utils/position_embedding_utils.py:56-105; with the defaults
    the positions are the integers the reference looks up in its 1024-entry table (:73-78)."""
    d = 128
    dims = [d - 4 * (d // 6), 2 * (d // 6), 2 * (d // 6)]

    def ang(pos, dim):
        inv = 1.0 / torch.pow(10000.0, torch.arange(0, dim, 2, dtype=torch.float64) / dim)
        return torch.outer(pos.to(torch.float64), inv)

    f, h, w = cfg.frames_per_chunk, cfg.grid_h, cfg.grid_w
    at = ang((torch.arange(start_frame, start_frame + f, dtype=torch.float64) + float(temporal_offset)) * float(t_scale), dims[0])
    ah = ang(torch.arange(h), dims[1])
    aw = ang(torch.arange(w), dims[2])
    full = torch.cat([at[:, None, None, :].expand(f, h, w, -1), ah[None, :, None, :].expand(f, h, w, -1),
                      aw[None, None, :, :].expand(f, h, w, -1)], dim=-1).reshape(f * h * w, d // 2)
    return full.cos().float().to(device).contiguous(), full.sin().float().to(device).contiguous()


class _Linear:
    """An NVFP4 weight [out, in] quantized once (4-over-6 MSE) plus its bf16 bias."""

    def __init__(self, out_f: int, in_f: int, gen, device, std: float = 0.02):
        w = (torch.randn(out_f, in_f, generator=gen, device=device) * std).bfloat16()
        self.q: QuantizedTensor = quantize_to_fp4(w, QuantizationConfig(scale_rule="mse"))
        self.bias = (torch.randn(out_f, generator=gen, device=device) * 0.02).bfloat16()
        self.out_f, self.in_f = out_f, in_f
        self.weight_bf16 = None

    def keep_master(self, w):
        self.weight_bf16 = w


class _Act:
    """A reusable NVFP4 activation buffer (codes / scales / amax) for up to ``rows`` x ``cols``."""

    def __init__(self, rows: int, cols: int, device):
        mp = ops.padded_rows(rows)
        self.codes = torch.zeros((mp, cols // 2), dtype=torch.uint8, device=device)
        self.sf = torch.zeros(mp * cols // 16, dtype=torch.float8_e4m3fn, device=device)
        self.amax = torch.zeros(1, dtype=torch.float32, device=device)
        self.rows, self.cols = rows, cols


class Block:
    def __init__(self, cfg: DiTConfig, gen, device):
        c, f = cfg.dim, cfg.ffn_dim
        self.q, self.k, self.v, self.o = (_Linear(c, c, gen, device) for _ in range(4))
        self.cq, self.ck, self.cv, self.co = (_Linear(c, c, gen, device) for _ in range(4))
        self.ffn0, self.ffn2 = _Linear(f, c, gen, device), _Linear(c, f, gen, device)
        ones = lambda: (1 + 0.05 * torch.randn(c, generator=gen, device=device)).bfloat16()
        self.norm_q, self.norm_k, self.cnorm_q, self.cnorm_k = ones(), ones(), ones(), ones()
        self.norm3_w, self.norm3_b = ones(), (0.02 * torch.randn(c, generator=gen, device=device)).bfloat16()
        self.modulation = (torch.randn(1, 6, c, generator=gen, device=device) / math.sqrt(c)).bfloat16()
        self.fuse_qkv()

    def fuse_qkv(self) -> None:
        """Concatenate the q, k and v weights (codes, swizzled scales, bias; one amax each) for the
        grouped GEMM launch.  Call again after the weights were replaced."""
        qs = [self.q.q, self.k.q, self.v.q]
        self.qkv_rule = qs[0].scale_rule
        self.qkv_ok = all(t.scale_rule == self.qkv_rule and t.original_shape == qs[0].original_shape for t in qs)
        self.qkv_codes = torch.cat([t.values for t in qs], 0)
        self.qkv_sf = torch.cat([t.scale_factors.view(torch.uint8).reshape(-1) for t in qs], 0).view(torch.float8_e4m3fn)
        self.qkv_amax = torch.cat([t.amax.reshape(1) for t in qs], 0)
        self.qkv_bias = torch.cat([self.q.bias, self.k.bias, self.v.bias], 0)


class KVCache:
    """Per layer ``max_blocks`` NVFP4 slots for K and V, each [block_tokens * local_heads, 128].

    ``order[layer]`` lists slot indices from oldest to newest; the last entry is the block of the
    current chunk.  Rolling (wan_5b/modules/causal_model.py:1396-1411) permutes this table."""

    def __init__(self, cfg: DiTConfig, local_heads: int, device):
        rows = cfg.chunk_tokens * local_heads
        mp = ops.padded_rows(rows)
        # the tensor amax of every block lives in one array [layer, slot, K / V], so that a forward can clear the scalars of
        # the block it is about to write for all layers with one fill
        self.amax_pool = torch.zeros((cfg.layers, cfg.max_blocks, 2), dtype=torch.float32, device=device)
        mk = lambda l, s, kv: QuantizedTensor(torch.zeros((mp, 64), dtype=torch.uint8, device=device),
                                              torch.zeros(mp * 8, dtype=torch.float8_e4m3fn, device=device),
                                              self.amax_pool[l, s, kv:kv + 1], "nvfp4", (rows, 128), "mse", (mp, 128))
        self.k = [[mk(l, s, 0) for s in range(cfg.max_blocks)] for l in range(cfg.layers)]
        self.v = [[mk(l, s, 1) for s in range(cfg.max_blocks)] for l in range(cfg.layers)]
        self.order = list(range(cfg.max_blocks))
        self.filled = 0                       # number of valid blocks, current chunk included
        self.version = 0                      # bumped whenever the set of past blocks changes
        self.pinned: int | None = None        # slot of the chunk pinned as shot sink at the last scene cut
        self.cfg = cfg
        if cfg.sink_frames % cfg.frames_per_chunk or cfg.global_sink_frames % cfg.frames_per_chunk:
            raise ValueError("sink_frames and global_sink_frames must be whole chunks (the cache is a table of chunk blocks)")


    def protected_blocks(self) -> int:
        """Leading blocks a roll must keep (``effective_sink`` of wan_5b/modules/causal_model.py:498-534):
        the global sink, plus the pinned chunk once it sits right behind it; a pinned chunk further
        back floats (the roll moves it forward with the others) and the original sink is no longer
        kept; without a pinned chunk the larger of global sink and sink."""
        cfg = self.cfg
        g = cfg.global_sink_frames // cfg.frames_per_chunk
        if self.pinned is None:
            return max(g, cfg.sink_frames // cfg.frames_per_chunk)
        return g + 1 if self.order.index(self.pinned) == g else g

    def begin_chunk(self) -> None:
        """Make room for a new chunk: grow until full, then evict the oldest block behind the
        protected prefix (causal_model.py:596-625, 1396-1446: with a table of blocks the roll is a
        permutation, and the pinned chunk's position follows it by construction)."""
        cfg = self.cfg
        self.version += 1
        if self.filled < cfg.max_blocks:
            self.filled += 1
            return
        victim = self.order.pop(self.protected_blocks())
        self.order.append(victim)

    def pin_current(self) -> None:
        """Scene cut: the chunk just cached becomes the shot sink; it replaces the original sink on the
        following rolls (pipeline/causal_diffusion_inference.py:659-664, 1026-1042).  A whole chunk is
        pinned: the reference pins min(sink_size, chunk) frames and its configurations use sink_size >= chunk."""
        if self.cfg.sink_frames < self.cfg.frames_per_chunk:
            raise NotImplementedError("pinning less than one chunk")
        self.pinned = self.current_slot()

    def reset_keep_global(self) -> None:
        """Scene cut with clean re-cache: drop every block but the global sink; the current chunk
        becomes the first block behind it and the pin is cleared
        (``_zero_kv_data``, pipeline/causal_diffusion_inference.py:1044-1052)."""
        g = self.cfg.global_sink_frames // self.cfg.frames_per_chunk
        cur = self.current_slot()
        keep = self.order[:g]
        if cur in keep:
            raise RuntimeError("the current chunk lies inside the global sink: nothing to reset")
        self.order = keep + [cur] + [s for s in self.order if s != cur and s not in keep]
        self.filled = g + 1
        self.pinned = None
        self.version += 1

    def past_slots(self) -> list[int]:
        return self.order[: self.filled - 1]

    def current_slot(self) -> int:
        return self.order[self.filled - 1]

    def bytes(self) -> int:
        return sum(t.values.numel() + t.scale_factors.numel() + 4 for layer in self.k + self.v for t in layer)


class CausalDiT:
    def __init__(self, cfg: DiTConfig | None = None, device="cuda", seed: int = 0, sp_group=None, sync_amax: bool = True,
                 cache_text_kv: bool = True, use_graphs: bool = False, peer_exchange: bool = True, edge_linear: str = "own",
                 ffn_requant: str = "two_pass"):
        self.cfg = cfg = cfg or DiTConfig()
        if edge_linear not in ("own", "library"):
            raise ValueError("edge_linear is 'own' (llnv_linear_bf16) or 'library' (torch.nn.functional.linear, i.e. cuBLAS)")
        if ffn_requant not in ("two_pass", "single_pass"):
            raise ValueError("ffn_requant is 'two_pass' (the reference's rounding: GEMM writes the bf16 hidden and its amax, a second "
                             "kernel quantizes it) or 'single_pass' (the GEMM epilogue quantizes with the previous forward's amax)")
        self.ffn_requant = ffn_requant
        self.edge_linear = edge_linear
        self.use_graphs = use_graphs
        self.device = torch.device(device)
        self.group = sp_group
        self.rank, self.P = sp.world(sp_group)
        self.sync_amax = sync_amax and self.P > 1
        self.cache_text_kv = cache_text_kv
        assert cfg.chunk_tokens % self.P == 0 and cfg.heads % self.P == 0, "tokens and heads must divide by the SP size"
        if cfg.chunk_tokens < 128:
            raise ValueError("a cache block (one chunk) must hold at least 128 tokens: the attention kernel decodes 128-key tiles "
                             "that may touch at most two blocks")
        gen = torch.Generator(device=self.device).manual_seed(seed)          # same weights on every rank
        self.blocks = [Block(cfg, gen, self.device) for _ in range(cfg.layers)]
        c = cfg.dim
        lin = lambda o, i: ((torch.randn(o, i, generator=gen, device=self.device) * 0.02).bfloat16(),
                            torch.zeros(o, dtype=torch.bfloat16, device=self.device))
        self.patch_w, self.patch_b = lin(c, cfg.patch_dim)
        self.time_w0, self.time_b0 = lin(c, cfg.freq_dim)
        self.time_w1, self.time_b1 = lin(c, c)
        self.tproj_w, self.tproj_b = lin(6 * c, c)
        self.text_w0, self.text_b0 = lin(c, cfg.text_dim)
        self.text_w1, self.text_b1 = lin(c, c)
        self.head_w, self.head_b = lin(cfg.patch_dim, c)
        self.head_mod = (torch.randn(1, 2, c, generator=gen, device=self.device) / math.sqrt(c)).bfloat16()

        S, Sl = cfg.chunk_tokens, cfg.chunk_tokens // self.P
        Hl = cfg.heads // self.P
        self.S, self.Sl, self.Hl, self.Cl = S, Sl, Hl, Hl * 128
        dev = self.device
        bf = lambda *shape: torch.empty(shape, dtype=torch.bfloat16, device=dev)
        self.act_c = _Act(Sl, c, dev)            # activations with `dim` columns
        # One amax scalar per (layer, producer) for the six activation amax values a block produces, so that a forward
        # clears all of them with one fill instead of one 4-byte memset per producer (llnv_set_amax_accumulate).
        self.amax_pool = torch.zeros(cfg.layers * 6, dtype=torch.float32, device=dev)
        self._amax_prezeroed = False             # True while _forward_impl runs the blocks with accumulate mode on
        self.act_f = _Act(Sl, cfg.ffn_dim, dev)  # FFN hidden
        self.act_t = _Act(cfg.text_len, c, dev)  # text context
        self.row_stats = torch.empty(2 * Sl, dtype=torch.float32, device=dev)
        self.q_buf, self.k_buf, self.v_buf = bf(Sl, c), bf(Sl, c), bf(Sl, c)
        self.q_rot, self.k_rot, self.k_smooth = bf(Sl, c), bf(Sl, c), bf(Sl, c)
        self.attn_out = bf(S, self.Cl)
        # partial results of a split or tail-balanced self-attention call (none when the call is not split)
        # (sized for every window length the cache passes through while it fills)
        with torch.cuda.device(dev):
            ws_bytes = max(ops.attention_workspace_bytes(S, n * cfg.chunk_tokens, self.Hl) for n in range(1, cfg.max_blocks + 1))
        self.attn_ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev) if ws_bytes else None
        self.arena = None
        self.check_peer_status = True         # run_chunk raises ops.DeviceTimeout when a peer barrier gave up
        if self.P > 1:
            P_, Cl_ = self.P, self.Cl
            if peer_exchange:
                # exchange targets in symmetric memory: peers store into them directly (longlive_b200/csrc/peer.cu)
                layout = {name: S * Cl_ * 2 for name in ("q_h", "kr_h", "cur_k", "cur_v", "attn_sh")}
                self.arena = sp.PeerArena.create(sp_group, dev, layout)
            if self.arena is not None:
                self.q_h, self.kr_h = self.arena.tensor("q_h", (S, Cl_)), self.arena.tensor("kr_h", (S, Cl_))
                self.cur_k, self.cur_v = self.arena.tensor("cur_k", (S, Cl_)), self.arena.tensor("cur_v", (S, Cl_))
                self.attn_sh = self.arena.tensor("attn_sh", (P_, Sl, Cl_))
            else:
                # NCCL exchange: send / receive layouts [rank][my tokens][that rank's heads] and
                # [all tokens][my heads], written and read in place by the kernels on either side
                self.q_sh, self.kr_sh, self.ks_sh, self.v_sh = bf(P_, Sl, Cl_), bf(P_, Sl, Cl_), bf(P_, Sl, Cl_), bf(P_, Sl, Cl_)
                self.q_h, self.kr_h = bf(S, Cl_), bf(S, Cl_)
                self.cur_k, self.cur_v = bf(S, Cl_), bf(S, Cl_)
                self.attn_sh = bf(P_, Sl, Cl_)
        else:
            self.cur_k, self.cur_v = bf(S, self.Cl), bf(S, self.Cl)
        self.x_a, self.x_b, self.x1, self.x2 = bf(Sl, c), bf(Sl, c), bf(Sl, c), bf(Sl, c)
        self.hidden = bf(Sl, cfg.ffn_dim)
        self.cq_buf, self.cq_n = bf(Sl, c), bf(Sl, c)
        self.ck_buf, self.cv_buf, self.ck_n = bf(cfg.text_len, c), bf(cfg.text_len, c), bf(cfg.text_len, c)
        self.cattn = bf(Sl, c)
        # The attention window is never materialised: the attention kernel decodes the NVFP4 cache blocks
        # of the layer in its load stage and reads the current chunk's smoothed keys / values from cur_k /
        # cur_v ([all chunk tokens, my heads], one pair shared by all layers; the reference dequantizes every
        # block into a bf16 window per layer and forward, causal_model.py:557-600).
        self.h_amax = torch.zeros(1, dtype=torch.float32, device=dev)
        # single-pass FFN requantization: per layer the amax the epilogue scales the hidden with (that of the layer's
        # previous forward) and the amax this forward measures
        self.ffn_amax_use = torch.zeros(cfg.layers, dtype=torch.float32, device=dev)
        self.ffn_amax_new = torch.zeros(cfg.layers, dtype=torch.float32, device=dev)
        self._ffn_calibrated = False
        self.modulation_all = torch.stack([b.modulation for b in self.blocks], 0)       # [layers, 1, 6, dim]
        self._prompts: list = []              # cached cross-attention K / V per prompt tensor, most recent last
        self._prompt_serial = 0
        self.cache = KVCache(cfg, Hl, dev)
        # static inputs of a forward (a captured graph reads these addresses on every replay)
        self.g_lat = bf(Sl, cfg.patch_dim)
        self.g_t = torch.zeros(cfg.frames_per_chunk, dtype=torch.float32, device=dev)
        self.cos_buf = torch.empty((Sl, 64), dtype=torch.float32, device=dev)
        self.sin_buf = torch.empty((Sl, 64), dtype=torch.float32, device=dev)
        self._rope_frame = None
        # temporal RoPE scale and multi-shot offset of the chunks to come (set before run_chunk; the reference passes
        # them down every forward, causal_model.py:479-486)
        self.rope_t_scale, self.rope_temporal_offset = 1.0, 0.0
        self._graphs: dict = {}
        self._scheduler = None
        self._time_cache: dict = {}
        self._graph_pool = None
        self._ran_eager = False

    # ---- helpers ----------------------------------------------------------------------------
    def _allreduce_max(self, t: torch.Tensor) -> None:
        """MAX over the group of a small fp32 tensor (per-tensor amax): through peer memory when the
        arena exists (one small kernel, no NCCL launch), else an NCCL all-reduce."""
        if self.arena is not None:
            self.arena.allreduce_max_(t)
        else:
            sp.allreduce_max_(t, self.group)

    def _gemm(self, a: _Act, rows: int, lin: _Linear, out, **epi):
        act = a
        return ops.gemm_nvfp4(act.codes, act.sf, act.amax, MSE, lin.q.values, lin.q.scale_factors, lin.q.amax, lin.q.scale_rule.cuda_id(),
                              rows, lin.out_f, lin.in_f, out=out, bias=lin.bias, **epi)

    def _quantize(self, x, act: _Act, amax_given: bool = False, have_local_amax: bool = False):
        """NVFP4-quantize x into ``act``.  ``amax_given``: act.amax already holds the final tensor
        amax.  ``have_local_amax``: act.amax holds this rank's amax of exactly the rows of x (written
        by the producing kernel's epilogue), which only needs the group reduction, if any."""
        if not amax_given:
            if self.sync_amax:
                if not have_local_amax:
                    ops.amax_bf16(x if x.dim() == 2 else x.view(-1, x.shape[-1]), act.amax)
                if self.arena is not None:
                    # the quantize kernel reduces the amax over the group itself (no separate all-reduce launch)
                    ops.quantize_nvfp4(x, MSE, act.amax, act.codes, act.sf, amax_given=True, group=self.arena)
                    return
                self._allreduce_max(act.amax)
                amax_given = True
            elif have_local_amax:
                amax_given = True
        ops.quantize_nvfp4(x, MSE, act.amax, act.codes, act.sf, amax_given=amax_given)

    def _adaln_quantize(self, x, scale, shift, act: _Act, add_one: bool = True):
        cfg = self.cfg
        kw = dict(codes=act.codes, sf=act.sf, amax=act.amax, row_stats=self.row_stats, row_offset=self.rank * self.Sl, add_one=add_one)
        if self.sync_amax and self.arena is not None:
            ops.adaln_quantize_nvfp4(x, scale, shift, cfg.frame_tokens, MSE, cfg.eps, group=self.arena, **kw)
        elif self.sync_amax:
            ops.adaln_quantize_nvfp4(x, scale, shift, cfg.frame_tokens, MSE, cfg.eps, phase=1, **kw)
            self._allreduce_max(act.amax)
            ops.adaln_quantize_nvfp4(x, scale, shift, cfg.frame_tokens, MSE, cfg.eps, phase=2, **kw)
        else:
            ops.adaln_quantize_nvfp4(x, scale, shift, cfg.frame_tokens, MSE, cfg.eps, **kw)

    def _ln_quantize(self, x, w, b, act: _Act):
        kw = dict(codes=act.codes, sf=act.sf, amax=act.amax, row_stats=self.row_stats)
        if self.sync_amax and self.arena is not None:
            ops.layernorm_quantize_nvfp4(x, w, b, MSE, self.cfg.eps, group=self.arena, **kw)
        elif self.sync_amax:
            ops.layernorm_quantize_nvfp4(x, w, b, MSE, self.cfg.eps, phase=1, **kw)
            self._allreduce_max(act.amax)
            ops.layernorm_quantize_nvfp4(x, w, b, MSE, self.cfg.eps, phase=2, **kw)
        else:
            ops.layernorm_quantize_nvfp4(x, w, b, MSE, self.cfg.eps, **kw)

    def _edge(self, x, w, b, act=None, out=None):
        """A bf16 Linear of an unquantized edge layer: the library's tcgen05 kernel, or cuBLAS through
        PyTorch (kept selectable: for these few small GEMMs cuBLAS is the faster of the two)."""
        if self.edge_linear == "own":
            return ops.linear_bf16(x, w, b, act=act, out=out)
        y = torch.nn.functional.linear(x, w, b)
        if act == "gelu_tanh":
            y = torch.nn.functional.gelu(y, approximate="tanh")
        elif act == "silu":
            y = torch.nn.functional.silu(y)
        if out is not None:
            out.copy_(y)
            return out
        return y

    # ---- text context -------------------------------------------------------------------------
    def encode_text(self, ctx_raw: torch.Tensor) -> torch.Tensor:
        """[text_len, text_dim] -> [text_len, dim] (text_embedding MLP, wan_5b/modules/causal_model.py:1568-1573)."""
        h = self._edge(ctx_raw.contiguous(), self.text_w0, self.text_b0, act="gelu_tanh")
        return self._edge(h, self.text_w1, self.text_b1).contiguous()

    MAX_PROMPTS = 4

    def _prompt(self, ctx: torch.Tensor) -> dict:
        """The cache entry of a prompt: the context tensor itself (object identity plus its in-place
        modification counter), so two prompts encoded up front never share cached K / V, and a tensor
        that was freed and whose address was reused cannot be mistaken for the old prompt (the entry
        keeps the tensor alive).  Entries carry a serial number that is part of a captured graph's key;
        when the oldest of MAX_PROMPTS entries is dropped, the graphs captured for it go with it."""
        for ent in self._prompts:
            if ent["ctx"] is ctx and ent["version"] == ctx._version:
                return ent
        self._prompt_serial += 1
        ent = {"ctx": ctx, "version": ctx._version, "serial": self._prompt_serial, "kv": [None] * self.cfg.layers}
        self._prompts.append(ent)
        while len(self._prompts) > self.MAX_PROMPTS:
            old = self._prompts.pop(0)
            self._graphs = {k: g for k, g in self._graphs.items() if k[2] != old["serial"]}
        return ent

    def _text_kv(self, layer: int, blk: Block, ctx: torch.Tensor):
        """Cross-attention K (RMS-normed) and V of the text context.  The reference recomputes them on
        every call (causal_model.py:229-235); they depend only on the prompt, so they are cached per
        prompt tensor (``_prompt``)."""
        ent = self._prompt(ctx) if self.cache_text_kv else None
        if ent is not None and ent["kv"][layer] is not None:
            return ent["kv"][layer]
        cfg = self.cfg
        if layer == 0 or not self.cache_text_kv:
            ops.quantize_nvfp4(ctx, MSE, self.act_t.amax, self.act_t.codes, self.act_t.sf, amax_given=False)
        k = self._gemm(self.act_t, cfg.text_len, blk.ck, None if self.cache_text_kv else self.ck_buf)
        v = self._gemm(self.act_t, cfg.text_len, blk.cv, None if self.cache_text_kv else self.cv_buf)
        kn, _, _ = ops.rmsnorm_rope(k, blk.cnorm_k, eps=cfg.eps, out=None if self.cache_text_kv else self.ck_n)
        if ent is not None:
            ent["kv"][layer] = (kn, v)
        return kn, v

    def _text_ready(self, ctx: torch.Tensor) -> bool:
        """True when a forward with this prompt computes no text K / V (nothing to cache, or all cached)."""
        return not self.cache_text_kv or all(kv is not None for kv in self._prompt(ctx)["kv"])

    # ---- one block ----------------------------------------------------------------------------
    def block_forward(self, li: int, x: torch.Tensor, x_out: torch.Tensor, e: torch.Tensor, ctx, cos, sin, write_cache: bool = True,
                      scales_folded: bool = False):
        """x: [Sl, dim] bf16 (my tokens); e: [F, 6, dim] (block modulation + time projection); returns x_out.
        ``write_cache=False`` leaves the current cache block unwritten (see ``run_chunk``).  ``scales_folded``: rows 1 and 4
        of ``e`` already hold bf16(1 + scale) (``_fold_scales``)."""
        cfg, blk, cache = self.cfg, self.blocks[li], self.cache
        Sl, S, ft = self.Sl, self.S, cfg.frame_tokens
        roff = self.rank * Sl
        am = self.amax_pool[li * 6:(li + 1) * 6]          # this layer's amax scalars, one per producer below
        act_amax = lambda i: am[i:i + 1]
        # -- self attention
        self.act_c.amax = act_amax(0)
        self._adaln_quantize(x, e[:, 1], e[:, 0], self.act_c, add_one=not scales_folded)
        T = cfg.chunk_tokens
        cur_k, cur_v = self.cur_k, self.cur_v
        ck, cv = cache.k[li][cache.current_slot()], cache.v[li][cache.current_slot()]
        # q, k and v projections in one grouped launch; V lands in cur_v (one GPU) or in v_buf, with its amax
        v_out = cur_v if self.P == 1 else self.v_buf
        # K / V amax of the chunk: the producers (RoPE kernel, V GEMM epilogue) write them straight into the cache block's
        # scalars, [k, v] adjacent in the cache's amax array, where a sequence-parallel group reduces them in place
        kv_amax = cache.amax_pool[li, cache.current_slot()]
        k_amax, v_am = ck.amax, cv.amax
        if blk.qkv_ok:
            a = self.act_c
            ops.gemm_nvfp4_grouped(a.codes, a.sf, a.amax, MSE, blk.qkv_codes, blk.qkv_sf, blk.qkv_amax, blk.qkv_rule.cuda_id(), Sl, cfg.dim,
                                   cfg.dim, [self.q_buf, self.k_buf, v_out], bias=blk.qkv_bias, out_amax=[None, None, v_am])
        else:
            self._gemm(self.act_c, Sl, blk.q, self.q_buf)
            self._gemm(self.act_c, Sl, blk.k, self.k_buf)
            v_am.zero_()
            self._gemm(self.act_c, Sl, blk.v, v_out, out_amax=v_am)
        if self.P == 1:
            # the tensor scales of the cache block are produced in place by the V GEMM epilogue and the RoPE kernel
            ops.rmsnorm_rope_qk(self.q_buf, blk.norm_q, [self.q_rot.data_ptr()], cfg.dim, self.k_buf, blk.norm_k, [self.k_rot.data_ptr()],
                                cfg.dim, [cur_k.data_ptr()], cfg.dim, ck.amax, cos, sin, cfg.eps)
            q_h, k_for_cache, v_for_cache = self.q_rot, self.k_rot, cur_v
        elif self.arena is not None:
            # tokens -> heads over peer memory: every producer stores each head shard at its final
            # address on the rank that owns those heads (q, rotated keys for the cache, smoothed keys
            # and values of the chunk); one barrier makes all of it visible.  The buffers are shared by
            # all layers: a rank overwrites them for the next layer only after the barrier behind this
            # layer's attention, which every rank reaches after its attention kernel has finished.
            ar, Cl = self.arena, self.Cl
            row_off = self.rank * Sl * Cl * 2                   # my token block inside an [S, Cl] buffer
            ops.rmsnorm_rope_qk(self.q_buf, blk.norm_q, ar.ptrs("q_h", row_off), Cl, self.k_buf, blk.norm_k, ar.ptrs("kr_h", row_off), Cl,
                                ar.ptrs("cur_k", row_off), Cl, k_amax, cos, sin, cfg.eps)
            ops.scatter_2d(self.v_buf, Cl * 2, ar.ptrs("cur_v", row_off), Cl * 2, Sl, Cl * 2)
            # the barrier that publishes the stores above also carries the K / V amax: its group maximum
            # is the tensor scale of every rank's cache block (and the one a single GPU would use)
            ar.allreduce_max_(kv_amax)
            q_h, k_for_cache, v_for_cache = self.q_h, self.kr_h, cur_v
        else:
            P_, grp = self.P, self.group
            # tokens -> heads with NCCL: every producer writes the send layout, every part lands where
            # its consumer reads it
            ops.rmsnorm_rope(x=self.q_buf, weight=blk.norm_q, cos=cos, sin=sin, eps=cfg.eps, out=self.q_sh, shards=P_)
            w_q = sp.exchange(self.q_sh, self.q_h, grp, async_op=True)
            ops.rmsnorm_rope(x=self.k_buf, weight=blk.norm_k, cos=cos, sin=sin, eps=cfg.eps, out=self.kr_sh, out_smooth=self.ks_sh,
                             amax_out=k_amax, shards=P_)
            w_ks = sp.exchange(self.ks_sh, cur_k, grp, async_op=True)
            w_kr = sp.exchange(self.kr_sh, self.kr_h, grp, async_op=True)
            self.v_sh.copy_(self.v_buf.view(Sl, P_, self.Cl).permute(1, 0, 2))
            w_v = sp.exchange(self.v_sh, cur_v, grp, async_op=True)
            if self.sync_amax:
                sp.allreduce_max_(kv_amax, grp)
            for w in (w_q, w_ks, w_kr, w_v):
                w.wait()
            q_h, k_for_cache, v_for_cache = self.q_h, self.kr_h, cur_v
        past = cache.past_slots()
        # The attention epilogue also produces max |out|.  Across a sequence-parallel group that is
        # the amax of (all tokens, my heads), which bounds the (my tokens, all heads) tensor quantized
        # after the exchange only once it is MAX-reduced: the peer-memory barrier after the exchange
        # does that for free; with the NCCL exchange it is used only under sync_amax.
        fused_amax = self.P == 1 or self.sync_amax or self.arena is not None
        self.act_c.amax = act_amax(1)
        ops.attention_nvfp4kv(q_h, [cache.k[li][s] for s in past], [cache.v[li][s] for s in past], T, cur_k, cur_v, self.Hl,
                              out=self.attn_out, out_amax=self.act_c.amax if fused_amax else None, workspace=self.attn_ws)
        # cache write: rotated (un-smoothed) keys and values of the chunk, straight into the slot
        if self.P == 1:
            kv_given = True
        elif self.sync_amax or self.arena is not None:
            # the producers' amax values, MAX-reduced over the group in place, are the amax of the cached tensors
            kv_given = True
        else:
            # per-rank scales: the producers saw (my tokens, all heads), the cache block holds (all tokens,
            # my heads); its own amax is taken so that no value can exceed the scale's range
            kv_given = False
        if write_cache:
            ops.quantize_nvfp4_pair(k_for_cache.reshape(S * self.Hl, 128), v_for_cache.reshape(S * self.Hl, 128), MSE, ck, cv, amax_given=kv_given)
        if self.arena is not None:
            # heads -> tokens over peer memory: rank r receives my heads of its tokens in attn_sh[my rank];
            # the quantizer reads that [source heads][my tokens] layout directly
            blk_bytes = Sl * self.Cl * 2
            ops.scatter_2d(self.attn_out, blk_bytes, self.arena.ptrs("attn_sh", self.rank * blk_bytes), self.Cl * 2, Sl, self.Cl * 2)
            self.arena.allreduce_max_(self.act_c.amax)          # barrier + group maximum of the attention output's amax
            attn = self.attn_sh
        elif self.P > 1:
            sp.exchange(self.attn_out, self.attn_sh, self.group)
            attn = self.attn_sh
        else:
            attn = self.attn_out
        self._quantize(attn, self.act_c, amax_given=self.arena is not None, have_local_amax=fused_amax)
        x1, x2 = self.x1, self.x2
        self._gemm(self.act_c, Sl, blk.o, x1, residual=x, gate=e[:, 2], frame_rows=ft, row_offset=roff)
        # -- cross attention
        self.act_c.amax = act_amax(2)
        self._ln_quantize(x1, blk.norm3_w, blk.norm3_b, self.act_c)
        self._gemm(self.act_c, Sl, blk.cq, self.cq_buf)
        ops.rmsnorm_rope(self.cq_buf, blk.cnorm_q, eps=cfg.eps, out=self.cq_n)
        kn, v = self._text_kv(li, blk, ctx)
        self.act_c.amax = act_amax(3)
        ops.attention_bf16(self.cq_n, kn, v, cfg.heads, out=self.cattn, out_amax=self.act_c.amax)
        self._quantize(self.cattn, self.act_c, have_local_amax=True)
        self._gemm(self.act_c, Sl, blk.co, x2, residual=x1)
        # -- FFN
        self.act_c.amax = act_amax(4)
        self._adaln_quantize(x2, e[:, 4], e[:, 3], self.act_c, add_one=not scales_folded)
        if self.ffn_requant == "single_pass" and self._ffn_calibrated:
            # The GEMM epilogue quantizes the GELU output itself: the 75.7 MB bf16 hidden is neither written nor re-read
            # and one launch goes away.  A quantizer needs the tensor amax before its first block; it is taken from this
            # layer's previous forward (values above it saturate as the quantizer saturates them), and this forward's
            # amax is measured for the next one.  Not the reference's rounding: 'two_pass' below is.
            use, new = self.ffn_amax_use[li:li + 1], self.ffn_amax_new[li:li + 1]
            a = self.act_c
            new.zero_()
            ops.gemm_nvfp4(a.codes, a.sf, a.amax, MSE, blk.ffn0.q.values, blk.ffn0.q.scale_factors, blk.ffn0.q.amax,
                           blk.ffn0.q.scale_rule.cuda_id(), Sl, blk.ffn0.out_f, blk.ffn0.in_f, bias=blk.ffn0.bias, act=1, out_amax=new,
                           requant=(self.act_f.codes, self.act_f.sf), requant_amax=use, store_out=False)
            f = self.act_f
            ops.gemm_nvfp4(f.codes, f.sf, use, MSE, blk.ffn2.q.values, blk.ffn2.q.scale_factors, blk.ffn2.q.amax,
                           blk.ffn2.q.scale_rule.cuda_id(), Sl, blk.ffn2.out_f, blk.ffn2.in_f, out=x_out, bias=blk.ffn2.bias, residual=x2,
                           gate=e[:, 5], frame_rows=ft, row_offset=roff)
            if self.sync_amax:
                self._allreduce_max(new)
            use.copy_(new)
            return x_out
        self.act_f.amax = act_amax(5)
        if not self._amax_prezeroed:
            self.act_f.amax.zero_()
        self._gemm(self.act_c, Sl, blk.ffn0, self.hidden, act=1, out_amax=self.act_f.amax)
        group = self.arena if self.sync_amax else None
        if self.sync_amax and group is None:
            self._allreduce_max(self.act_f.amax)
        ops.quantize_nvfp4(self.hidden, MSE, self.act_f.amax, self.act_f.codes, self.act_f.sf, amax_given=True, group=group)
        self._gemm(self.act_f, Sl, blk.ffn2, x_out, residual=x2, gate=e[:, 5], frame_rows=ft, row_offset=roff)
        if self.ffn_requant == "single_pass":
            self.ffn_amax_use[li:li + 1].copy_(self.act_f.amax)      # calibration: the first forward runs the two-pass form
        return x_out

    # ---- whole model ----------------------------------------------------------------------------
    def time_embed(self, t: torch.Tensor):
        """t: [F] timesteps -> (e [F, dim], e0 [F, 6, dim]) (causal_model.py:1561-1564)."""
        cfg = self.cfg
        half = cfg.freq_dim // 2
        freqs = torch.pow(10000.0, -torch.arange(half, device=self.device, dtype=torch.float64) / half)
        ang = t.to(torch.float64)[:, None] * freqs[None]
        emb = torch.cat([ang.cos(), ang.sin()], dim=1).to(torch.bfloat16)
        e = self._edge(self._edge(emb, self.time_w0, self.time_b0, act="silu"), self.time_w1, self.time_b1)
        e0 = self._edge(torch.nn.functional.silu(e), self.tproj_w, self.tproj_b).view(-1, 6, cfg.dim)
        return e, e0

    def _set_rope(self, start_frame: int) -> None:
        key = (start_frame, self.rope_t_scale, self.rope_temporal_offset)
        if self._rope_frame == key:
            return
        cos, sin = rope_tables(self.cfg, start_frame, self.device, self.rope_t_scale, self.rope_temporal_offset)
        lo, hi = self.rank * self.Sl, (self.rank + 1) * self.Sl
        self.cos_buf.copy_(cos[lo:hi])
        self.sin_buf.copy_(sin[lo:hi])
        self._rope_frame = key

    @staticmethod
    def _fold_scales(em: torch.Tensor) -> torch.Tensor:
        """The two adaLN scale rows of every block's modulation as bf16(1 + scale), which is what the modulation
        multiplies with (utils/adaln_triton.py:62-86 forms it per element in every call): formed once per timestep
        vector here, so that the kernels run with add_one = 0.  Shifts and gates are untouched."""
        em = em.clone()
        em[:, :, 1] = (em[:, :, 1].float() + 1.0).to(em.dtype)
        em[:, :, 4] = (em[:, :, 4].float() + 1.0).to(em.dtype)
        return em

    def _time_inputs(self, t: torch.Tensor, t_key):
        """(e, per-layer modulation) of the timesteps ``t``.  They depend on the timesteps and the weights
        only, and a video runs the same few timesteps in every chunk, so with a host-side key for ``t``
        (``t_key``, e.g. the tuple of its values) they are computed once and kept; the reference recomputes
        the time MLP and the time projection in every forward (causal_model.py:1561-1564)."""
        if t_key is None:
            e, e0 = self.time_embed(t)
            return e, self._fold_scales(self.modulation_all + e0.unsqueeze(0))     # [layers, F, 6, dim], causal_model.py:863 for every block at once
        hit = self._time_cache.get(t_key)
        if hit is None:
            if len(self._time_cache) >= 64:
                self._time_cache.clear()
                self._graphs.clear()                             # captured graphs read the dropped tensors
            e, e0 = self.time_embed(t)
            hit = self._time_cache[t_key] = (e, self._fold_scales(self.modulation_all + e0.unsqueeze(0)))
        return hit

    def forward(self, latent_tokens: torch.Tensor, t: torch.Tensor, ctx: torch.Tensor, start_frame: int, t_key=None,
                write_cache: bool = True) -> torch.Tensor:
        """latent_tokens: [Sl, patch_dim] (my token shard of the patchified chunk) -> [Sl, patch_dim].

        ``write_cache``: quantize this forward's rotated keys and values into the current cache block, as every
        forward of the reference does (causal_model.py:1644-1645).  ``run_chunk`` switches it off for the denoising
        forwards: nothing reads the current block before the chunk's clean re-cache forward overwrites it.

        With ``use_graphs`` the whole forward (about a thousand launches, the collectives included)
        is captured once per state of the KV block table and replayed afterwards: the launch sequence
        depends only on which cache slots are past / current, every other input lives at a fixed
        address.  The returned tensor is then the graph's output buffer: consume it before the next
        forward.  The first forward and the chunks that still fill the window run eagerly (one-time
        set-up such as the text K/V and the communicators must not happen inside a capture)."""
        self._set_rope(start_frame)
        if not self.use_graphs:
            return self._forward_impl(latent_tokens, t, ctx, self._time_inputs(t, t_key) if t_key is not None else None, write_cache)
        self.g_lat.copy_(latent_tokens)
        self.g_t.copy_(t)
        tin = self._time_inputs(t, t_key) if t_key is not None else None     # outside any capture: the tensors outlive the graphs
        prompt_key = self._prompt(ctx)["serial"] if self.cache_text_kv else ctx.data_ptr()
        key = (tuple(self.cache.order), self.cache.filled, prompt_key, t_key, write_cache)
        entry = self._graphs.get(key)
        if entry is None:
            # eager when one-time set-up is still due (first forward, the text K / V of a new prompt) or
            # while the window still fills: none of that may happen inside a capture
            if not self._ran_eager or self.cache.filled < self.cfg.max_blocks or not self._text_ready(ctx):
                return self._forward_impl(self.g_lat, self.g_t, ctx, tin, write_cache)
            if self._graph_pool is None:
                self._graph_pool = torch.cuda.graph_pool_handle()
            graph = torch.cuda.CUDAGraph()
            torch.cuda.synchronize(self.device)
            with torch.cuda.graph(graph, pool=self._graph_pool, capture_error_mode="thread_local"):
                out = self._forward_impl(self.g_lat, self.g_t, ctx, tin, write_cache)
            entry = self._graphs[key] = (graph, out)
        entry[0].replay()
        return entry[1]

    def close(self) -> None:
        """Drop the captured graphs.  Call this before the process group is destroyed: a communicator
        cannot be torn down while a live graph still holds its collectives."""
        self._graphs.clear()
        self._graph_pool = None

    def _forward_impl(self, latent_tokens: torch.Tensor, t: torch.Tensor, ctx: torch.Tensor, time_inputs=None,
                      write_cache: bool = True) -> torch.Tensor:
        cfg = self.cfg
        self._edge(latent_tokens, self.patch_w, self.patch_b, out=self.x_a)       # patch embedding, causal_model.py:1535-1540
        e, em_all = time_inputs if time_inputs is not None else self._time_inputs(t, None)
        cos, sin = self.cos_buf, self.sin_buf
        ran_before = self._ran_eager
        self._ran_eager = True
        cur, nxt = self.x_a, self.x_b
        # every activation amax of the forward cleared by one fill; the attention and LN-quantize entry points then
        # accumulate into their scalars instead of clearing them one by one
        self.amax_pool.zero_()
        lib = _lib.lib()
        # the V GEMM and the RoPE kernel write the amax of the cache block in place: clear the current block's scalars of
        # all layers at once as well
        self.cache.amax_pool[:, self.cache.current_slot()].zero_()
        before = lib.llnv_set_amax_accumulate(3)
        self._amax_prezeroed = True
        try:
            for li, blk in enumerate(self.blocks):
                self.block_forward(li, cur, nxt, em_all[li], ctx, cos, sin, write_cache, scales_folded=True)
                cur, nxt = nxt, cur
        finally:
            self._amax_prezeroed = False
            lib.llnv_set_amax_accumulate(before)
        if not ran_before:
            self._ffn_calibrated = True          # every layer's hidden amax is known from here on
        # head: LayerNorm, modulate with (head.modulation + e), project (CausalHead.forward, causal_model.py:950-959):
        # the same bf16 rounding points as a block's adaLN, so the quantizer's load-side transform produces y
        # (nothing is quantized: the head Linear stays bf16)
        hm = self.head_mod + e.unsqueeze(1)                             # [F, 2, dim]: shift, scale
        _, _, _, y = ops.adaln_quantize_nvfp4(cur, hm[:, 1], hm[:, 0], cfg.frame_tokens, MSE, cfg.eps, y_only=True,
                                              amax=self.h_amax, row_stats=self.row_stats, row_offset=self.rank * self.Sl)
        return self._edge(y, self.head_w, self.head_b)

    def run_chunk(self, latent_tokens: torch.Tensor, ctx: torch.Tensor, chunk_index: int,
                  sampling_steps: int = 4, timestep_shift: float = 5.0, scene_cut: bool = False,
                  clean_recache: bool = True) -> torch.Tensor:
        """One AR chunk: ``sampling_steps`` denoising forwards, each followed by a UniPC scheduler step,
        then one clean re-cache forward at timestep 0 (pipeline/causal_diffusion_inference.py:566-647;
        4 steps at shift 5 are the timesteps 999, 937, 833, 624 of configs/inference.yaml).  At a
        ``scene_cut`` the re-cache forward sees only the global sink (``clean_recache``, :621-629) and
        the chunk is pinned as the new shot sink afterwards (:659-664)."""
        cfg = self.cfg
        self.cache.begin_chunk()
        start_frame = chunk_index * cfg.frames_per_chunk
        F = cfg.frames_per_chunk
        if self._scheduler is None:
            self._scheduler = FlowUniPCMultistepScheduler(num_train_timesteps=1000, shift=1, use_dynamic_shifting=False)
        sched = self._scheduler
        sched.set_timesteps(sampling_steps, device="cpu", shift=timestep_shift)      # a new scheduler per chunk, :566, :892-899
        x_t = latent_tokens
        for t in sched.timesteps.tolist():
            tt = torch.full((F,), float(t), device=self.device)
            # the block these forwards would write is overwritten by the re-cache forward below before anything reads it
            flow = self.forward(x_t, tt, ctx, start_frame, t_key=(float(t),) * F, write_cache=False)
            x_t = sched.step(flow, t, x_t, return_dict=False)[0]
        if scene_cut and clean_recache:
            self.cache.reset_keep_global()
        self.forward(x_t, torch.zeros(F, device=self.device), ctx, start_frame, t_key=(0.0,) * F)
        if scene_cut:
            self.cache.pin_current()
        if self.arena is not None and self.check_peer_status:
            # a peer barrier that gave up (a rank that is seconds late) leaves this chunk's exchange buffers
            # undefined: find out here, once per chunk, instead of returning a wrong chunk silently
            ops.check_status(self.device)
        return x_t
