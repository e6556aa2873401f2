"""Block-table bookkeeping of the KV cache (no GPU): rolling, the pinned shot sink of a scene cut and the
clean re-cache reset, against a token-index model of the reference's cache arithmetic."""
import random

import pytest
import torch

from longlive_b200.dit import DiTConfig, KVCache


def _cfg(window_chunks=5, sink_chunks=1, global_chunks=0):
    return DiTConfig(dim=128, ffn_dim=256, heads=1, layers=1, text_len=8, text_dim=16, freq_dim=16, grid_h=2, grid_w=2,
                     frames_per_chunk=3, window_frames=3 * window_chunks, sink_frames=3 * sink_chunks,
                     global_sink_frames=3 * global_chunks, in_channels=4)


class TokenIndexModel:
    """The reference's bookkeeping in token indices (wan_5b/modules/causal_model.py:490-534, 596-625,
    1443-1446; pipeline/causal_diffusion_inference.py:1026-1052), on a buffer of chunk ids: one list
    entry per token block, ``local_end`` / ``pinned_start`` / ``pinned_len`` counted in tokens."""

    def __init__(self, cfg):
        self.blk = cfg.chunk_tokens
        self.size = cfg.max_blocks * self.blk
        self.sink = cfg.sink_frames * cfg.frame_tokens
        self.glob = cfg.global_sink_frames * cfg.frame_tokens
        self.sink_size_tokens = cfg.sink_frames * cfg.frame_tokens
        self.buf = [None] * cfg.max_blocks
        self.local_end = 0
        self.pinned_start, self.pinned_len = -1, 0

    def effective_sink(self):
        has = self.pinned_start >= 0 and self.pinned_len > 0
        if has and self.pinned_start == self.glob:
            return self.glob + self.pinned_len
        return self.glob if has else max(self.glob, self.sink)

    def insert(self, chunk_id):
        n = self.blk
        if self.local_end + n > self.size:                           # roll_and_insert
            eff = self.effective_sink()
            evicted = self.local_end + n - self.size
            rolled = self.local_end - evicted - eff
            tokens = [c for c in self.buf for _ in range(self.blk)]
            tokens[eff:eff + rolled] = tokens[eff + evicted:eff + evicted + rolled]
            self.buf = tokens[::self.blk]
            if self.pinned_start >= 0 and self.pinned_len > 0 and self.pinned_start >= eff:
                self.pinned_start -= evicted
            self.local_end -= evicted
        self.buf[self.local_end // n] = chunk_id
        self.local_end += n

    def pin_current(self):
        self.pinned_len = min(self.sink_size_tokens, self.blk)
        self.pinned_start = self.local_end - self.blk

    def zero_kv(self):
        self.local_end = self.glob
        self.pinned_start, self.pinned_len = -1, 0

    def chunks(self):
        return self.buf[: self.local_end // self.blk]

    def pinned_chunk(self):
        return None if self.pinned_start < 0 else self.buf[self.pinned_start // self.blk]


def _table_chunks(cache, content):
    return [content[s] for s in cache.order[: cache.filled]]


@pytest.mark.parametrize("window,sink,glob", [(5, 1, 0), (5, 1, 1), (3, 1, 0), (6, 2, 1), (4, 0, 0)])
@pytest.mark.parametrize("seed", [0, 1, 2])
def test_table_follows_the_token_index_model(window, sink, glob, seed):
    """Random videos with scene cuts (with and without clean re-cache): after every chunk the table
    lists the same chunks in the same order as the reference's buffer, and pins the same chunk."""
    cfg = _cfg(window, sink, glob)
    if sink == 0:
        cfg.sink_frames = 0
    cache = KVCache(cfg, 1, torch.device("cpu"))
    model = TokenIndexModel(cfg)
    rng = random.Random(seed)
    content = {}
    for chunk in range(40):
        cut = chunk > glob and rng.random() < 0.2 and sink > 0
        clean = rng.random() < 0.5
        # denoising forwards + recache forward of the reference all write the chunk at the same place
        cache.begin_chunk()
        content[cache.current_slot()] = chunk
        model.insert(chunk)
        if cut and clean:
            cache.reset_keep_global()
            content[cache.current_slot()] = chunk
            model.zero_kv()
            model.insert(chunk)
        if cut:
            cache.pin_current()
            model.pin_current()
        assert _table_chunks(cache, content) == model.chunks(), (chunk, cut, clean)
        assert (None if cache.pinned is None else content[cache.pinned]) == model.pinned_chunk()
        assert sorted(cache.order) == list(range(cfg.max_blocks))             # a permutation: no slot lost or doubled
        assert cache.current_slot() == cache.order[cache.filled - 1]


def test_pinned_chunk_replaces_the_sink():
    cfg = _cfg(4, 1, 0)
    cache = KVCache(cfg, 1, torch.device("cpu"))
    content = {}
    for chunk in range(6):
        cache.begin_chunk()
        content[cache.current_slot()] = chunk
    assert _table_chunks(cache, content) == [0, 3, 4, 5]                      # chunk 0 is the sink
    cache.pin_current()                                                       # scene cut at chunk 5
    seen = []
    for chunk in range(6, 10):
        cache.begin_chunk()
        content[cache.current_slot()] = chunk
        seen.append(_table_chunks(cache, content))
    assert seen == [[3, 4, 5, 6], [4, 5, 6, 7], [5, 6, 7, 8], [5, 7, 8, 9]]   # the old sink goes first, then 5 is kept


def test_versions_and_errors():
    cfg = _cfg(3, 1, 1)
    cache = KVCache(cfg, 1, torch.device("cpu"))
    cache.begin_chunk()
    with pytest.raises(RuntimeError):
        cache.reset_keep_global()                                             # the only chunk is the global sink
    cache.begin_chunk()
    v = cache.version
    cache.reset_keep_global()
    assert cache.version == v + 1 and cache.filled == 2 and cache.pinned is None
    with pytest.raises(ValueError):
        KVCache(DiTConfig(dim=128, ffn_dim=256, heads=1, layers=1, grid_h=2, grid_w=2, frames_per_chunk=3, window_frames=9,
                          sink_frames=2, in_channels=4), 1, torch.device("cpu"))


def test_block_amax_scalars_are_views_of_one_array():
    """Every cache block's tensor amax lives in KVCache.amax_pool[layer, slot, K / V]: writing a block's scalar shows in the
    array, and clearing one slot column of the array clears exactly that slot's K and V scalars of every layer (what a
    forward does with one fill before the producers accumulate into them)."""
    cfg = DiTConfig(dim=256, ffn_dim=256, heads=2, layers=3, text_len=128, grid_h=6, grid_w=8, frames_per_chunk=3, window_frames=9,
                    sink_frames=3, in_channels=4)
    cache = KVCache(cfg, local_heads=2, device="cpu")
    assert tuple(cache.amax_pool.shape) == (3, 3, 2)
    for layer in range(3):
        for slot in range(3):
            cache.k[layer][slot].amax.fill_(10 * layer + slot + 0.25)
            cache.v[layer][slot].amax.fill_(10 * layer + slot + 0.5)
            assert cache.k[layer][slot].amax.shape == (1,) and cache.v[layer][slot].amax.shape == (1,)
    assert float(cache.amax_pool[2, 1, 0]) == 21.25 and float(cache.amax_pool[1, 2, 1]) == 12.5
    cache.amax_pool[:, 1].zero_()
    for layer in range(3):
        assert float(cache.k[layer][1].amax) == 0.0 and float(cache.v[layer][1].amax) == 0.0
        assert float(cache.k[layer][0].amax) == 10 * layer + 0.25 and float(cache.v[layer][2].amax) == 10 * layer + 2.5
    # [k, v] of one block are adjacent: the pair a sequence-parallel group reduces in place
    pair = cache.amax_pool[1, 0]
    assert pair.is_contiguous() and pair.data_ptr() == cache.k[1][0].amax.data_ptr() and pair.data_ptr() + 4 == cache.v[1][0].amax.data_ptr()


def test_fold_scales_forms_one_plus_scale_once():
    """CausalDiT._fold_scales: rows 1 and 4 of every block's modulation become bf16(1 + scale) (fp32 add, one rounding, as the
    adaLN kernel forms it per element with add_one = 1); shifts and gates are untouched and the input is not modified."""
    from longlive_b200.dit import CausalDiT
    g = torch.Generator().manual_seed(1)
    em = (torch.randn(2, 3, 6, 64, generator=g) * 0.3).bfloat16()
    keep = em.clone()
    out = CausalDiT._fold_scales(em)
    assert torch.equal(em, keep)
    for row in (1, 4):
        assert torch.equal(out[:, :, row], (keep[:, :, row].float() + 1.0).bfloat16())
    for row in (0, 2, 3, 5):
        assert torch.equal(out[:, :, row], keep[:, :, row])
