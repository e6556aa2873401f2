"""Sequence parallelism on real GPUs (2, 4 or 8 of them): a token/head-sharded run of the DiT block stack
must reproduce the single-GPU result bit for bit when the per-tensor amax values are MAX-reduced
(all per-token kernels see the same rows, attention sees the same heads, quantizers the same scale).
Plus, on one GPU, the give-up path of the peer barrier's bounded wait."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

# 8 heads and 144 chunk tokens divide by every world size tested; cache blocks hold >= 128 tokens
CFG = dict(dim=1024, ffn_dim=1024, heads=8, layers=2, text_len=128, text_dim=64, freq_dim=32, grid_h=6, grid_w=8,
           frames_per_chunk=3, window_frames=9, sink_frames=3, in_channels=4)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q, use_graphs=False, peer=False):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from longlive_b200 import dit
        cfg = dit.DiTConfig(**CFG)
        par = dit.CausalDiT(cfg, device=dev, seed=4, sp_group=dist.group.WORLD, sync_amax=True, use_graphs=use_graphs, peer_exchange=peer)
        assert (par.arena is not None) == peer
        ref = dit.CausalDiT(cfg, device=dev, seed=4)
        g = torch.Generator(device=dev).manual_seed(9)
        ctx_raw = torch.randn(cfg.text_len, cfg.text_dim, generator=g, device=dev).bfloat16()
        ctx_p, ctx_r = par.encode_text(ctx_raw), ref.encode_text(ctx_raw)
        sl = cfg.chunk_tokens // world
        ok = True
        for chunk in range(6 if use_graphs else 4):
            lat = torch.randn(cfg.chunk_tokens, cfg.patch_dim, generator=g, device=dev).bfloat16()
            out_r = ref.run_chunk(lat, ctx_r, chunk)
            out_p = par.run_chunk(lat[rank * sl:(rank + 1) * sl].contiguous(), ctx_p, chunk)
            ok = ok and torch.equal(out_p, out_r[rank * sl:(rank + 1) * sl])
            flow_r = ref.forward(lat, torch.full((3,), 500.0, device=dev), ctx_r, chunk * 3)
            flow_p = par.forward(lat[rank * sl:(rank + 1) * sl].contiguous(), torch.full((3,), 500.0, device=dev), ctx_p, chunk * 3)
            ok = ok and torch.equal(flow_p, flow_r[rank * sl:(rank + 1) * sl])
        # head-sharded cache block of the last chunk equals the matching head slice of the full cache
        hl = cfg.heads // world
        cur_r, cur_p = ref.cache.current_slot(), par.cache.current_slot()
        kr = ref.cache.k[0][cur_r].dequantize(torch.float32).view(cfg.chunk_tokens, cfg.heads, 128)
        kp = par.cache.k[0][cur_p].dequantize(torch.float32).view(cfg.chunk_tokens, hl, 128)
        ok = ok and torch.equal(kp, kr[:, rank * hl:(rank + 1) * hl])
        if use_graphs:
            ok = ok and len(par._graphs) == 12     # 2 table states x (5 timesteps of a chunk + the extra forward)
        from longlive_b200 import ops
        ops.check_status(dev)                      # no bounded wait gave up on this rank
        torch.cuda.synchronize()
        par.close()
        q.put((rank, "ok" if ok else "mismatch"))
    except Exception as exc:  # pragma: no cover
        import traceback
        q.put((rank, traceback.format_exc()[-1500:]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("use_graphs,peer", [(False, False), (True, False), (False, True), (True, True)])
def test_sequence_parallel_matches_single_gpu(use_graphs, peer, world):
    """peer=False exchanges with NCCL all-to-alls, peer=True with stores into the other GPU's
    symmetric memory and the library's own barrier."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, use_graphs, peer)) for r in range(world)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=600) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.kill()
    assert results == [(r, "ok") for r in range(world)], results


def test_peer_barrier_gives_up_and_reports_timeout():
    """The bounded wait of the peer barrier, on one GPU: the barrier is launched as rank 0 of a world of two whose
    second signal area nobody writes, with a short poll limit.  The kernel must return by itself, llnv_check_status
    must report the timeout (code 3, where 700) once and clear it, and the context must stay usable."""
    from longlive_b200 import _lib, ops
    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    mine = torch.zeros(64, dtype=torch.int32, device=dev)          # rank 0's signal area (flag r written by rank r)
    theirs = torch.zeros(64, dtype=torch.int32, device=dev)        # stands for rank 1's area; nobody plays rank 1
    epoch = torch.zeros(1, dtype=torch.int32, device=dev)
    ops.check_status(dev)
    lib.llnv_set_peer_poll_limit(20000)
    try:
        ops.peer_barrier([mine.data_ptr(), theirs.data_ptr()], 0, epoch)
        with pytest.raises(ops.DeviceTimeout, match="code=3 where=700"):
            ops.check_status(dev)
        ops.check_status(dev)                                      # reported once, then clear
        assert int(epoch.item()) == 1 and int(theirs[0].item()) == 1 and int(mine[0].item()) == 1
        vals = torch.tensor([1.0, 2.0], device=dev)
        slots = torch.zeros(2 * 8 * 32, dtype=torch.float32, device=dev)
        ops.peer_allreduce_max(vals, [slots.data_ptr(), slots.data_ptr()], [mine.data_ptr(), theirs.data_ptr()], 0, epoch)
        with pytest.raises(ops.DeviceTimeout, match="code=3 where=701"):
            ops.check_status(dev)
    finally:
        lib.llnv_set_peer_poll_limit(0)
    # a world of one needs no peer and must pass
    ops.peer_barrier([mine.data_ptr()], 0, epoch)
    ops.check_status(dev)
    assert torch.equal(torch.ones(4, device=dev) * 2, torch.full((4,), 2.0, device=dev))


class _FakeArena:
    """What ``ops._group_args`` reads of a ``sp.PeerArena``, on local buffers: ``base[r]`` is rank r's area, the signal
    flags first, the value slots ``SIGNAL_BYTES`` further."""
    SIGNAL_BYTES = 256

    def __init__(self, areas, rank, epoch):
        self.base = [a.data_ptr() for a in areas]
        self.rank, self.world, self.epoch = rank, len(areas), epoch


def test_group_quantizer_on_one_gpu_with_a_played_peer_and_with_a_missing_one():
    """llnv_quantize_nvfp4_group on one GPU.  (1) World of two in which the test plays rank 1 beforehand: it stores rank 1's
    amax into rank 0's slot and raises rank 1's flag for the coming epoch, so rank 0's kernel finds the exchange complete:
    codes and scales must be those of the standalone quantizer under max(own, peer) amax, the amax scalar must hold that
    maximum afterwards, the epoch must have advanced and the CTA counter be back at zero.  (2) Nobody plays rank 1 and the
    poll limit is short: the kernel returns by itself and the status word reports the timeout (where 702)."""
    from longlive_b200 import _lib, ops
    lib = _lib.lib()
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(11)
    x = torch.randn(300, 512, generator=g, device=dev).bfloat16()
    own = x.float().abs().max().reshape(1)
    area0 = torch.zeros(256 // 4 + 2 * 8 * 32, dtype=torch.float32, device=dev)      # flags (as int32 bits) + slots
    area1 = torch.zeros_like(area0)
    epoch = torch.zeros(2, dtype=torch.int32, device=dev)
    arena = _FakeArena([area0, area1], 0, epoch)
    ops.check_status(dev)
    for peer_amax in (float(own.item()) * 2.0, float(own.item()) * 0.5):
        e = int(epoch[0].item()) + 1
        area0[64 + ((e & 1) * 8 + 1) * 32] = peer_amax                 # slot [parity][rank 1][0] of rank 0's area
        area0.view(torch.int32)[1] = e                                # rank 1's flag in rank 0's signal area
        amax = own.clone()
        codes, sf, _ = ops.quantize_nvfp4(x, 3, amax, amax_given=True, group=arena)
        torch.cuda.synchronize()
        ops.check_status(dev)
        want = torch.tensor([max(float(own.item()), peer_amax)], device=dev)
        ref_codes, ref_sf, _ = ops.quantize_nvfp4(x, 3, want.clone(), amax_given=True)
        assert torch.equal(amax, want) and torch.equal(codes, ref_codes) and torch.equal(sf.view(torch.uint8), ref_sf.view(torch.uint8))
        assert epoch.tolist() == [e, 0]
        assert int(area1.view(torch.int32)[0].item()) == e            # rank 0 raised its flag in rank 1's area ...
        assert float(area1[64 + ((e & 1) * 8 + 0) * 32].item()) == float(own.item())     # ... after publishing its value there
    lib.llnv_set_peer_poll_limit(20000)
    try:
        amax = own.clone()
        ops.quantize_nvfp4(x, 3, amax, amax_given=True, group=arena)
        with pytest.raises(ops.DeviceTimeout, match="code=3 where=702"):
            ops.check_status(dev)
        ops.check_status(dev)
    finally:
        lib.llnv_set_peer_poll_limit(0)
