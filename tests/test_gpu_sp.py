"""Sequence parallelism on real GPUs (needs >= 2): a token/head-sharded run of the DiT block stack
must reproduce the single-GPU result bit for bit when the per-tensor amax values are MAX-reduced
(all per-token kernels see the same rows, attention sees the same heads, quantizers the same scale)."""
import os
import socket
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CFG = dict(dim=512, ffn_dim=1024, heads=4, layers=2, text_len=128, text_dim=64, freq_dim=32, grid_h=4, grid_w=6,
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
        torch.cuda.synchronize()
        par.close()
        q.put((rank, "ok" if ok else "mismatch"))
    except Exception as exc:  # pragma: no cover
        import traceback
        q.put((rank, traceback.format_exc()[-1500:]))
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
@pytest.mark.parametrize("use_graphs,peer", [(False, False), (True, False), (False, True), (True, True)])
def test_sequence_parallel_matches_single_gpu(use_graphs, peer):
    """peer=False exchanges with NCCL all-to-alls, peer=True with stores into the other GPU's
    symmetric memory and the library's own barrier."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, use_graphs, peer)) for r in range(2)]
    for p in procs:
        p.start()
    results = sorted(q.get(timeout=600) for _ in procs)
    for p in procs:
        p.join(timeout=60)
        if p.is_alive():
            p.kill()
    assert results == [(0, "ok"), (1, "ok")], results
