"""Sequence-parallel exchange helpers on CPU ranks (gloo, world size 2): layouts of the two
all-to-alls, the packed variant, the amax reduction and the final gather."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from longlive_b200 import sp
        S, H, D = 12, 4, 8
        C = H * D
        full = torch.arange(S * C, dtype=torch.float32).view(S, C)
        sl = S // world
        mine = full[rank * sl:(rank + 1) * sl].contiguous()
        g = dist.group.WORLD
        heads = sp.seq_to_head(mine, g)                       # all tokens, my heads
        cl = C // world
        assert torch.equal(heads, full[:, rank * cl:(rank + 1) * cl])
        back = sp.head_to_seq(heads, g)
        assert torch.equal(back, mine)
        a, b = sp.seq_to_head_many([mine, mine * 2], g)
        assert torch.equal(a, heads) and torch.equal(b, heads * 2)
        # copy-free form: the send buffer is already [destination][my tokens][its heads]
        send = mine.view(sl, world, cl).permute(1, 0, 2).contiguous()
        recv = torch.empty(S, cl)
        sp.exchange(send, recv, g)
        assert torch.equal(recv, heads)
        back_sh = torch.empty(world, sl, cl)                  # [source heads][my tokens]
        sp.exchange(heads, back_sh, g)
        assert torch.equal(back_sh.permute(1, 0, 2).reshape(sl, C), mine)
        am = torch.tensor([float(rank + 1)])
        sp.allreduce_max_(am, g)
        assert float(am) == float(world)
        assert torch.equal(sp.all_gather_tokens(mine, g), full)
        q.put((rank, "ok"))
    except Exception as exc:  # pragma: no cover
        q.put((rank, repr(exc)))
    finally:
        dist.destroy_process_group()


def test_sp_exchange_world2():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_sp_identity_without_group():
    sys.path.insert(0, ROOT)
    from longlive_b200 import sp
    x = torch.randn(6, 16)
    assert sp.seq_to_head(x, None) is x and sp.head_to_seq(x, None) is x
    assert sp.world(None) == (0, 1)
