"""Sequence-parallel exchange steps of the chunk attention (tokens <-> heads).

Outside attention every rank holds a contiguous shard of the chunk's tokens with all channels;
inside attention it holds all tokens of ``heads / P`` heads.  The two all-to-alls are the only
data-path collectives of the hot path (the reference's ``ulysses_seq_to_head`` /
``ulysses_head_to_seq``, wan_5b/distributed/sp_ulysses_inference.py:122-154); a one-float
MAX all-reduce keeps per-tensor NVFP4 scales identical to the single-GPU run.

Pure ``torch.distributed`` (NCCL on GPUs, gloo in the CPU tests); with ``group=None`` or a world
of one rank every function is the identity.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def world(group) -> tuple[int, int]:
    if group is None or not dist.is_initialized():
        return 0, 1
    return dist.get_rank(group), dist.get_world_size(group)


def seq_to_head(x: torch.Tensor, group, out: torch.Tensor | None = None) -> torch.Tensor:
    """[S/P, C] (my tokens, all heads) -> [S, C/P] (all tokens, my heads); token order is global."""
    rank, p = world(group)
    if p == 1:
        return x
    sl, c = x.shape
    send = x.view(sl, p, c // p).permute(1, 0, 2).contiguous()          # [dest rank][token][my-head channels]
    recv = out if out is not None else torch.empty((p * sl, c // p), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(recv.view(p, sl, c // p), send, group=group)
    return recv


def head_to_seq(x: torch.Tensor, group, out: torch.Tensor | None = None) -> torch.Tensor:
    """[S, C/P] (all tokens, my heads) -> [S/P, C] (my tokens, all heads)."""
    rank, p = world(group)
    if p == 1:
        return x
    s, cl = x.shape
    sl = s // p
    recv = torch.empty((p, sl, cl), dtype=x.dtype, device=x.device)
    dist.all_to_all_single(recv, x.view(p, sl, cl).contiguous(), group=group)
    res = recv.permute(1, 0, 2).reshape(sl, p * cl)
    if out is not None:
        out.copy_(res)
        return out
    return res.contiguous()


def seq_to_head_many(tensors, group):
    """One all-to-all for several [S/P, C] tensors (q, k, v ... packed along a leading axis)."""
    rank, p = world(group)
    if p == 1:
        return list(tensors)
    n = len(tensors)
    sl, c = tensors[0].shape
    send = torch.stack([t.view(sl, p, c // p) for t in tensors], 0).permute(2, 0, 1, 3).contiguous()   # [P][n][sl][c/p]
    recv = torch.empty_like(send)
    dist.all_to_all_single(recv, send, group=group)
    # recv[src][i] holds tokens of rank src for tensor i -> [n][P*sl][c/p]
    recv = recv.permute(1, 0, 2, 3).reshape(n, p * sl, c // p)
    return [recv[i] for i in range(n)]


def exchange(send: torch.Tensor, recv: torch.Tensor, group, async_op: bool = False):
    """One all-to-all of equal contiguous parts: part r of ``send`` goes to rank r, part s of ``recv``
    comes from rank s.  With ``send`` = [P][S/P][C/P] (my tokens, destination's heads) ``recv`` is
    [S][C/P] in global token order (tokens -> heads); with ``send`` = [S][C/P] viewed as P token
    ranges ``recv`` is [P][S/P][C/P] (source's heads, my tokens).  Neither side needs a pack or
    unpack copy: the producers write and the consumers read these layouts directly."""
    rank, p = world(group)
    assert send.is_contiguous() and recv.is_contiguous() and send.numel() == recv.numel()
    return dist.all_to_all_single(recv.view(p, -1), send.view(p, -1), group=group, async_op=async_op)


def allreduce_max_(t: torch.Tensor, group) -> torch.Tensor:
    """In-place MAX all-reduce of a small fp32 tensor (per-tensor amax values)."""
    rank, p = world(group)
    if p > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return t


def all_gather_tokens(x: torch.Tensor, group) -> torch.Tensor:
    """[S/P, C] -> [S, C] (final gather of the head output, sp_ulysses_inference.py:94-112)."""
    rank, p = world(group)
    if p == 1:
        return x
    out = torch.empty((p * x.shape[0], x.shape[1]), dtype=x.dtype, device=x.device)
    dist.all_gather_into_tensor(out, x.contiguous(), group=group)
    return out
