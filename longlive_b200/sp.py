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

import os

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


class PeerArena:
    """One symmetric-memory allocation per rank, mapped on every GPU of the group, from which the
    exchange buffers are carved.  ``tensor(name)`` is this rank's buffer, ``ptr(rank, name, offset)``
    the address of the same buffer on another rank, as seen from this GPU (NVLink peer mapping).
    The first 256 bytes hold the barrier flags (``llnv_peer_barrier``), the next 2 KiB the value
    slots of ``llnv_peer_allreduce_max``.

    Built on ``torch.distributed._symmetric_memory`` (plain peer mappings; NVLink multicast binding
    is switched off, nothing here uses it).  ``PeerArena.create`` returns None when symmetric
    memory cannot be set up for the group, and callers fall back to the NCCL exchange."""

    SIGNAL_BYTES = 256
    SLOT_BYTES = 2 * 8 * 32 * 4

    def __init__(self, group, device, layout: dict[str, int]):
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem
        self.group = group
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.offsets, off = {}, self.SIGNAL_BYTES + self.SLOT_BYTES
        for name, nbytes in layout.items():
            self.offsets[name] = (off, nbytes)
            off += (nbytes + 255) // 256 * 256
        self.nbytes = off
        self.buf = symm_mem.empty(off, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group.group_name)
        self.base = [int(p) for p in self.handle.buffer_ptrs]
        self.epoch = torch.zeros(2, dtype=torch.int32, device=device)      # [epoch, finished-CTA counter of the group quantizers]
        torch.cuda.synchronize(device)
        dist.barrier(group)                     # every rank's flags are zero before anyone signals

    @classmethod
    def create(cls, group, device, layout):
        try:
            return cls(group, device, layout)
        except Exception as exc:  # symmetric memory unavailable (no peer access, old driver, ...)
            import warnings
            warnings.warn(f"peer-memory exchange unavailable, using NCCL all-to-all: {exc!r}")
            return None

    def tensor(self, name: str, shape, dtype=torch.bfloat16) -> torch.Tensor:
        off, nbytes = self.offsets[name]
        t = self.buf[off:off + nbytes].view(dtype)
        return t.view(*shape)

    def ptr(self, rank: int, name: str, byte_offset: int = 0) -> int:
        return self.base[rank] + self.offsets[name][0] + byte_offset

    def ptrs(self, name: str, byte_offset: int = 0) -> list[int]:
        return [self.ptr(r, name, byte_offset) for r in range(self.world)]

    def barrier(self) -> None:
        from . import ops
        ops.peer_barrier(self.base, self.rank, self.epoch)

    def allreduce_max_(self, vals: torch.Tensor) -> torch.Tensor:
        """In-place MAX all-reduce of up to 32 fp32 values; also a barrier."""
        from . import ops
        ops.peer_allreduce_max(vals, [b + self.SIGNAL_BYTES for b in self.base], self.base, self.rank, self.epoch)
        return vals
