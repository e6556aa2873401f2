"""Streaming hand-off of finished chunks to the VAE side.

The reference decodes every chunk as soon as its denoising ends, on a second CUDA stream or on a
second GPU, so that the diffusion of chunk i+1 overlaps the decode of chunk i
(pipeline/causal_diffusion_inference.py:666-695: ``async_vae`` records an event and decodes on
``vae_stream``; ``pipeline_vae`` copies ``latents.permute(0, 2, 1, 3, 4).contiguous()`` to the VAE's
device and queues it).  ``LatentHandoff`` is that seam for a model that keeps its latents
patchified: ``push(tokens)`` unpatchifies the chunk straight into a slot of a ring of [C, F, H, W]
buffers (``llnv_unpatchify``, on the diffusion stream), then a side stream copies the slot to its
destination -- pinned host memory, or a buffer on another GPU -- and records an event.  The
diffusion stream never waits for a copy unless the ring is full (back-pressure: the slot about to
be overwritten must have left).  ``pop()`` returns chunks in order once their copy has finished.
"""
from __future__ import annotations

from collections import deque

import torch

from . import ops


class LatentHandoff:
    def __init__(self, channels: int, frames: int, height: int, width: int, device="cuda", target="host", depth: int = 3):
        """``height`` / ``width``: latent size (twice the token grid).  ``target``: "host" (pinned memory)
        or a ``torch.device`` / string naming another GPU."""
        if depth < 1:
            raise ValueError("depth must be at least 1")
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise ValueError("the hand-off starts on a CUDA device (there is no CPU path)")
        self.shape = (channels, frames, height, width)
        self.to_host = target == "host"
        self.target = None if self.to_host else torch.device(target)
        if not self.to_host and self.target.type != "cuda":
            raise ValueError('target is "host" or a CUDA device')
        self.stage = [torch.empty(self.shape, dtype=torch.bfloat16, device=self.device) for _ in range(depth)]
        if self.to_host:
            self.dest = [torch.empty(self.shape, dtype=torch.bfloat16).pin_memory() for _ in range(depth)]
        else:
            self.dest = [torch.empty(self.shape, dtype=torch.bfloat16, device=self.target) for _ in range(depth)]
        self.copy_stream = torch.cuda.Stream(self.device)
        self.copied = [None] * depth                      # event: the slot's copy has finished
        self.consumed = [True] * depth                    # the destination slot may be overwritten
        self.pending: deque = deque()                     # (sequence number, slot) in push order
        self.pushed = 0
        self.bytes_per_chunk = self.stage[0].numel() * 2

    def push(self, tokens: torch.Tensor) -> int:
        """Queue the chunk whose patchified latents are ``tokens`` [F*h*w, 4*C]; returns its sequence number.
        Stream-ordered after the work already queued on the current stream of the device."""
        slot = self.pushed % len(self.stage)
        if not self.consumed[slot]:
            raise RuntimeError("hand-off ring is full: pop() the oldest chunk first (its destination buffer is still owned by the consumer)")
        cur = torch.cuda.current_stream(self.device)
        if self.copied[slot] is not None:
            cur.wait_event(self.copied[slot])            # the staging slot is read by an earlier copy
        ops.unpatchify(tokens, self.stage[slot])
        ready = torch.cuda.Event()
        ready.record(cur)
        with torch.cuda.stream(self.copy_stream):
            self.copy_stream.wait_event(ready)
            self.dest[slot].copy_(self.stage[slot], non_blocking=True)
            done = torch.cuda.Event()
            done.record(self.copy_stream)
        self.copied[slot] = done
        self.consumed[slot] = False
        self.pending.append((self.pushed, slot))
        self.pushed += 1
        return self.pushed - 1

    def ready(self) -> bool:
        """True when the oldest queued chunk has arrived."""
        return bool(self.pending) and self.copied[self.pending[0][1]].query()

    def pop(self, wait: bool = True):
        """(sequence number, latent [C, F, H, W] at the destination) of the oldest queued chunk, or None
        when nothing is queued (or, with ``wait=False``, nothing has arrived yet).  The tensor is the
        ring's buffer: it is valid until ``release(sequence number)``."""
        if not self.pending or (not wait and not self.ready()):
            return None
        seq, slot = self.pending.popleft()
        self.copied[slot].synchronize()
        return seq, self.dest[slot]

    def release(self, seq: int) -> None:
        """The consumer is done with chunk ``seq``: its destination buffer may be reused."""
        self.consumed[seq % len(self.stage)] = True
