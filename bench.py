#!/usr/bin/env python
"""Benchmark of the NVFP4 hot path: the W4A4 GEMM shape sweep of one Wan2.2-5B-shaped DiT block.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (seeded synthetic tensors with the benchmark's shapes and value distributions):
q/k/v/o and cross-attention q/o 3072->3072, cross-attention k/v over 512 text tokens, FFN
3072->14336->3072, for M in {880, 2640, 10560} tokens; activations ~N(0,1) with 0.1 % entries
x20, weights ~N(0, 0.02), both quantized to NVFP4 with the 4-over-6 MSE rule.

One "step" is one pass over all 30 GEMMs of the sweep.
  value  W4A4 GEMM TFLOP/s (2*M*N*K with the logical M) with NVFP4 operands resident in HBM,
         timed with CUDA events around each step, L2 flushed between steps, max over ranks.
  e2e    the same FLOPs through the public Linear path from HOST buffers: pinned bf16
         activations -> device, quantize, GEMM + bias, result -> host, all inside the timed region.
With --gpus N every rank runs the sweep on its own token shard (tokens are sharded across
ranks for every Linear; there is no collective on this path): weak scaling.

--impl reference times the CPU restatement of the reference's dequantize-then-matmul path
(oracle/, numpy) on the host cores for the same metric, on a bounded sample of the workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

DIM, FFN, TEXT = 3072, 14336, 512
M_SWEEP = (880, 2640, 10560)


def sweep_shapes(m_values=M_SWEEP):
    """(name, M, N, K) of every GEMM of the sweep."""
    shapes = []
    for m in m_values:
        for name in ("self_attn.q", "self_attn.k", "self_attn.v", "self_attn.o", "cross_attn.q", "cross_attn.o"):
            shapes.append((name, m, DIM, DIM))
        shapes.append(("cross_attn.k", TEXT, DIM, DIM))
        shapes.append(("cross_attn.v", TEXT, DIM, DIM))
        shapes.append(("ffn.0", m, FFN, DIM))
        shapes.append(("ffn.2", m, DIM, FFN))
    return shapes


def flops_of(shapes) -> float:
    return float(sum(2.0 * m * n * k for _, m, n, k in shapes))


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200", "-i", str(self.gpu)],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self):
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, smax, reasons = [], [], set()
        try:
            for line in open(self.path):
                parts = [p.strip() for p in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    sm.append(float(parts[1]))
                    smax.append(float(parts[2]))
                except ValueError:
                    continue
                for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            # the loop is busy for most samples; use the upper half to skip idle gaps between steps
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = max(smax)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


# ---------------------------------------------------------------------------------------------
# CPU arm (oracle port): dequantize-then-fp32-matmul on the host cores
# ---------------------------------------------------------------------------------------------

def cpu_port_tflops(sample_shapes, repeats: int = 1):
    """Times oracle.fp4_matmul (the reference's PyTorch matmul backend restated in numpy) on
    pre-quantized operands; returns (TFLOP/s, seconds, description)."""
    import numpy as np

    from oracle import nvfp4_oracle as O

    rng = np.random.default_rng(0)
    ops_ = []
    for name, m, n, k in sample_shapes:
        x = rng.standard_normal((m, k), dtype=np.float32)
        x = np.where(rng.random((m, k)) < 0.001, x * 20, x).astype(np.float32)
        w = (rng.standard_normal((n, k), dtype=np.float32) * 0.02).astype(np.float32)
        # quantization of the operands is not part of the GEMM metric: use the static rule (one pass)
        ops_.append((O.quantize_nvfp4(O.bf16_round(x), "static_6"), O.quantize_nvfp4(O.bf16_round(w), "static_6"), (m, k), (n, k)))
    t0 = time.perf_counter()
    for _ in range(repeats):
        for xq, wq, xs, ws in ops_:
            O.fp4_matmul(xq, wq, xs, ws, "static_6", "static_6")
    dt = time.perf_counter() - t0
    fl = flops_of(sample_shapes) * repeats
    return fl / dt / 1e12, dt, "; ".join(f"{n} {m}x{nn}x{k}" for n, m, nn, k in sample_shapes)


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = [s for s in sweep_shapes((880,)) if s[0] in ("self_attn.q", "cross_attn.k", "ffn.0")]
    for _ in range(max(0, min(args.warmup, 1))):
        cpu_port_tflops(sample[:1])
    vals, secs = [], []
    for _ in range(max(1, min(args.steps, 5))):
        v, dt, desc = cpu_port_tflops(sample)
        vals.append(v)
        secs.append(dt)
    value = statistics.mean(vals)
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": "w4a4_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": len(vals), "warmup": min(args.warmup, 1), "ms_per_step": statistics.mean(secs) * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "nvfp4 (dequantized to f32 on the CPU)",
        "data": "synthetic",
        "config": {"workload": "DiT-block W4A4 GEMM sweep (3072/14336, M in {880,2640,10560}); CPU arm runs a bounded sample",
                   "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                         "sample": f"numpy restatement of the reference's dequantize-then-fp32-matmul backend on: {desc}"},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    import longlive_b200 as L
    from longlive_b200 import _lib, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.lib()

    shapes = sweep_shapes()
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)

    def activation(m, k):
        x = torch.randn(m, k, generator=gen, device=dev)
        mask = torch.rand(m, k, generator=gen, device=dev) < 0.001
        return torch.where(mask, x * 20, x).bfloat16()

    cfg = L.QuantizationConfig(scale_rule="mse")
    weights = {}
    for name, m, n, k in shapes:
        if (name, n, k) not in weights:
            w = (torch.randn(n, k, generator=gen, device=dev) * 0.02).bfloat16()
            weights[(name, n, k)] = (L.quantize_to_fp4(w, cfg), torch.zeros(n, dtype=torch.bfloat16, device=dev))
            del w
    acts = {}
    for name, m, n, k in shapes:
        if (m, k) not in acts:
            acts[(m, k)] = L.quantize_to_fp4(activation(m, k), cfg)
    outs = {}
    for name, m, n, k in shapes:
        if (m, n) not in outs:
            outs[(m, n)] = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def gemm_step():
        for name, m, n, k in shapes:
            xq = acts[(m, k)]
            wq, _ = weights[(name, n, k)]
            ops.gemm_nvfp4(xq.values, xq.scale_factors, xq.amax, 3, wq.values, wq.scale_factors, wq.amax, 3, m, n, k,
                           out=outs[(m, n)])

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    # The 30 launches of a step are captured once in a CUDA graph and replayed: a step is short
    # enough (about a millisecond) that launching from Python would otherwise bound it, more so
    # with several ranks sharing the host.
    gemm_step()
    torch.cuda.synchronize(dev)
    step_graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(step_graph, capture_error_mode="thread_local"):
        gemm_step()
    for _ in range(max(args.warmup, 3)):
        flush.fill_(1)
        step_graph.replay()
    sync_all()
    assert lib.llnv_check_status(None) == 0, lib.llnv_last_error()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    ends = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    sync_all()
    wall0 = time.perf_counter()
    for i in range(args.steps):
        flush.fill_(i & 0xFF)          # evict the 126 MB L2 (not timed)
        starts[i].record()
        step_graph.replay()
        ends[i].record()
    sync_all()
    wall = time.perf_counter() - wall0
    step_ms = [s.elapsed_time(e) for s, e in zip(starts, ends)]
    total_ms = sum(step_ms)
    if world > 1:
        t = torch.tensor([total_ms], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    fl_step = flops_of(shapes)
    value = fl_step * world / (ms_per_step * 1e-3) / 1e12
    assert lib.llnv_check_status(None) == 0, lib.llnv_last_error()

    # ---- end to end through the public Linear path, host buffers -------------------------------
    e2e_steps = max(1, min(args.steps, 3))
    host_in = {}
    for name, m, n, k in shapes:
        if (m, k) not in host_in:
            host_in[(m, k)] = torch.randn(m, k, dtype=torch.bfloat16).pin_memory()
    torch.cuda.current_stream(dev).synchronize()
    host_out = {}
    for name, m, n, k in shapes:
        if (m, n) not in host_out:
            host_out[(m, n)] = torch.empty(m, n, dtype=torch.bfloat16).pin_memory()
    h2d = sum(m * k * 2 for _, m, n, k in shapes)
    d2h = sum(m * n * 2 for _, m, n, k in shapes)

    # Three streams: host->device copies, quantize + GEMM, device->host copies, chained with events so
    # that the copies of neighbouring GEMMs overlap the compute (PCIe is full duplex).
    st_in, st_cmp, st_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    dev_in = [torch.empty(m, k, dtype=torch.bfloat16, device=dev) for _, m, n, k in shapes]
    dev_out = [torch.empty(m, n, dtype=torch.bfloat16, device=dev) for _, m, n, k in shapes]
    step_done = torch.cuda.Event()

    def e2e_step():
        st_in.wait_event(step_done)                    # buffers of the previous step are free again
        st_cmp.wait_event(step_done)
        for i, (name, m, n, k) in enumerate(shapes):
            with torch.cuda.stream(st_in):
                dev_in[i].copy_(host_in[(m, k)], non_blocking=True)
                ev_in = torch.cuda.Event()
                ev_in.record(st_in)
            with torch.cuda.stream(st_cmp):
                st_cmp.wait_event(ev_in)
                wq, bias = weights[(name, n, k)]
                L.fp4_matmul(L.quantize_to_fp4(dev_in[i], cfg), wq, bias=bias, out=dev_out[i])
                ev_c = torch.cuda.Event()
                ev_c.record(st_cmp)
            with torch.cuda.stream(st_out):
                st_out.wait_event(ev_c)
                host_out[(m, n)].copy_(dev_out[i], non_blocking=True)
        step_done.record(st_out)
        torch.cuda.current_stream(dev).wait_event(step_done)

    e2e_step()
    sync_all()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    sync_all()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_s], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_value = fl_step * world / e2e_s / 1e12
    clocks = sampler.stop() if rank == 0 else {}

    dit_chunk = None
    if not args.no_dit:
        del flush
        torch.cuda.empty_cache()
        grp = dist.group.WORLD if world > 1 else None
        # Sequence-parallel ranks quantize their own token shard with its own tensor scale, as the
        # reference's sequence-parallel path does (it has no amax exchange).  The variant with every
        # amax MAX-reduced over the group reproduces the 1-GPU codes bit for bit and is timed beside it.
        dit_chunk = bench_dit_chunk(dev, rank, world, grp, args.chunk_steps, sync_amax=False)
        if world > 1:
            torch.cuda.empty_cache()
            synced = bench_dit_chunk(dev, rank, world, grp, min(3, args.chunk_steps), sync_amax=True)
            dit_chunk["bit_identical_to_1gpu_amax_allreduce"] = {"value": synced["value"], "ms_per_chunk": synced["ms_per_chunk"]}
        torch.cuda.empty_cache()
        eager = bench_dit_chunk(dev, rank, world, grp, min(3, args.chunk_steps), sync_amax=False, use_graphs=False)
        dit_chunk["eager_launches"] = {"value": eager["value"], "ms_per_chunk": eager["ms_per_chunk"]}

    if rank == 0:
        peaks = load_peaks()
        fp4_peak = 4.0 * peaks["bf16_tflops"]
        per_gpu = value / world
        line = {
            "metric": "w4a4_gemm_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "nvfp4 (e2m1 x ue4m3 block scale, f32 accumulate, bf16 out)", "data": "synthetic",
            "config": {"workload": "DiT-block W4A4 GEMM sweep: q/k/v/o + cross q/o 3072x3072, cross k/v M=512, FFN 3072<->14336; "
                                   "M in {880,2640,10560}; 30 GEMMs per step",
                       "flops_per_step": fl_step, "l2": "flushed between timed steps (256 MiB write)",
                       "launches": "the 30 GEMM launches of a step replayed as one CUDA graph",
                       "parallelism": f"tokens sharded over {world} rank(s), no collective"},
            "clocks": clocks,
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": e2e_s * 1e3},
            "gpu_launches": len(shapes) * args.steps,
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": fp4_peak, "unit": "TFLOP/s",
                         "frac": per_gpu / fp4_peak,
                         "traffic": 51.3e6, "traffic_case": "dram read+write of one captured launch, M=2640 N=14336 K=3072 "
                                                            "(profiles/gemm_nvfp4_kernel__2640x14336x3072.md); algorithmic "
                                                            "operand+output bytes of that launch: 105 MB, of which 52 MB of output "
                                                            "stay dirty in L2",
                         "peak_note": f"4 x {peaks['source']} dense bf16 burst peak ({peaks['bf16_tflops']} TFLOP/s); "
                                      "no FP4 entry is measured; nominal dense FP4 is 9000",
                         "kernel": "gemm_nvfp4_kernel", "frac_of_nominal_9pf": per_gpu / 9000.0},
            "wall_s_timed_region": wall,
        }
        if dit_chunk is not None:
            line["dit_chunk"] = dit_chunk
        if world == 1 and not args.no_cpu_baseline:
            sample = [s for s in sweep_shapes((880,)) if s[0] in ("self_attn.q", "cross_attn.k", "ffn.0")]
            v, dt, desc = cpu_port_tflops(sample, repeats=8)
            line["cpu_baseline"] = {"value": v, "unit": "TFLOP/s", "cores": os.cpu_count() or 1, "kind": "port",
                                    "sample": f"numpy restatement of the reference's dequantize-then-fp32-matmul backend, "
                                              f"{dt:.1f} s for 8 passes over: {desc}"}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def bench_dit_chunk(dev, rank, world, group, steps: int, sync_amax: bool = True, use_graphs: bool = True):
    """Second headline of the benchmark: one AR chunk (3 latent frames, 4 denoising forwards + 1
    clean re-cache forward) of the 30-layer random-init Wan2.2-5B-shaped causal DiT with NVFP4
    W4A4 linears and the NVFP4 KV cache in steady state (full 15-frame window).  With N > 1 ranks
    the chunk is sequence-parallel over the N GPUs (tokens sharded, heads sharded inside
    self-attention, NCCL all-to-all at the attention boundary): strong scaling.  DiT only (no T5,
    no VAE); video fps = 4 * 3 latent frames / chunk time."""
    import torch
    import torch.distributed as dist

    from longlive_b200 import _lib, dit

    cfg = dit.DiTConfig()
    model = dit.CausalDiT(cfg, device=dev, seed=0, sp_group=group, sync_amax=sync_amax, use_graphs=use_graphs,
                          edge_linear=os.environ.get("LLNV_EDGE_LINEAR", "own"))
    gen = torch.Generator(device=dev).manual_seed(7)
    ctx = model.encode_text(torch.randn(cfg.text_len, cfg.text_dim, generator=gen, device=dev).bfloat16())
    lat_full = torch.randn(cfg.chunk_tokens, cfg.patch_dim, generator=gen, device=dev).bfloat16()
    sl = cfg.chunk_tokens // world
    lat = lat_full[rank * sl:(rank + 1) * sl].contiguous()
    chunk = 0
    # fill the window, then one full period of the rolling block table (each of its states is
    # captured as a CUDA graph on first use; the timed chunks below are replays)
    period = cfg.max_blocks - cfg.sink_frames // cfg.frames_per_chunk
    for _ in range(cfg.max_blocks + period):
        model.run_chunk(lat, ctx, chunk)
        chunk += 1
    torch.cuda.synchronize(dev)
    if world > 1:
        dist.barrier()
    # every finished chunk leaves through the streaming hand-off (unpatchify into a ring slot, copy to
    # pinned host memory on a side stream); with token shards each rank would hand off a partial image
    handoff = None
    if world == 1:
        from longlive_b200.handoff import LatentHandoff
        handoff = LatentHandoff(cfg.in_channels, cfg.frames_per_chunk, 2 * cfg.grid_h, 2 * cfg.grid_w, device=dev, target="host", depth=3)
    times = []
    for _ in range(steps):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        out = model.run_chunk(lat, ctx, chunk)
        if handoff is not None:
            handoff.push(out)
        e.record()
        torch.cuda.synchronize(dev)
        times.append(s.elapsed_time(e))
        if handoff is not None:
            seq, _host_latent = handoff.pop()
            handoff.release(seq)
        chunk += 1
    assert _lib.lib().llnv_check_status(None) == 0, _lib.lib().llnv_last_error()
    exchange = "producer kernels store into peer memory (NVLink), own barrier" if model.arena is not None else "NCCL all-to-all"
    model.close()
    ts = sorted(times)
    stats = [statistics.median(times), ts[int(0.1 * (len(ts) - 1))], ts[int(round(0.9 * (len(ts) - 1)))]]
    if world > 1:
        t = torch.tensor(stats, dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        stats = [float(v) for v in t.tolist()]
    ms = stats[0]
    # bytes every rank stores into other ranks' memory per chunk: q, rotated k, smoothed k, v and the
    # attention output, each [2640 / P tokens, 3072 channels] bf16 per block and forward, (P - 1) / P of it remote
    nvlink = 0 if world == 1 else int(5 * (cfg.chunk_tokens // world) * cfg.dim * 2 * (world - 1) / world) * cfg.layers * 5
    return {"metric": "dit_chunk_video_fps", "value": 12.0 / (ms * 1e-3), "unit": "frames/s", "latent_fps": 3.0 / (ms * 1e-3),
            "ms_per_chunk": ms, "ms_per_chunk_p10": stats[1], "ms_per_chunk_p90": stats[2], "chunks_timed": steps,
            "nvlink_bytes_sent_per_rank_per_chunk": nvlink, "layers": cfg.layers, "forwards_per_chunk": 5,
            "window_tokens": cfg.window_frames * cfg.frame_tokens, "chunk_tokens": cfg.chunk_tokens,
            "parallelism": f"sequence-parallel over {world} GPU(s)" if world > 1 else "single GPU",
            "amax_sync": bool(world > 1 and sync_amax), "cuda_graphs": bool(use_graphs), "scaling": "strong",
            "exchange": ("none" if world == 1 else exchange),
            "kv_cache_bytes_per_rank": model.cache.bytes(),
            "handoff": (None if handoff is None else {"target": "pinned host", "bytes_per_chunk": handoff.bytes_per_chunk, "in_timed_region": True}),
            "data": "synthetic, random-init weights"}


def run_kernel_case(spec: str, iters: int):
    """Run one kernel on one shape a few times (used for ncu captures and quick timing):
    gemm:MxNxK[:tile]   quantize:MxK[:rule]   kvdequant:BLOCKSxTOKENSxHEADS   attention:LQxLKxHEADS   ropenorm:TOKENSxHEADS
    attnkv:LQxBLOCKSxTOKENSxHEADS[:twostep]  (attention over BLOCKS NVFP4 cache blocks + one bf16 chunk; twostep = dequantize, then attend)
    linear:MxNxK  (the bf16 Linear of the edge layers)
    unipc:ELEMENTS[:f32]  (the scheduler step with order-2 corrector and predictor: 5 tensors read, 3 written)"""
    import torch

    import longlive_b200 as L
    from longlive_b200 import _lib, ops

    lib = _lib.lib()
    kind, _, rest = spec.partition(":")
    dims, _, opt = rest.partition(":")
    d = [int(v) for v in dims.split("x")]
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    gen = torch.Generator(device=dev).manual_seed(0)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    if kind == "gemm":
        m, n, k = d
        xq = L.quantize_to_fp4(torch.randn(m, k, generator=gen, device=dev).bfloat16())
        wq = L.quantize_to_fp4((torch.randn(n, k, generator=gen, device=dev) * 0.02).bfloat16())
        out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        fn = lambda: ops.gemm_nvfp4(xq.values, xq.scale_factors, xq.amax, 3, wq.values, wq.scale_factors, wq.amax, 3,
                                    m, n, k, out=out, tile=int(opt or 0))
        work, unit = 2.0 * m * n * k / 1e12, "TFLOP/s"
    elif kind == "quantize":
        m, k = d
        x = torch.randn(m, k, generator=gen, device=dev).bfloat16()
        rule = L.ScaleRule(opt or "mse").cuda_id()
        mp = ops.padded_rows(m)
        codes = torch.empty(mp, k // 2, dtype=torch.uint8, device=dev)
        sf = torch.empty(mp * k // 16, dtype=torch.float8_e4m3fn, device=dev)
        amax = torch.empty(1, dtype=torch.float32, device=dev)
        fn = lambda: ops.quantize_nvfp4(x, rule, amax, codes, sf, amax_given=False)
        work, unit = 2.5625 * m * k / 1e9, "GB/s"
    elif kind == "kvdequant":
        blocks, tokens, heads = d
        qs = [L.quantize_to_fp4(torch.randn(tokens * heads, 128, generator=gen, device=dev).bfloat16()) for _ in range(blocks)]
        out = torch.empty(1, blocks * tokens, heads, 128, dtype=torch.bfloat16, device=dev)
        fn = lambda: L.dequantize_kv_cache(qs, blocks, heads, tokens, torch.bfloat16, dev, out=out)
        work, unit = blocks * tokens * heads * 128 * (0.5 + 1 / 16 + 2) / 1e9, "GB/s"
    elif kind == "attention":
        lq, lk, heads = d
        q = torch.randn(lq, heads * 128, generator=gen, device=dev).bfloat16()
        k = torch.randn(lk, heads * 128, generator=gen, device=dev).bfloat16()
        v = torch.randn(lk, heads * 128, generator=gen, device=dev).bfloat16()
        out = torch.empty_like(q)
        fn = lambda: ops.attention_bf16(q, k, v, heads, out=out)
        work, unit = 4.0 * lq * lk * heads * 128 / 1e12, "TFLOP/s"
    elif kind == "attnkv":
        # chunk attention reading the NVFP4 cache: LQ queries, BLOCKS cached blocks of TOKENS tokens + a bf16 chunk of TOKENS
        lq, blocks, tokens, heads = d
        kq = [L.quantize_to_fp4(torch.randn(tokens * heads, 128, generator=gen, device=dev).bfloat16()) for _ in range(blocks)]
        vq = [L.quantize_to_fp4(torch.randn(tokens * heads, 128, generator=gen, device=dev).bfloat16()) for _ in range(blocks)]
        q = torch.randn(lq, heads * 128, generator=gen, device=dev).bfloat16()
        kc = torch.randn(tokens, heads * 128, generator=gen, device=dev).bfloat16()
        vc = torch.randn(tokens, heads * 128, generator=gen, device=dev).bfloat16()
        out = torch.empty_like(q)
        if opt == "twostep":      # the unfused form it replaces: dequantize every block into a bf16 window, then attend
            win_k = torch.empty((blocks + 1) * tokens, heads * 128, dtype=torch.bfloat16, device=dev)
            win_v = torch.empty_like(win_k)
            win_k[blocks * tokens:] = kc
            win_v[blocks * tokens:] = vc

            def fn():
                L.dequantize_kv_cache(kq, blocks, heads, tokens, torch.bfloat16, dev, out=win_k[: blocks * tokens].view(1, -1, heads, 128))
                L.dequantize_kv_cache(vq, blocks, heads, tokens, torch.bfloat16, dev, out=win_v[: blocks * tokens].view(1, -1, heads, 128))
                ops.attention_bf16(q, win_k, win_v, heads, out=out)
        else:
            fn = lambda: ops.attention_nvfp4kv(q, kq, vq, tokens, kc, vc, heads, out=out)
        work, unit = 4.0 * lq * (blocks + 1) * tokens * heads * 128 / 1e12, "TFLOP/s"
    elif kind == "ropenorm":
        s_, heads = d
        x = torch.randn(s_, heads * 128, generator=gen, device=dev).bfloat16()
        w = torch.ones(heads * 128, device=dev).bfloat16()
        cos = torch.rand(s_, 64, generator=gen, device=dev)
        sin = torch.rand(s_, 64, generator=gen, device=dev)
        out = torch.empty_like(x)
        sm = torch.empty_like(x)
        amax = torch.empty(1, dtype=torch.float32, device=dev)
        fn = lambda: ops.rmsnorm_rope(x, w, cos, sin, out=out, out_smooth=sm, amax_out=amax)
        work, unit = s_ * heads * 128 * 6 / 1e9, "GB/s"
    elif kind == "linear":
        m, n, k = d
        x = torch.randn(m, k, generator=gen, device=dev).bfloat16()
        w = (torch.randn(n, k, generator=gen, device=dev) * 0.02).bfloat16()
        b = torch.randn(n, generator=gen, device=dev).bfloat16()
        out = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
        fn = lambda: ops.linear_bf16(x, w, b, out=out)
        work, unit = 2.0 * m * n * k / 1e12, "TFLOP/s"
    elif kind == "unipc":
        import ctypes
        from longlive_b200.scheduler import FlowUniPCMultistepScheduler
        n, = d
        dt = torch.float32 if opt == "f32" else torch.bfloat16
        sched = FlowUniPCMultistepScheduler(num_train_timesteps=1000, shift=1, use_dynamic_shifting=False)
        sched.set_timesteps(4, device="cpu", shift=5.0)
        coef = sched.coefficients(2, dt)
        t8 = [torch.randn(n, generator=gen, device=dev).to(dt) for _ in range(8)]
        stream = torch.cuda.current_stream().cuda_stream
        fn = lambda: _lib.check(lib.llnv_unipc_step(*[t.data_ptr() for t in t8], n, 0 if dt == torch.bfloat16 else 1,
                                                    ctypes.byref(coef), stream))
        work, unit = 8.0 * n * t8[0].element_size() / 1e9, "GB/s"
    else:
        raise SystemExit(f"unknown kernel case {spec}")
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    times = []
    for i in range(iters):
        flush.fill_(i)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        times.append(s.elapsed_time(e))
    assert lib.llnv_check_status(None) == 0, lib.llnv_last_error()
    med = statistics.median(times)
    print(json.dumps({"kernel_case": spec, "iters": iters, "median_us": med * 1e3, "min_us": min(times) * 1e3,
                      "rate": work / (med * 1e-3), "unit": unit}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel-case", default=None, help="run one kernel case instead of the benchmark (see run_kernel_case)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-dit", action="store_true", help="skip the 30-layer DiT chunk measurement")
    ap.add_argument("--chunk-steps", type=int, default=8, help="AR chunks timed for the dit_chunk figure (two periods of the rolling block table)")
    args = ap.parse_args()
    if args.kernel_case:
        run_kernel_case(args.kernel_case, args.iters)
        return
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
