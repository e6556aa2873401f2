#!/usr/bin/env python
"""Benchmark of the NVFP4 hot path of the causal Wan2.2-5B-shaped DiT.

    python bench.py --gpus N --steps K --warmup W [--impl reference]
    torchrun --nproc-per-node N bench.py --gpus N ...        (N > 1: one rank per GPU)

Headline (`value`): video frames per second of the 30-layer DiT, one step = one autoregressive chunk of 3
latent frames = 4 denoising forwards + UniPC steps + 1 clean re-cache forward, NVFP4 W4A4 Linears, NVFP4 KV
cache read by the attention kernel, full 15-frame window (steady state).  N > 1 ranks run the SAME chunk
sequence-parallel (tokens sharded, heads sharded inside self-attention, one exchange per direction per layer
over NVLink): strong scaling.  With N > 1 every per-tensor amax is MAX-reduced over the group, so the ranks
compute bit for bit what one GPU computes; that is checked on the live ranks before timing (`sp_parity`).
Seeded synthetic tensors and random-init weights of the benchmark's shapes stand in for prompts and checkpoints.

  value          device-timed (CUDA events per chunk, max over ranks), inputs resident in HBM
  e2e            the same chunks driven from HOST buffers: pinned latents -> device and the finished chunk
                 -> pinned host memory inside the timed region (wall clock around synchronised chunks)
  roofline       the dominant kernel (the chunk attention, about half of a chunk) timed live with CUDA events
                 at the rank's shape; `chunk_roofline` and `gemm_sweep.roofline` are the whole-chunk and GEMM views
  gemm_sweep     the W4A4 GEMM shape sweep of one DiT block (M in {880, 2640, 10560}), per rank, no collective
  rollout        240 latent frames (80 chunks) from an empty cache: fill phase and steady state, p10/p50/p90
  cpu_baseline   the CPU restatement of the reference's fake-quant block (oracle/, numpy) timed on the host cores
                 for a bounded sample (one block, one frame of tokens) and extrapolated; N = 1 only

--impl reference times that CPU path alone, same metric and unit.
--kernel-case runs one kernel on one shape (ncu captures, quick timing).
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

DIM, FFN, TEXT, HEADS, LAYERS = 3072, 14336, 512, 24, 30
M_SWEEP = (880, 2640, 10560)
CHUNK_TOKENS, WINDOW_TOKENS, FORWARDS = 2640, 13200, 5


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


def chunk_flops():
    """Algorithmic FLOPs of one chunk in steady state: (FP4 GEMM flops, bf16 attention flops)."""
    s = CHUNK_TOKENS
    gemm = LAYERS * (6 * 2.0 * s * DIM * DIM + 2 * 2.0 * s * DIM * FFN)
    attn = LAYERS * (4.0 * s * WINDOW_TOKENS * DIM + 4.0 * s * TEXT * DIM)
    return FORWARDS * gemm, FORWARDS * attn


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return {"hbm_gbs": float(p["hbm_gbs"]), "bf16_tflops": float(p["bf16_tflops"]),
                "bf16_tflops_sustained": float(p.get("bf16_tflops_sustained", p["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


_REAL_STDOUT = None


def quiet_stdout():
    """Point file descriptor 1 at stderr for the rest of the run, so that whatever libraries print on their own (NCCL's
    version banner, for one) cannot get between the caller and the ONE JSON line; `emit` writes that line to the real stdout."""
    global _REAL_STDOUT
    if _REAL_STDOUT is None:
        sys.stdout.flush()
        _REAL_STDOUT = os.dup(1)
        os.dup2(2, 1)


def emit(line: dict) -> None:
    text = (json.dumps(line) + "\n").encode()
    if _REAL_STDOUT is None:
        sys.stdout.write(text.decode())
        sys.stdout.flush()
    else:
        sys.stdout.flush()
        os.write(_REAL_STDOUT, text)


def dram_traffic(kernel: str, shape: str):
    """DRAM read+write bytes per launch from the committed ncu summaries (profiles/dram_traffic.md: one row per
    captured kernel and shape).  None when no capture of that shape is committed."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.md")
    if not os.path.exists(path):
        return None
    for line in open(path):
        cells = [c.strip() for c in line.strip().strip("|").split("|")]
        if len(cells) >= 3 and cells[0] == kernel and cells[1] == shape:
            try:
                return float(cells[2])
            except ValueError:
                return None
    return None


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int, period_ms: int = 200):
        self.gpu = gpu_index
        self.period_ms = period_ms
        self.proc = None
        self.path = None

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(prefix="clocks_", suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", str(self.period_ms), "-i", str(self.gpu)],
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
            out["sm_mhz"] = statistics.median(sm)
            out["sm_max_mhz"] = max(smax)
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        return out


def percentiles(times):
    ts = sorted(times)
    return statistics.median(ts), ts[int(0.1 * (len(ts) - 1))], ts[int(round(0.9 * (len(ts) - 1)))]


# ---------------------------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the reference's fake-quant DiT block on the host cores
# ---------------------------------------------------------------------------------------------

def cpu_block_seconds(repeats: int = 1):
    """Times oracle.dit_oracle.block_forward (the reference's CPU path restated in numpy: quantize every Linear
    input with the 4-over-6 rule, dequantize-then-fp32-matmul, window attention over dequantized NVFP4 blocks) for
    ONE block at the benchmark's widths on ONE frame of tokens (880 queries; the window keeps its 4 cached blocks of
    2640 tokens plus the new frame).  Weight and cache codes are random bytes: their values do not change the work.
    Returns (seconds per block call, description)."""
    import numpy as np

    from oracle import dit_oracle as DO
    from oracle import nvfp4_oracle as O

    rng = np.random.default_rng(0)
    s, c, f, heads = 880, DIM, FFN, HEADS

    def rand_q(rows, cols):
        mp = (rows + 127) // 128 * 128
        codes = rng.integers(0, 256, size=(mp, cols // 2), dtype=np.uint8)
        sf = rng.integers(0x30, 0x50, size=mp * cols // 16, dtype=np.uint8)
        return codes, sf, np.float32(1.0)

    p = {"ffn_dim": f}
    for n_, (o, i) in {"q": (c, c), "k": (c, c), "v": (c, c), "o": (c, c), "cq": (c, c), "co": (c, c), "ffn0": (f, c), "ffn2": (c, f)}.items():
        p[n_] = rand_q(o, i)
        p[n_ + "_b"] = np.zeros(o, dtype=np.float32)
    for n_ in ("norm_q", "norm_k", "cnorm_q", "cnorm_k", "norm3_w"):
        p[n_] = np.ones(c, dtype=np.float32)
    p["norm3_b"] = np.zeros(c, dtype=np.float32)
    x = O.bf16_round(rng.standard_normal((s, c), dtype=np.float32))
    e = O.bf16_round(rng.standard_normal((1, 6, c), dtype=np.float32) * 0.1)
    ctx_kn = O.bf16_round(rng.standard_normal((TEXT, heads, 128), dtype=np.float32))
    ctx_v = O.bf16_round(rng.standard_normal((TEXT, heads, 128), dtype=np.float32))
    cos, sin = O.rope_tables(12, 1, 22, 40)
    past = [rand_q(CHUNK_TOKENS * heads, 128) for _ in range(4)]
    t0 = time.perf_counter()
    for _ in range(repeats):
        DO.block_forward(x, e, p, ctx_kn, ctx_v, cos, sin, past, past, heads, 880, CHUNK_TOKENS)
    dt = (time.perf_counter() - t0) / repeats
    return dt, ("oracle/dit_oracle.block_forward (numpy restatement of the reference's CPU fake-quant block): 1 block, 880 query tokens "
                "(one of the chunk's 3 frames), window of 4 cached NVFP4 blocks + the frame; extrapolated x3 frames x30 layers x5 forwards")


def cpu_chunk_fps(repeats: int = 1):
    dt, desc = cpu_block_seconds(repeats)
    chunk_s = dt * 3 * LAYERS * FORWARDS
    return 12.0 / chunk_s, dt, chunk_s, desc


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    steps = max(1, min(args.steps, 10))              # one step = one bounded sample (about 11 s of host time)
    warm = 1 if args.warmup > 0 else 0
    for _ in range(warm):
        cpu_chunk_fps(1)
    vals = [cpu_chunk_fps(1) for _ in range(steps)]
    value = statistics.mean(v[0] for v in vals)
    chunk_s = statistics.mean(v[2] for v in vals)
    cores = os.cpu_count() or 1
    line = {
        "impl": "reference", "metric": "dit_chunk_video_fps", "value": value, "unit": "frames/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": chunk_s * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "nvfp4 fake-quant (dequantized to f32 on the CPU)", "data": "synthetic",
        "config": {"workload": "30-layer Wan2.2-5B-shaped causal DiT, one AR chunk (3 latent frames, 5 forwards), 15-frame window; "
                               "the CPU arm times a bounded sample and extrapolates", "l2": "n/a (CPU)"},
        "cpu_baseline": {"value": value, "unit": "frames/s", "cores": cores, "kind": "port",
                         "sample": vals[0][3] + f"; {vals[0][1]:.1f} s per block call"},
        "e2e": {"value": value, "unit": "frames/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)


# ---------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------

def sp_parity_check(dev, rank, world, group):
    """Bit-equality of the sequence-parallel DiT with the single-GPU DiT on the live ranks (reduced configuration,
    amax MAX-reduced over the group, peer-memory exchange when available): every rank runs both models on the same
    inputs and compares its token shard of five chunks and its head shard of the last cache block.
    Returns ('bit-exact' or 'mismatch', exchange kind)."""
    import torch
    import torch.distributed as dist

    from longlive_b200 import dit, ops

    cfg = dit.DiTConfig(dim=1024, ffn_dim=1024, heads=8, layers=2, text_len=128, text_dim=64, freq_dim=32, grid_h=6, grid_w=8,
                        frames_per_chunk=3, window_frames=9, sink_frames=3, in_channels=4)
    par = dit.CausalDiT(cfg, device=dev, seed=4, sp_group=group, sync_amax=True, use_graphs=True)
    ref = dit.CausalDiT(cfg, device=dev, seed=4)
    g = torch.Generator(device=dev).manual_seed(9)
    raw = torch.randn(cfg.text_len, cfg.text_dim, generator=g, device=dev).bfloat16()
    ctx_p, ctx_r = par.encode_text(raw), ref.encode_text(raw)
    sl = cfg.chunk_tokens // world
    ok = True
    for chunk in range(5):
        lat = torch.randn(cfg.chunk_tokens, cfg.patch_dim, generator=g, device=dev).bfloat16()
        out_r = ref.run_chunk(lat, ctx_r, chunk)
        out_p = par.run_chunk(lat[rank * sl:(rank + 1) * sl].contiguous(), ctx_p, chunk)
        ok = ok and bool(torch.equal(out_p, out_r[rank * sl:(rank + 1) * sl]))
    hl = cfg.heads // world
    kr = ref.cache.k[0][ref.cache.current_slot()].dequantize(torch.float32).view(cfg.chunk_tokens, cfg.heads, 128)
    kp = par.cache.k[0][par.cache.current_slot()].dequantize(torch.float32).view(cfg.chunk_tokens, hl, 128)
    ok = ok and bool(torch.equal(kp, kr[:, rank * hl:(rank + 1) * hl]))
    ops.check_status(dev)
    exchange = "peer stores" if par.arena is not None else "nccl"
    par.close()
    flag = torch.tensor([1 if ok else 0], device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    del par, ref
    torch.cuda.empty_cache()
    return ("bit-exact" if int(flag.item()) == 1 else "mismatch"), exchange


def fp4_mma_issue_rate(dev, k_blocks=4000, reps=5):
    """TFLOP/s of block-scaled FP4 MMAs issued back to back on operands resident in shared memory (llnv_fp4_mma_rate): the
    tensor-core ceiling of the W4A4 main loop on this device, measured live."""
    import ctypes

    import torch

    from longlive_b200 import _lib
    lib = _lib.lib()
    flop = ctypes.c_double()
    stream = torch.cuda.current_stream(dev).cuda_stream
    times = []
    for i in range(reps + 2):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        _lib.check(lib.llnv_fp4_mma_rate(k_blocks, ctypes.byref(flop), stream))
        e.record()
        torch.cuda.synchronize(dev)
        if i >= 2:
            times.append(s.elapsed_time(e))
    return flop.value / (statistics.median(times) * 1e-3) / 1e12


def run_gemm_sweep(dev, rank, world, steps, warmup, peaks):
    """One pass over the 30 GEMMs of the DiT-block shape sweep per step (operands resident, L2 flushed between steps,
    the 30 launches replayed as one CUDA graph), on every rank independently; beside it the ten GEMMs a block runs on a
    2640-token chunk, so that the large-M shapes cannot hide them."""
    import torch
    import torch.distributed as dist

    import longlive_b200 as L
    from longlive_b200 import ops

    shapes = sweep_shapes()
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)

    def activation(m, k):
        x = torch.randn(m, k, generator=gen, device=dev)
        mask = torch.rand(m, k, generator=gen, device=dev) < 0.001
        return torch.where(mask, x * 20, x).bfloat16()

    cfg = L.QuantizationConfig(scale_rule="mse")
    weights, acts, outs = {}, {}, {}
    for name, m, n, k in shapes:
        if (name, n, k) not in weights:
            weights[(name, n, k)] = L.quantize_to_fp4((torch.randn(n, k, generator=gen, device=dev) * 0.02).bfloat16(), cfg)
        if (m, k) not in acts:
            acts[(m, k)] = L.quantize_to_fp4(activation(m, k), cfg)
        if (m, n) not in outs:
            outs[(m, n)] = torch.empty(m, n, dtype=torch.bfloat16, device=dev)
    flush = torch.empty(256 * 1024 * 1024, dtype=torch.uint8, device=dev)

    def graph_of(sel):
        def step():
            for name, m, n, k in sel:
                xq, wq = acts[(m, k)], weights[(name, n, k)]
                ops.gemm_nvfp4(xq.values, xq.scale_factors, xq.amax, 3, wq.values, wq.scale_factors, wq.amax, 3, m, n, k, out=outs[(m, n)])
        step()
        torch.cuda.synchronize(dev)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, capture_error_mode="thread_local"):
            step()
        return g

    def timed(g, n_steps):
        for _ in range(max(warmup, 3)):
            flush.fill_(1)
            g.replay()
        torch.cuda.synchronize(dev)
        total = 0.0
        for i in range(n_steps):
            flush.fill_(i & 0xFF)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            g.replay()
            e.record()
            torch.cuda.synchronize(dev)
            total += s.elapsed_time(e)
        ms = total / n_steps
        if world > 1:
            t = torch.tensor([ms], dtype=torch.float64, device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    fp4_peak = 4.0 * peaks["bf16_tflops"]
    ms_all = timed(graph_of(shapes), steps)
    dit_shapes = [s for s in shapes if s[1] in (CHUNK_TOKENS, TEXT)][:10]       # the 10 GEMMs a chunk forward runs per block
    ms_dit = timed(graph_of(dit_shapes), steps)
    tf_all = flops_of(shapes) / (ms_all * 1e-3) / 1e12
    tf_dit = flops_of(dit_shapes) / (ms_dit * 1e-3) / 1e12
    del flush
    mma_peak = fp4_mma_issue_rate(dev)
    return {
        "metric": "w4a4_gemm_tflops", "unit": "TFLOP/s per GPU", "value": tf_all, "ms_per_step": ms_all, "steps": steps,
        "workload": "q/k/v/o + cross q/o 3072x3072, cross k/v M=512, FFN 3072<->14336; M in {880,2640,10560}; 30 GEMMs per step, "
                    "every rank on its own operands, no collective",
        "flops_per_step": flops_of(shapes), "l2": "flushed between timed steps (256 MiB write)",
        "roofline": {"bound": "tensor", "achieved": tf_all, "peak": fp4_peak, "unit": "TFLOP/s", "frac": tf_all / fp4_peak,
                     "traffic": dram_traffic("gemm_nvfp4_kernel", "2640x14336x3072"), "traffic_case": "M=2640 N=14336 K=3072 launch (profiles/dram_traffic.md)",
                     "peak_note": f"4 x {peaks['source']} dense bf16 burst peak ({peaks['bf16_tflops']} TFLOP/s): no FP4 entry is measured; nominal dense FP4 is 9000",
                     "kernel": "gemm_nvfp4_kernel", "frac_of_nominal_9pf": tf_all / 9000.0,
                     "mma_issue_peak": mma_peak, "frac_of_mma_issue_peak": tf_all / mma_peak,
                     "mma_issue_peak_note": "llnv_fp4_mma_rate measured in this run: every SM issues 128x256x64 block-scaled FP4 MMAs back to "
                                            "back on operands resident in shared memory (no loads, no epilogue)"},
        "m2640_only": {"value": tf_dit, "ms_per_step": ms_dit, "frac": tf_dit / fp4_peak, "frac_of_nominal_9pf": tf_dit / 9000.0,
                       "frac_of_mma_issue_peak": tf_dit / mma_peak,
                       "workload": "the 10 GEMMs one block runs on a 2640-token chunk (cross k/v at M=512)", "flops_per_step": flops_of(dit_shapes)},
    }


def attention_roofline(dev, rank, world, peaks, iters=8):
    """The chunk attention at the rank's shape (2640 queries, 4 cached NVFP4 blocks + the bf16 chunk, 24 / N heads),
    timed live with CUDA events on the launching stream, L2 flushed between launches."""
    import torch

    import longlive_b200 as L
    from longlive_b200 import ops

    heads, t, blocks = HEADS // world, CHUNK_TOKENS, 4
    gen = torch.Generator(device=dev).manual_seed(3)
    kq = [L.quantize_to_fp4(torch.randn(t * heads, 128, generator=gen, device=dev).bfloat16()) for _ in range(blocks)]
    vq = [L.quantize_to_fp4(torch.randn(t * heads, 128, generator=gen, device=dev).bfloat16()) for _ in range(blocks)]
    q = torch.randn(t, heads * 128, generator=gen, device=dev).bfloat16()
    kc = torch.randn(t, heads * 128, generator=gen, device=dev).bfloat16()
    vc = torch.randn(t, heads * 128, generator=gen, device=dev).bfloat16()
    out = torch.empty_like(q)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    for _ in range(3):
        ops.attention_nvfp4kv(q, kq, vq, t, kc, vc, heads, out=out)
    torch.cuda.synchronize(dev)
    times = []
    for i in range(iters):
        flush.fill_(i)
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        ops.attention_nvfp4kv(q, kq, vq, t, kc, vc, heads, out=out)
        e.record()
        torch.cuda.synchronize(dev)
        times.append(s.elapsed_time(e))
    ms = statistics.mean(times)
    fl = 4.0 * t * (blocks + 1) * t * heads * 128
    achieved = fl / (ms * 1e-3) / 1e12
    peak = peaks["bf16_tflops"]
    return {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s", "frac": achieved / peak,
            "traffic": (lambda t: None if t is None else t * heads / 24.0)(dram_traffic("attention_kernel<fused>", "2640x4x2640x24")),
            "traffic_case": "ncu capture at 24 heads (profiles/dram_traffic.md), scaled by heads / 24", "kernel": "attention_kernel<true> (NVFP4 K/V decoded in the load stage)",
            "shape": f"{t} queries x {(blocks + 1) * t} keys x {heads} heads", "avg_launch_us": ms * 1e3, "launches_timed": iters,
            "algorithmic_flops_per_launch": fl,
            "peak_note": f"{peaks['source']} dense bf16 burst peak (cuBLAS GEMM); the kernel's MMAs are bf16 (kind::f16)"}


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    from longlive_b200 import _lib, dit, ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    group = dist.group.WORLD if world > 1 else None
    lib = _lib.lib()
    peaks = load_peaks()

    def sync_all():
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize(dev)

    def max_over_ranks(vals):
        if world == 1:
            return list(vals)
        t = torch.tensor(list(vals), dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return [float(v) for v in t.tolist()]

    sp_parity, sp_exchange = (None, "none")
    if world > 1:
        sp_parity, sp_exchange = sp_parity_check(dev, rank, world, group)

    # ---- the chunk, steady state ---------------------------------------------------------------------------
    cfg = dit.DiTConfig()
    sync_amax = world > 1 and not args.per_shard_scales
    model = dit.CausalDiT(cfg, device=dev, seed=0, sp_group=group, sync_amax=sync_amax, use_graphs=not args.eager,
                          edge_linear=os.environ.get("LLNV_EDGE_LINEAR", "own"), ffn_requant=args.ffn_requant)
    gen = torch.Generator(device=dev).manual_seed(7)
    ctx = model.encode_text(torch.randn(cfg.text_len, cfg.text_dim, generator=gen, device=dev).bfloat16())
    sl = cfg.chunk_tokens // world
    lat_full = torch.randn(cfg.chunk_tokens, cfg.patch_dim, generator=gen, device=dev).bfloat16()
    lat = lat_full[rank * sl:(rank + 1) * sl].contiguous()
    handoff = None
    if world == 1:
        from longlive_b200.handoff import LatentHandoff
        handoff = LatentHandoff(cfg.in_channels, cfg.frames_per_chunk, 2 * cfg.grid_h, 2 * cfg.grid_w, device=dev, target="host", depth=3)
    chunk = 0
    # fill the window, then one full period of the rolling block table (each of its states is captured as a CUDA
    # graph on first use); at least `warmup` chunks in total
    period = cfg.max_blocks - cfg.sink_frames // cfg.frames_per_chunk
    launches0 = lib.llnv_launch_count()
    model.run_chunk(lat, ctx, chunk)
    chunk += 1
    launches_per_chunk = lib.llnv_launch_count() - launches0             # eager chunk: every kernel of 5 forwards + 4 scheduler steps
    sampler = ClockSampler(local_rank)
    n_warm = max(cfg.max_blocks + period - 1, args.warmup)
    for i in range(n_warm):
        if i == n_warm - 2 and rank == 0:
            sampler.start()            # nvidia-smi's own start-up (NVML initialisation) falls into the last warm-up chunks, not the timed ones
        model.run_chunk(lat, ctx, chunk)
        chunk += 1
    sync_all()
    times = []
    wall0 = time.perf_counter()
    for _ in range(args.steps):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
        s.record()
        out = model.run_chunk(lat, ctx, chunk)
        e.record()
        torch.cuda.synchronize(dev)
        times.append(s.elapsed_time(e))
        chunk += 1
    wall = time.perf_counter() - wall0
    ops.check_status(dev)
    med, p10, p90 = max_over_ranks(percentiles(times))
    total_ms = max_over_ranks([sum(times)])[0]
    ms_per_step = total_ms / args.steps
    value = 12.0 / (ms_per_step * 1e-3)

    # ---- end to end from host buffers ----------------------------------------------------------------------
    e2e_steps = max(1, min(args.steps, 5))
    host_lat = lat.cpu().pin_memory()
    dev_lat = torch.empty_like(lat)
    host_out = torch.empty_like(host_lat).pin_memory()
    sync_all()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        dev_lat.copy_(host_lat, non_blocking=True)                       # this chunk's noise latents, pinned host -> device
        out = model.run_chunk(dev_lat, ctx, chunk)
        if handoff is not None:
            handoff.push(out)                                            # unpatchify + side-stream copy to pinned host memory
            seq, _host = handoff.pop()                                   # waits for that copy
            handoff.release(seq)
        else:
            host_out.copy_(out, non_blocking=True)                       # the rank's token shard of the finished chunk
            torch.cuda.synchronize(dev)
        chunk += 1
    sync_all()
    e2e_s = max_over_ranks([(time.perf_counter() - t0) / e2e_steps])[0]
    clocks = sampler.stop() if rank == 0 else {}
    h2d = lat.numel() * 2
    d2h = handoff.bytes_per_chunk if handoff is not None else lat.numel() * 2
    kv_bytes = model.cache.bytes()
    cur_bytes = (model.cur_k.numel() + model.cur_v.numel()) * 2
    exchange = "none" if world == 1 else ("producer kernels store into peer memory (NVLink), own barrier" if model.arena is not None else "NCCL all-to-all")
    model.close()
    del model
    torch.cuda.empty_cache()

    # ---- rollout from an empty cache (240 latent frames) ---------------------------------------------------
    rollout = None
    if not args.no_rollout:
        m2 = dit.CausalDiT(cfg, device=dev, seed=0, sp_group=group, sync_amax=sync_amax, use_graphs=not args.eager)
        ctx2 = m2.encode_text(torch.randn(cfg.text_len, cfg.text_dim, generator=gen, device=dev).bfloat16())
        rt = []
        for c in range(args.rollout_chunks):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            m2.run_chunk(lat, ctx2, c)
            e.record()
            torch.cuda.synchronize(dev)
            rt.append(s.elapsed_time(e))
        ops.check_status(dev)
        rt = max_over_ranks(rt)
        fill_n = cfg.max_blocks + period                                 # chunks that run eagerly or capture a graph
        steady = rt[fill_n:] if len(rt) > fill_n + 2 else rt
        smed, sp10, sp90 = percentiles(steady)
        rollout = {"chunks": len(rt), "latent_frames": 3 * len(rt), "total_s": sum(rt) * 1e-3, "video_fps_whole_rollout": 12.0 * len(rt) / (sum(rt) * 1e-3),
                   "fill_phase_chunks": fill_n, "fill_phase_ms_per_chunk": [round(v, 2) for v in rt[:fill_n]],
                   "steady_ms_per_chunk_p50": smed, "steady_ms_per_chunk_p10": sp10, "steady_ms_per_chunk_p90": sp90,
                   "note": "cache starts empty; the window grows for 5 chunks, then the block table rolls; the first pass over each table "
                           "state captures its CUDA graphs"}
        m2.close()
        del m2
        torch.cuda.empty_cache()

    attn = attention_roofline(dev, rank, world, peaks)
    gemm = None if args.no_gemm_sweep else run_gemm_sweep(dev, rank, world, max(3, min(args.steps, 10)), args.warmup, peaks)

    if rank == 0:
        gemm_fl, attn_fl = chunk_flops()
        fp4_peak = 4.0 * peaks["bf16_tflops_sustained"]
        ideal_s = (gemm_fl / (fp4_peak * 1e12) + attn_fl / (peaks["bf16_tflops_sustained"] * 1e12)) / world
        line = {
            "metric": "dit_chunk_video_fps", "value": value, "unit": "frames/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(cfg.max_blocks + period, args.warmup + 1), "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "nvfp4 W4A4 Linears (f32 accumulate, bf16 out) + bf16 attention over an NVFP4 KV cache",
            "data": "synthetic, random-init weights",
            "config": {"workload": "30-layer Wan2.2-5B-shaped causal DiT (dim 3072, FFN 14336, 24 heads), one AR chunk = 3 latent frames "
                                   "(2640 tokens) x (4 denoising forwards + UniPC steps + 1 re-cache forward), window 15 frames (13200 keys), "
                                   "512 text tokens; BASELINE config 4 at N=1, config 5's steady state at N>1",
                       "l2": "inputs larger than L2: a chunk streams 2.9 GB of NVFP4 weights five times",
                       "launches": "CUDA graph per (block-table state, timestep)" if not args.eager else "eager launches",
                       "parallelism": "single GPU" if world == 1 else f"sequence-parallel over {world} GPUs (tokens / heads), exchange: {exchange}",
                       "amax_sync": bool(sync_amax), "ffn_requant": args.ffn_requant, "latent_fps": 3.0 / (ms_per_step * 1e-3)},
            "ms_per_chunk_p50": med, "ms_per_chunk_p10": p10, "ms_per_chunk_p90": p90,
            "clocks": clocks,
            "e2e": {"value": 12.0 / e2e_s, "unit": "frames/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                    "ms_per_step": e2e_s * 1e3,
                    "path": "CausalDiT.run_chunk from a pinned host latent; finished chunk through LatentHandoff to pinned host memory"
                            if world == 1 else "CausalDiT.run_chunk from pinned host latents; every rank copies its token shard of the chunk to pinned host memory"},
            "gpu_launches": int(launches_per_chunk) * args.steps,
            "gpu_launches_note": f"{int(launches_per_chunk)} kernels of this library per chunk (counted on an eagerly launched chunk; timed chunks replay them from graphs)",
            "roofline": attn,
            "chunk_roofline": {"bound": "tensor", "algorithmic_flops_fp4_gemm": gemm_fl, "algorithmic_flops_bf16_attention": attn_fl,
                               "ideal_ms_per_chunk": ideal_s * 1e3, "frac": ideal_s / (ms_per_step * 1e-3),
                               "peak_note": f"GEMM flops at 4 x {peaks['source']} sustained bf16 peak ({peaks['bf16_tflops_sustained']} TFLOP/s), "
                                            f"attention flops at that peak, divided over {world} GPU(s)"},
            "memory": {"kv_cache_bytes_per_rank": kv_bytes, "current_chunk_kv_bytes_per_rank": cur_bytes,
                       "note": "no bf16 copy of the cache exists: the attention kernel decodes the NVFP4 blocks in its load stage"},
            "wall_s_timed_region": wall,
        }
        if sp_parity is not None:
            line["sp_parity"] = sp_parity
            line["sp_parity_note"] = f"reduced-configuration DiT, {world} ranks vs 1 GPU on every rank, amax MAX-reduced, exchange: {sp_exchange}"
            line["nvlink_bytes_sent_per_rank_per_chunk"] = int(5 * (cfg.chunk_tokens // world) * cfg.dim * 2 * (world - 1) / world) * cfg.layers * 5
        if rollout is not None:
            line["rollout"] = rollout
        if gemm is not None:
            line["gemm_sweep"] = gemm
        if world == 1 and not args.no_cpu_baseline:
            fps, dt, chunk_s, desc = cpu_chunk_fps(1)
            line["cpu_baseline"] = {"value": fps, "unit": "frames/s", "cores": os.cpu_count() or 1, "kind": "port",
                                    "sample": desc + f"; {dt:.1f} s per block call -> {chunk_s:.0f} s per chunk"}
        emit(line)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_kernel_case(spec: str, iters: int):
    """Run one kernel on one shape a few times (used for ncu captures and quick timing):
    gemm:MxNxK[:tile]   quantize:MxK[:rule]   kvdequant:BLOCKSxTOKENSxHEADS   attention:LQxLKxHEADS   ropenorm:TOKENSxHEADS
    attnkv:LQxBLOCKSxTOKENSxHEADS[:twostep]  (attention over BLOCKS NVFP4 cache blocks + one bf16 chunk; twostep = dequantize, then attend)
    linear:MxNxK  (the bf16 Linear of the edge layers)
    fp4peak:KBLOCKS  (MMA issue only: every SM issues KBLOCKS x 4 block-scaled FP4 MMAs of 128 x 256 x 64 on operands resident
                      in shared memory; the rate is the tensor-core ceiling of the W4A4 main loop on this device)
    refgemm:MxNxK  (the same NVFP4 operands through torch._scaled_mm, i.e. the vendor library's block-scaled FP4 GEMM: an
                    anchor on the same box, not part of the product path; prints the error text if the build refuses NVFP4)
    adalnq:MxC[:PHASE]  (adaLN on load + quantize of an M x C activation with 880-row frames; PHASE 1 = row statistics + amax only,
                         2 = quantize only, default both)
    unipc:ELEMENTS[:f32]  (the scheduler step with order-2 corrector and predictor: 5 tensors read, 3 written)
    forward:LAYERS  (one eager forward of a LAYERS-layer DiT at the benchmark's widths with a full window; the cache blocks are
                     filled with quantized noise instead of running the chunks that would fill them)"""
    import torch

    import longlive_b200 as L
    from longlive_b200 import _lib, ops

    lib = _lib.lib()
    kind, _, rest = spec.partition(":")
    if kind == "forward":
        from longlive_b200 import dit
        dev = torch.device("cuda", 0)
        torch.cuda.set_device(dev)
        cfg = dit.DiTConfig(layers=int(rest))
        model = dit.CausalDiT(cfg, device=dev, seed=0)
        gen = torch.Generator(device=dev).manual_seed(7)
        ctx = model.encode_text(torch.randn(cfg.text_len, cfg.text_dim, generator=gen, device=dev).bfloat16())
        lat = torch.randn(cfg.chunk_tokens, cfg.patch_dim, generator=gen, device=dev).bfloat16()
        noise = torch.randn(cfg.chunk_tokens * cfg.heads, 128, generator=gen, device=dev).bfloat16()
        for layer in range(cfg.layers):
            for slot in range(cfg.max_blocks):
                L.quantize_to_fp4(noise, out=model.cache.k[layer][slot])
                L.quantize_to_fp4(noise, out=model.cache.v[layer][slot])
        model.cache.filled = cfg.max_blocks
        t = torch.full((cfg.frames_per_chunk,), 937.0, device=dev)
        times = []
        for i in range(iters + 1):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            model.forward(lat, t, ctx, 12, t_key=(937.0,) * 3)
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
        ops.check_status(dev)
        print(json.dumps({"kernel_case": spec, "iters": iters, "median_ms": statistics.median(times[1:]), "first_ms": times[0]}))
        return
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
    elif kind == "fp4peak":
        import ctypes
        flop = ctypes.c_double()
        stream = torch.cuda.current_stream().cuda_stream
        fn = lambda: _lib.check(lib.llnv_fp4_mma_rate(d[0], ctypes.byref(flop), stream))
        fn()
        work, unit = flop.value / 1e12, "TFLOP/s"
    elif kind == "refgemm":
        m, n, k = d
        xq = L.quantize_to_fp4(torch.randn(m, k, generator=gen, device=dev).bfloat16())
        wq = L.quantize_to_fp4((torch.randn(n, k, generator=gen, device=dev) * 0.02).bfloat16())
        try:
            a = xq.values.view(torch.float4_e2m1fn_x2)            # rows padded to 128, as the scale layout needs
            b = wq.values.view(torch.float4_e2m1fn_x2).t()
            fn = lambda: torch._scaled_mm(a, b, xq.scale_factors, wq.scale_factors, out_dtype=torch.bfloat16)
            fn()
            torch.cuda.synchronize()
        except Exception as exc:          # noqa: BLE001 - the point is to record why the anchor is unavailable
            print(json.dumps({"kernel_case": spec, "unavailable": f"{type(exc).__name__}: {str(exc)[:300]}"}))
            return
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
    elif kind == "adalnq":
        import ctypes
        m, c = d
        frames = max(1, m // 880)
        x = torch.randn(m, c, generator=gen, device=dev).bfloat16()
        mod = (torch.randn(frames, 6, c, generator=gen, device=dev) * 0.2).bfloat16()
        mp = ops.padded_rows(m)
        codes = torch.empty(mp, c // 2, dtype=torch.uint8, device=dev)
        sf = torch.empty(mp * c // 16, dtype=torch.uint8, device=dev)
        amax = torch.zeros(1, dtype=torch.float32, device=dev)
        stats = torch.empty(2 * m, dtype=torch.float32, device=dev)
        stream = torch.cuda.current_stream().cuda_stream
        phase = int(opt or 0)
        call = lambda ph: _lib.check(lib.llnv_adaln_quantize_nvfp4_ex(
            x.data_ptr(), m, c, x.stride(0), mod[:, 1].data_ptr(), mod[:, 0].data_ptr(), mod.stride(0), (m + frames - 1) // frames,
            ctypes.c_float(1e-6), 1, 3, codes.data_ptr(), sf.data_ptr(), amax.data_ptr(), None, 0, stats.data_ptr(), 0, ph, stream))
        call(0)
        fn = lambda: call(phase)
        work, unit = (2.0 if phase == 1 else 2.5625) * m * c / 1e9, "GB/s"
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
    ap.add_argument("--steps", type=int, default=8, help="AR chunks timed (two periods of the rolling block table)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-gemm-sweep", action="store_true")
    ap.add_argument("--no-rollout", action="store_true")
    ap.add_argument("--rollout-chunks", type=int, default=80, help="chunks of the from-empty rollout (80 = 240 latent frames)")
    ap.add_argument("--ffn-requant", default="two_pass", choices=["two_pass", "single_pass"],
                    help="two_pass = the reference's rounding (default); single_pass = the FFN-up GEMM quantizes its own output under the "
                         "previous forward's tensor amax (not the reference's rounding, and measured slower)")
    ap.add_argument("--eager", action="store_true", help="launch every kernel eagerly instead of replaying CUDA graphs")
    ap.add_argument("--per-shard-scales", action="store_true",
                    help="N > 1: every rank quantizes its token shard with its own tensor scale (what the reference's "
                         "sequence-parallel path does; valid NVFP4, not bit-identical to one GPU) instead of reducing amax")
    args = ap.parse_args()
    if args.kernel_case:
        run_kernel_case(args.kernel_case, args.iters)
        return
    quiet_stdout()
    if args.impl == "reference":
        run_reference_arm(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
