"""Generate ``unipc_steps.npz`` by running the REFERENCE's flow-matching UniPC scheduler on CPU.

    python tests/golden/make_golden_unipc.py --reference /path/to/LongLive

The scheduler file (wan_5b/utils/fm_solvers_unipc.py) is loaded by path, with a stand-in for the
few names it takes from ``diffusers`` (the config decorator that records the constructor's
arguments in ``self.config``, two empty base classes, ``deprecate``), which is not installed here.
For every case a seeded sequence of (model_output, sample) pairs is stepped through
``scheduler.step`` exactly as the chunk loop does (pipeline/causal_diffusion_inference.py:566-609):
the sample of step k+1 is the scheduler's output of step k.  Stored per case: the timesteps, the
sigmas, the model outputs and the samples after every step; bf16 tensors as uint16 bit patterns.
Also stored: the fp32 solutions ``torch.linalg.solve`` returned for the order-2 corrector weights
(fm_solvers_unipc.py:605), one row per step (NaN where the step made no such call) -- the last bit
of a LAPACK solve depends on the library build, so a restatement can only be compared bit for bit
once that input is fixed.
"""
from __future__ import annotations

import argparse
import functools
import importlib.util
import inspect
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

# (name, sampling steps, shift, dtype, elements)
CASES = (("steps4_shift5_bf16", 4, 5.0, torch.bfloat16, 4096), ("steps4_shift5_f32", 4, 5.0, torch.float32, 4096),
         ("steps8_shift3_bf16", 8, 3.0, torch.bfloat16, 2048), ("steps8_shift3_f32", 8, 3.0, torch.float32, 2048),
         ("steps3_shift1_bf16", 3, 1.0, torch.bfloat16, 1024), ("steps1_shift5_bf16", 1, 5.0, torch.bfloat16, 1024),
         ("steps2_shift5_f32", 2, 5.0, torch.float32, 1024), ("steps50_shift5_bf16", 50, 5.0, torch.bfloat16, 512))


def _load_scheduler(reference_root: str):
    def register_to_config(init):
        @functools.wraps(init)
        def wrapped(self, *args, **kwargs):
            sig = inspect.signature(init)
            bound = sig.bind(self, *args, **kwargs)
            bound.apply_defaults()
            values = {k: v for k, v in bound.arguments.items() if k != "self"}
            self.config = types.SimpleNamespace(**values)
            self.register_to_config = lambda **kw: self.config.__dict__.update(kw)
            init(self, *args, **kwargs)
        return wrapped

    mods = {n: types.ModuleType(n) for n in ("diffusers", "diffusers.configuration_utils", "diffusers.schedulers",
                                             "diffusers.schedulers.scheduling_utils", "diffusers.utils")}
    mods["diffusers.configuration_utils"].ConfigMixin = type("ConfigMixin", (), {})
    mods["diffusers.configuration_utils"].register_to_config = register_to_config
    su = mods["diffusers.schedulers.scheduling_utils"]
    su.KarrasDiffusionSchedulers = ()
    su.SchedulerMixin = type("SchedulerMixin", (), {})
    su.SchedulerOutput = type("SchedulerOutput", (), {"__init__": lambda self, prev_sample: setattr(self, "prev_sample", prev_sample)})
    mods["diffusers.utils"].deprecate = lambda *a, **k: None
    mods["diffusers.utils"].is_scipy_available = lambda: False
    saved = {n: sys.modules.get(n) for n in mods}
    sys.modules.update(mods)
    try:
        path = os.path.join(reference_root, "wan_5b", "utils", "fm_solvers_unipc.py")
        spec = importlib.util.spec_from_file_location("_ref_fm_solvers_unipc", path)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
    finally:
        for n, m in saved.items():
            if m is None:
                sys.modules.pop(n, None)
            else:
                sys.modules[n] = m
    return mod.FlowUniPCMultistepScheduler


def _bits(t: torch.Tensor) -> np.ndarray:
    return t.view(torch.uint16).numpy().copy() if t.dtype == torch.bfloat16 else t.numpy().copy()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the LongLive checkout")
    args = ap.parse_args()
    Scheduler = _load_scheduler(args.reference)
    out = {}
    for ci, (name, steps, shift, dtype, n) in enumerate(CASES):
        gen = torch.Generator().manual_seed(1000 + ci)
        sched = Scheduler(num_train_timesteps=1000, shift=1, use_dynamic_shifting=False)
        sched.set_timesteps(steps, device="cpu", shift=shift)       # pipeline/causal_diffusion_inference.py:894-899
        sample = torch.randn(1, 2, n // 2, generator=gen).to(dtype)
        if name.startswith("steps4"):
            sample.view(-1)[:4] = torch.tensor([0.0, -0.0, 1e-30, -3.0]).to(dtype)
        outputs, samples, solves = [], [sample], []
        real_solve = torch.linalg.solve

        def recording_solve(A, B):
            x = real_solve(A, B)
            solves[-1] = x.detach().float().numpy().copy()
            return x

        for t in sched.timesteps:
            v = (torch.randn(1, 2, n // 2, generator=gen) * 1.3).to(dtype)
            solves.append(np.full(2, np.nan, dtype=np.float32))
            torch.linalg.solve = recording_solve
            try:
                sample = sched.step(v, t, sample, return_dict=False)[0]
            finally:
                torch.linalg.solve = real_solve
            assert sample.dtype == dtype
            outputs.append(v)
            samples.append(sample)
        out[f"{name}.timesteps"] = sched.timesteps.numpy().copy()
        out[f"{name}.sigmas"] = sched.sigmas.numpy().copy()
        out[f"{name}.shift"] = np.float64(shift)
        out[f"{name}.model_outputs"] = np.stack([_bits(v) for v in outputs])
        out[f"{name}.samples"] = np.stack([_bits(s) for s in samples])
        out[f"{name}.corrector_solves"] = np.stack(solves)
        print(name, [int(t) for t in sched.timesteps][:8], float(samples[-1].float().abs().mean()))
    np.savez_compressed(os.path.join(HERE, "unipc_steps.npz"), **out)


if __name__ == "__main__":
    main()
