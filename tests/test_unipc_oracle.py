"""The scheduler oracle against samples produced by the reference's own UniPC scheduler on CPU
(tests/golden/unipc_steps.npz, written by tests/golden/make_golden_unipc.py)."""
import os

import numpy as np
import pytest

from oracle import unipc_oracle as uo
from oracle.nvfp4_oracle import bf16_bits, bf16_from_bits

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "unipc_steps.npz")
CASES = ("steps4_shift5_bf16", "steps4_shift5_f32", "steps8_shift3_bf16", "steps8_shift3_f32", "steps3_shift1_bf16",
         "steps1_shift5_bf16", "steps2_shift5_f32", "steps50_shift5_bf16")


def _case(g, name):
    bf16 = name.endswith("bf16")
    dec = (lambda a: bf16_from_bits(a)) if bf16 else (lambda a: a.astype(np.float32))
    return bf16, g[f"{name}.timesteps"], g[f"{name}.sigmas"], float(g[f"{name}.shift"]), dec(g[f"{name}.model_outputs"]), g[f"{name}.samples"]


def _solve_of(g, name, k):
    """The corrector weights the reference's LAPACK solve returned at step k (None: no solve at that step)."""
    r = g[f"{name}.corrector_solves"][k]
    return None if np.isnan(r[0]) else r


@pytest.mark.parametrize("name", CASES)
def test_schedule_matches_reference(name):
    g = np.load(GOLDEN)
    _, timesteps, sigmas, shift, _, _ = _case(g, name)
    t, s = uo.set_timesteps(len(timesteps), shift)
    assert np.array_equal(t, timesteps)
    assert np.array_equal(s.view(np.uint32), sigmas.view(np.uint32))


def test_inference_schedule_is_the_chunk_loops():
    """4 steps at shift 5 are the timesteps the chunk loop runs the generator at."""
    t, s = uo.set_timesteps(4, 5.0)
    assert t.tolist() == [999, 937, 833, 624]
    assert s[-1] == 0.0 and np.all(np.diff(s) < 0)


@pytest.mark.parametrize("name", CASES)
def test_steps_bit_exact_in_host_mode(name):
    """Every sample of every step, bit for bit, with the 2 x 2 corrector solve taken from the reference run."""
    g = np.load(GOLDEN)
    bf16, timesteps, _, shift, outputs, samples = _case(g, name)
    sched = uo.FlowUniPC(len(timesteps), shift, dtype="bf16" if bf16 else "f32", scalars="host")
    x = bf16_from_bits(samples[0]) if bf16 else samples[0].astype(np.float32)
    for k in range(len(timesteps)):
        x = sched.step(outputs[k], x, rhos_c=_solve_of(g, name, k))
        got = bf16_bits(x) if bf16 else x.view(np.uint32)
        want = samples[k + 1] if bf16 else samples[k + 1].view(np.uint32)
        bad = np.flatnonzero(got != want)
        assert bad.size == 0, f"{name} step {k}: {bad.size} of {got.size} differ, first at {bad[:4]}"


@pytest.mark.parametrize("name", [c for c in CASES if c.endswith("bf16")])
def test_bf16_steps_bit_exact_with_own_solve(name):
    """In bf16 the weights are rounded to bf16 before use: the oracle's own 2 x 2 solve gives the same samples."""
    g = np.load(GOLDEN)
    _, timesteps, _, shift, outputs, samples = _case(g, name)
    sched = uo.FlowUniPC(len(timesteps), shift, dtype="bf16", scalars="host")
    x = bf16_from_bits(samples[0])
    for k in range(len(timesteps)):
        x = sched.step(outputs[k], x)
        assert np.array_equal(bf16_bits(x), samples[k + 1]), f"{name} step {k}"


@pytest.mark.parametrize("name", CASES)
def test_own_solve_within_2_ulp_of_lapack(name):
    """ulp of the larger weight: the smaller one is a difference of numbers of that size."""
    g = np.load(GOLDEN)
    _, timesteps, sigmas, _, _, _ = _case(g, name)
    seen = 0
    for k in range(2, len(timesteps)):
        want = _solve_of(g, name, k)
        if want is None:
            continue
        c = uo._coefficients(sigmas[k], sigmas[k - 1], [sigmas[k - 2]], 2)
        got = uo._solve2(c["R"], c["b"])
        assert np.all(np.abs(got - want) <= 2 * np.spacing(np.max(np.abs(want)))), (k, got, want)
        seen += 1
    assert seen == max(0, len(timesteps) - 2)


@pytest.mark.parametrize("name", CASES)
def test_device_mode_stays_within_rounding_of_host_mode(name):
    """The two scalar conventions differ by coefficient rounding only: a few ulp of the latents' dtype."""
    g = np.load(GOLDEN)
    bf16, timesteps, _, shift, outputs, samples = _case(g, name)
    sched = uo.FlowUniPC(len(timesteps), shift, dtype="bf16" if bf16 else "f32", scalars="device")
    dec = bf16_from_bits if bf16 else (lambda a: a.astype(np.float32))
    eps = 2.0 ** -8 if bf16 else 2.0 ** -23
    host = uo.FlowUniPC(len(timesteps), shift, dtype="bf16" if bf16 else "f32", scalars="host")
    for k in range(len(timesteps)):
        x = sched.step(outputs[k], dec(samples[k]))           # restart from the golden sample: no drift across steps
        want = host.step(outputs[k], dec(samples[k]))
        # the terms of one update: sample, two x0 predictions and their difference divided by r_k
        scale = np.abs(dec(samples[k])) + 4 * np.abs(outputs[k]) + np.abs(want) + 4.0
        assert np.all(np.abs(x - want) <= 16 * eps * scale), f"{name} step {k}: {np.max(np.abs(x - want) / scale) / eps:.1f} eps"


def test_last_step_returns_the_x0_prediction():
    """With final sigma zero the last predictor step is the model's x0 (fm_solvers_unipc.py:457-467 at sigma_t = 0)."""
    rng = np.random.default_rng(3)
    sched = uo.FlowUniPC(1, 5.0, dtype="f32", scalars="device")
    x, v = rng.standard_normal(256).astype(np.float32), rng.standard_normal(256).astype(np.float32)
    out = sched.step(v, x)
    assert np.array_equal(out, (x - sched.sigmas[0] * v).astype(np.float32) + np.float32(0))
