"""Host side of the UniPC scheduler (no GPU): schedule, step orders and the scalar coefficients, against
the golden vectors of the reference's scheduler and against the oracle."""
import os

import numpy as np
import pytest
import torch

from longlive_b200.scheduler import FlowUniPCMultistepScheduler
from oracle import unipc_oracle as uo
from oracle.nvfp4_oracle import bf16_round

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "unipc_steps.npz")
CASES = (("steps4_shift5_bf16", 4, 5.0), ("steps8_shift3_f32", 8, 3.0), ("steps3_shift1_bf16", 3, 1.0), ("steps1_shift5_bf16", 1, 5.0),
         ("steps2_shift5_f32", 2, 5.0), ("steps50_shift5_bf16", 50, 5.0))


def _sched(steps, shift):
    s = FlowUniPCMultistepScheduler(num_train_timesteps=1000, shift=1, use_dynamic_shifting=False)
    s.set_timesteps(steps, device="cpu", shift=shift)
    return s


def _f32(x):
    return np.float32(x).view(np.uint32)


@pytest.mark.parametrize("name,steps,shift", CASES)
def test_schedule_matches_reference(name, steps, shift):
    g = np.load(GOLDEN)
    s = _sched(steps, shift)
    assert np.array_equal(s.timesteps.numpy(), g[f"{name}.timesteps"])
    assert np.array_equal(s.sigmas.numpy().view(np.uint32), g[f"{name}.sigmas"].view(np.uint32))
    assert s.step_index is None and s.num_inference_steps == steps


def test_orders_follow_warmup_and_lower_order_final():
    s = _sched(4, 5.0)
    assert [s._orders(k) for k in range(4)] == [(0, 1), (1, 2), (2, 2), (2, 1)]
    assert [_sched(1, 5.0)._orders(0)] == [(0, 1)]
    assert [_sched(2, 5.0)._orders(k) for k in range(2)] == [(0, 1), (1, 1)]
    one = FlowUniPCMultistepScheduler(solver_order=1)
    one.set_timesteps(5, shift=3.0)
    assert [one._orders(k) for k in range(5)] == [(0, 1)] + [(1, 1)] * 4


@pytest.mark.parametrize("name,steps,shift", CASES)
def test_coefficients_match_oracle_and_recorded_solves(name, steps, shift):
    """Same fp32 scalars as the oracle derives, bit for bit; the order-2 corrector weights are the
    reference run's own LAPACK solutions (rounded to bf16 for bf16 latents)."""
    g = np.load(GOLDEN)
    s = _sched(steps, shift)
    sig = s.sigmas.numpy()
    for dtype in (torch.float32, torch.bfloat16):
        for k in range(steps):
            c = s.coefficients(k, dtype)
            co, po = s._orders(k)
            assert (c.use_corrector, c.predictor_order) == (int(k > 0), po)
            assert _f32(c.sigma) == _f32(sig[k])
            p = uo._coefficients(sig[k + 1], sig[k], [sig[k - 1]] if po == 2 else [], po)
            assert (_f32(c.pc1), _f32(c.pc2), _f32(c.pc3)) == (_f32(p["c1"]), _f32(p["c2"]), _f32(p["c3"])), (k, "predictor")
            if po == 2:
                assert _f32(c.p_inv_rk) == _f32(np.float32(1.0) / p["rks"][0])
            if k > 0:
                assert c.corrector_order == co
                q = uo._coefficients(sig[k], sig[k - 1], [sig[k - 2]] if co == 2 else [], co)
                assert (_f32(c.cc1), _f32(c.cc2), _f32(c.cc3)) == (_f32(q["c1"]), _f32(q["c2"]), _f32(q["c3"])), (k, "corrector")
                if co == 2:
                    assert _f32(c.c_inv_rk) == _f32(np.float32(1.0) / q["rks"][0])
                    want = g[f"{name}.corrector_solves"][k]
                    if dtype == torch.bfloat16:
                        want = bf16_round(want)
                    assert (_f32(c.c_rho0), _f32(c.c_rho1)) == (_f32(want[0]), _f32(want[1])), (k, "rho")
                else:
                    assert c.c_rho1 == 0.5
    assert s.coefficients(steps - 1, torch.float32).pc1 == 0.0          # the last step goes to sigma 0


def test_same_grid_keeps_the_coefficient_cache():
    s = _sched(4, 5.0)
    c = s.coefficients(2, torch.bfloat16)
    s.set_timesteps(4, device="cpu", shift=5.0)
    assert s.coefficients(2, torch.bfloat16) is c
    s.set_timesteps(4, device="cpu", shift=3.0)
    assert s.coefficients(2, torch.bfloat16) is not c


def test_unsupported_configurations_raise():
    for kw in ({"solver_order": 3}, {"prediction_type": "epsilon"}, {"thresholding": True}, {"predict_x0": False},
               {"solver_type": "bh1"}, {"use_dynamic_shifting": True}, {"final_sigmas_type": "sigma_min"}, {"lower_order_final": False}):
        with pytest.raises(NotImplementedError):
            FlowUniPCMultistepScheduler(**kw)
    FlowUniPCMultistepScheduler(solver_type="midpoint")                  # mapped to bh2 as in the reference


def test_step_needs_set_timesteps_and_a_cuda_tensor():
    s = FlowUniPCMultistepScheduler()
    x = torch.zeros(8, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        s.step(x, 999, x)
    s.set_timesteps(4, shift=5.0)
    with pytest.raises(ValueError, match="CUDA tensor"):
        s.step(x, 999, x)                                               # CPU tensors: there is no CPU path
    assert s.index_for_timestep(833) == 2 and s.index_for_timestep(5) == 3
