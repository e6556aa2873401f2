"""The scheduler-step kernel (llnv_unipc_step behind FlowUniPCMultistepScheduler.step) against

* the oracle in its device-scalar mode, bit for bit, on the golden inputs;
* the golden samples of the reference's CPU run, within the rounding of the coefficients
  (PyTorch's CPU kernels round fp32 scalars to the tensor dtype, its CUDA kernels do not);
* the same sequence of PyTorch calls the reference makes, run eagerly on the GPU, bit for bit:
  this is what the reference computes on a GPU.
"""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "unipc_steps.npz")
CASES = ("steps4_shift5_bf16", "steps4_shift5_f32", "steps8_shift3_bf16", "steps8_shift3_f32", "steps3_shift1_bf16",
         "steps1_shift5_bf16", "steps2_shift5_f32", "steps50_shift5_bf16")


def _sched(steps, shift, **kw):
    from longlive_b200.scheduler import FlowUniPCMultistepScheduler
    s = FlowUniPCMultistepScheduler(num_train_timesteps=1000, shift=1, use_dynamic_shifting=False, **kw)
    s.set_timesteps(steps, device="cpu", shift=shift)
    return s


def _to_dev(a, bf16):
    t = torch.from_numpy(np.ascontiguousarray(a))
    return (t.view(torch.bfloat16) if bf16 else t).cuda()


def _bits(t):
    return (t.view(torch.uint16) if t.dtype == torch.bfloat16 else t.view(torch.int32)).cpu().numpy()


@pytest.mark.parametrize("name", CASES)
def test_kernel_matches_oracle_bit_exact(name):
    from oracle import unipc_oracle as uo
    from oracle.nvfp4_oracle import bf16_bits, bf16_from_bits
    g = np.load(GOLDEN)
    bf16 = name.endswith("bf16")
    steps, shift = len(g[f"{name}.timesteps"]), float(g[f"{name}.shift"])
    sched = _sched(steps, shift)
    orc = uo.FlowUniPC(steps, shift, dtype="bf16" if bf16 else "f32", scalars="device")
    dec = bf16_from_bits if bf16 else (lambda a: a.astype(np.float32))
    x_dev = _to_dev(g[f"{name}.samples"][0], bf16)
    x_orc = dec(g[f"{name}.samples"][0])
    for k, t in enumerate(sched.timesteps.tolist()):
        v = g[f"{name}.model_outputs"][k]
        c = sched.coefficients(k, torch.bfloat16 if bf16 else torch.float32)
        x_dev = sched.step(_to_dev(v, bf16), t, x_dev, return_dict=False)[0]
        x_orc = orc.step(dec(v), x_orc, rhos_c=[c.c_rho0, c.c_rho1] if c.corrector_order == 2 else None)
        got = _bits(x_dev)
        want = bf16_bits(x_orc) if bf16 else x_orc.view(np.int32)
        bad = np.flatnonzero(got.ravel() != want.ravel())
        assert bad.size == 0, f"{name} step {k}: {bad.size} of {got.size} differ, first at {bad[:4]}"
        # the stored history is the oracle's too
        assert np.array_equal(_bits(sched.model_outputs[-1]).ravel(), (bf16_bits(orc.m[1]) if bf16 else orc.m[1].view(np.int32)).ravel())
        assert np.array_equal(_bits(sched.last_sample).ravel(), (bf16_bits(orc.last_sample) if bf16 else orc.last_sample.view(np.int32)).ravel())


@pytest.mark.parametrize("name", CASES)
def test_kernel_close_to_reference_cpu_samples(name):
    """Restarting every step from the golden sample, the result stays within a few ulp of the
    latents' dtype of the reference's CPU result (the difference is the coefficient rounding)."""
    g = np.load(GOLDEN)
    bf16 = name.endswith("bf16")
    steps, shift = len(g[f"{name}.timesteps"]), float(g[f"{name}.shift"])
    sched = _sched(steps, shift)
    eps = 2.0 ** -8 if bf16 else 2.0 ** -23
    x = _to_dev(g[f"{name}.samples"][0], bf16)
    for k, t in enumerate(sched.timesteps.tolist()):
        v = _to_dev(g[f"{name}.model_outputs"][k], bf16)
        x = sched.step(v, t, x, return_dict=False)[0]
        want = _to_dev(g[f"{name}.samples"][k + 1], bf16)
        scale = x.float().abs() + want.float().abs() + 4 * v.float().abs() + 4.0
        # drift accumulates over the steps of a run: a few ulp per step
        assert bool(((x.float() - want.float()).abs() <= 16 * (k + 1) * eps * scale).all()), f"{name} step {k}"


def _eager_step(state, sigmas, k, n_steps, v, x):
    """The PyTorch calls of the reference's scheduler.step in their order, on the tensors' device:
    scalars are 0-dim fp32 CPU tensors, tensor operations run in the latents' dtype."""
    lam = lambda s: torch.log(1 - s) - torch.log(s)

    def update(x, m0, m_older, t, s0, older, order, model_t=None):
        sigma_t, sigma_s0 = sigmas[t], sigmas[s0]
        alpha_t = 1 - sigma_t
        h = lam(sigma_t) - lam(sigma_s0)
        rks, D1s = [], []
        if order == 2:
            rk = (lam(sigmas[older]) - lam(sigma_s0)) / h
            rks.append(rk)
            D1s.append((m_older - m0) / rk)
        rks.append(1.0)
        rks = torch.tensor(rks, device=x.device)
        hh = -h
        h_phi_1 = torch.expm1(hh)
        B_h = torch.expm1(hh)
        x_t_ = sigma_t / sigma_s0 * x - alpha_t * h_phi_1 * m0
        if model_t is None:
            if not D1s:
                return (x_t_ - alpha_t * B_h * 0).to(x.dtype)
            rhos_p = torch.tensor([0.5], dtype=x.dtype, device=x.device)
            pred_res = torch.einsum("k,bkc...->bc...", rhos_p, torch.stack(D1s, dim=1))
            return (x_t_ - alpha_t * B_h * pred_res).to(x.dtype)
        rhos_c = state["rhos"][k].to(device=x.device, dtype=x.dtype)
        corr_res = torch.einsum("k,bkc...->bc...", rhos_c[:-1], torch.stack(D1s, dim=1)) if D1s else 0
        D1_t = model_t - m0
        return (x_t_ - alpha_t * B_h * (corr_res + rhos_c[-1] * D1_t)).to(x.dtype)

    x0 = x - sigmas[k] * v
    if k > 0:
        x = update(state["last"], state["m"][1], state["m"][0], k, k - 1, k - 2, state["order"], model_t=x0)
    state["m"] = [state["m"][1], x0]
    state["order"] = min(2, n_steps - k, k + 1)
    state["last"] = x
    return update(x, state["m"][1], state["m"][0], k + 1, k, k - 1, state["order"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("steps,shift,shape", [(4, 5.0, (1, 3, 48, 22, 40)), (6, 3.0, (2, 2, 5, 7, 9))])
def test_kernel_matches_eager_pytorch_on_gpu(dtype, steps, shift, shape):
    """Bit-exact against the reference's own sequence of PyTorch CUDA calls, at the latent shape of a
    chunk ([batch, frames, channels, h, w]) and at a small odd shape."""
    sched = _sched(steps, shift)
    gen = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(shape, device="cuda", generator=gen).to(dtype)
    x_ref = x.clone()
    rhos = {}
    for k in range(steps):
        c = sched.coefficients(k, dtype)
        rhos[k] = torch.tensor([c.c_rho0, c.c_rho1] if c.corrector_order == 2 else [c.c_rho1])
    state = {"m": [None, None], "last": None, "order": 0, "rhos": rhos}
    for k, t in enumerate(sched.timesteps.tolist()):
        v = (torch.randn(shape, device="cuda", generator=gen) * 1.5).to(dtype)
        x_in, x_keep, v_keep = x, x.clone(), v.clone()
        x = sched.step(v, t, x, return_dict=False)[0]
        x_ref = _eager_step(state, sched.sigmas, k, steps, v, x_ref)
        assert x.shape == x_ref.shape and x.dtype == dtype
        assert torch.equal(x_in, x_keep) and torch.equal(v, v_keep)      # inputs are left alone
        bad = (_bits(x) != _bits(x_ref)).sum()
        assert bad == 0, f"step {k}: {bad} of {x.numel()} differ"
    with pytest.raises(IndexError):
        sched.step(v, 0, x)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("n,offset", [(1, 0), (7, 0), (8, 1), (1029, 3), (4096, 0)])
def test_unaligned_and_ragged_sizes(dtype, n, offset):
    """Any length and any element-aligned address: the vector path needs 16-byte alignment of every
    tensor, everything else goes through the scalar path; both give the same bits."""
    gen = torch.Generator(device="cuda").manual_seed(n + offset)
    big = [torch.randn(n + 16, device="cuda", generator=gen).to(dtype) for _ in range(8)]
    a, b = _sched(4, 5.0), _sched(4, 5.0)
    xa = big[0][offset:offset + n]
    xb = xa.clone()
    for k, t in enumerate(a.timesteps.tolist()):
        va = big[1 + k][offset:offset + n]
        xa = a.step(va, t, xa, return_dict=False)[0]
        xb = b.step(va.clone(), t, xb, return_dict=False)[0]
        assert np.array_equal(_bits(xa), _bits(xb))


def test_empty_and_mismatched_inputs():
    s = _sched(4, 5.0)
    e = torch.empty(0, dtype=torch.bfloat16, device="cuda")
    assert s.step(e, 999, e, return_dict=False)[0].numel() == 0
    s = _sched(4, 5.0)
    x = torch.zeros(16, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(RuntimeError):
        s.step(x.float(), 999, x)
    with pytest.raises(RuntimeError):
        s.step(x.half(), 999, x.half())
    out = s.step(x, 999, x)
    assert out.prev_sample.shape == x.shape


def test_new_run_after_set_timesteps_repeats_the_first():
    """set_timesteps clears the history: two runs over the same inputs give the same samples."""
    gen = torch.Generator(device="cuda").manual_seed(5)
    vs = [torch.randn(4096, device="cuda", generator=gen).bfloat16() for _ in range(4)]
    x0 = torch.randn(4096, device="cuda", generator=gen).bfloat16()
    s = _sched(4, 5.0)
    runs = []
    for _ in range(2):
        s.set_timesteps(4, device="cpu", shift=5.0)
        x = x0
        for v, t in zip(vs, s.timesteps.tolist()):
            x = s.step(v, t, x, return_dict=False)[0]
        runs.append(x)
    assert torch.equal(runs[0], runs[1])
