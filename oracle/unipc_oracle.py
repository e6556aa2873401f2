"""CPU restatement of the reference's flow-matching UniPC scheduler step.  TEST INFRASTRUCTURE:
only tests, the smoke check and the CPU legs of the benchmark may import this file; the product
never does.

Follows wan_5b/utils/fm_solvers_unipc.py of the reference (solver_order 2, ``bh2``, ``predict_x0``,
``flow_prediction``, ``lower_order_final``, final sigma zero -- the configuration the chunk loop
builds, pipeline/causal_diffusion_inference.py:892-899):

* ``set_timesteps``   fm_solvers_unipc.py:162-229  (sigma grid, shift, integer timesteps)
* ``convert``         fm_solvers_unipc.py:281-327  (x0 = sample - sigma * flow)
* ``predictor``       fm_solvers_unipc.py:352-486  (UniP, B(h) = expm1(-h))
* ``corrector``       fm_solvers_unipc.py:488-628  (UniC)
* ``step``            fm_solvers_unipc.py:657-741  (order warm-up, history rotation)

Parity is pinned: ``tests/golden/unipc_steps.npz`` holds samples produced by the reference's own
scheduler on CPU (``tests/golden/make_golden_unipc.py``), and ``tests/test_unipc_oracle.py`` checks
this file against them bit for bit, in fp32 and in bf16.

Rounding.  The reference computes every scalar (sigma ratios, log-SNR differences, expm1) as a
0-dim fp32 tensor and every tensor operation in the dtype of the latents, one PyTorch call per
operation, so each intermediate tensor is rounded to that dtype.  How a 0-dim fp32 scalar enters a
tensor operation depends on where PyTorch runs it:

* ``scalars="host"``: PyTorch's CPU kernels first cast the scalar of a multiply or subtract to the
  tensor dtype (bf16 latents see bf16 coefficients); a division keeps the fp32 divisor.  This is the
  mode the golden vectors were produced in.
* ``scalars="device"``: PyTorch's CUDA kernels keep the scalar in fp32 and turn a division by a
  scalar into a multiplication by its fp32 reciprocal.  This is what the reference does on a GPU,
  and what the CUDA kernel of this repository reproduces.

With fp32 latents the two modes differ only in the division.
"""
from __future__ import annotations

import numpy as np

from .nvfp4_oracle import bf16_round

F32 = np.float32


def set_timesteps(steps: int, shift: float, num_train_timesteps: int = 1000):
    """(timesteps int64 [steps], sigmas fp32 [steps + 1]) -- fm_solvers_unipc.py:107-133, 184-212."""
    alphas = np.linspace(1, 1 / num_train_timesteps, num_train_timesteps)[::-1].copy()
    base = (1.0 - alphas).astype(F32)                       # constructor: shift 1, stored as fp32
    sigma_max, sigma_min = float(base[0]), float(base[-1])
    sig = np.linspace(sigma_max, sigma_min, steps + 1).copy()[:-1]
    sig = shift * sig / (1 + (shift - 1) * sig)
    timesteps = (sig * num_train_timesteps).astype(np.int64)
    sigmas = np.concatenate([sig, [0.0]]).astype(F32)
    return timesteps, sigmas


class _Ops:
    """Tensor arithmetic in the latents' dtype with PyTorch's scalar handling (see module docstring)."""

    def __init__(self, dtype: str, scalars: str):
        if dtype not in ("bf16", "f32") or scalars not in ("host", "device"):
            raise ValueError("dtype is 'bf16' or 'f32', scalars 'host' or 'device'")
        self.bf16, self.host = dtype == "bf16", scalars == "host"

    def r(self, x):
        x = np.asarray(x, dtype=F32)
        return bf16_round(x) if self.bf16 else x

    def scalar(self, s):
        s = F32(s)
        return F32(bf16_round(np.array([s], dtype=F32))[0]) if (self.bf16 and self.host) else s

    def mul_s(self, s, t):
        return self.r(self.scalar(s) * t)

    def sub_s(self, t, s):
        return self.r(t - self.scalar(s))

    def div_s(self, t, s):
        with np.errstate(divide="ignore", invalid="ignore"):
            return self.r(t / F32(s)) if self.host else self.r(t * (F32(1.0) / F32(s)))

    def sub(self, a, b):
        return self.r(a - b)

    def add(self, a, b):
        return self.r(a + b)

    def mul_t(self, s, t):
        """Multiply by a coefficient that already is a tensor of the latents' dtype."""
        return self.r(self.r(np.array(s, dtype=F32)) * t)


def _log(x) -> np.float32:
    """fp32 logarithm, correctly rounded (PyTorch's CPU logf is accurate to 1 ulp and agrees with the
    correctly rounded value on every sigma of the golden cases; numpy's own fp32 log does not)."""
    with np.errstate(divide="ignore"):
        return F32(np.log(np.float64(F32(x))))


def _expm1(x) -> np.float32:
    return F32(np.expm1(np.float64(F32(x))))


def _lambda(sigma: np.float32) -> np.float32:
    return F32(_log(F32(1.0) - sigma) - _log(sigma))


def _coefficients(sig_t, sig_s0, sig_hist, order: int):
    """Scalars shared by predictor and corrector (fm_solvers_unipc.py:407-455 / 550-598), all fp32.
    ``sig_hist``: sigmas of the older history entries (one per order above 1)."""
    with np.errstate(divide="ignore", invalid="ignore", over="ignore"):
        alpha_t = F32(1.0) - sig_t
        lam_t, lam_s0 = _lambda(sig_t), _lambda(sig_s0)
        h = F32(lam_t - lam_s0)
        rks = [F32(F32(_lambda(s) - lam_s0) / h) for s in sig_hist[:order - 1]] + [F32(1.0)]
        hh = F32(-h)
        h_phi_1 = _expm1(hh)
        B_h = h_phi_1
        h_phi_k = F32(F32(h_phi_1 / hh) - F32(1.0))
        R, b, fact = [], [], 1
        for i in range(1, order + 1):
            R.append(np.array([F32(rk) ** (i - 1) for rk in rks], dtype=F32))
            b.append(F32(F32(h_phi_k * F32(fact)) / B_h))
            fact *= i + 1
            h_phi_k = F32(F32(h_phi_k / hh) - F32(1.0 / fact))
    return {"c1": F32(sig_t / sig_s0), "c2": F32(alpha_t * h_phi_1), "c3": F32(alpha_t * B_h), "rks": rks,
            "R": np.stack(R), "b": np.array(b, dtype=F32)}


def _solve2(R: np.ndarray, b: np.ndarray) -> np.ndarray:
    """fp32 LU with partial pivoting of a 2 x 2 system, the operation order of LAPACK's sgesv
    (torch.linalg.solve, fm_solvers_unipc.py:605)."""
    A = R.astype(F32).copy()
    y = b.astype(F32).copy()
    if abs(A[1, 0]) > abs(A[0, 0]):
        A, y = A[::-1].copy(), y[::-1].copy()
    l = F32(A[1, 0] * F32(F32(1.0) / A[0, 0]))
    u11 = F32(A[1, 1] - F32(l * A[0, 1]))
    y1 = F32(y[1] - F32(l * y[0]))
    x1 = F32(y1 / u11)
    x0 = F32(F32(y[0] - F32(A[0, 1] * x1)) / A[0, 0])
    return np.array([x0, x1], dtype=F32)


class FlowUniPC:
    """State machine of ``FlowUniPCMultistepScheduler.step`` for solver order <= 2."""

    def __init__(self, steps: int, shift: float, dtype: str = "bf16", scalars: str = "device", solver_order: int = 2):
        if solver_order not in (1, 2):
            raise NotImplementedError("solver_order 1 or 2")
        self.timesteps, self.sigmas = set_timesteps(steps, shift)
        self.ops = _Ops(dtype, scalars)
        self.order = solver_order
        self.k = 0
        self.lower_order_nums = 0
        self.this_order = 0
        self.m = [None, None]            # x0 predictions: [-2], [-1]
        self.last_sample = None

    def _update(self, x, m0, m_older, sig_t, sig_s0, sig_hist, order, model_t=None, rhos_c=None):
        """UniP (``model_t`` None) or UniC.  x: the sample the update starts from."""
        o = self.ops
        c = _coefficients(sig_t, sig_s0, sig_hist, order)
        x_t_ = o.sub(o.mul_s(c["c1"], x), o.mul_s(c["c2"], m0))
        D1 = o.div_s(o.sub(m_older, m0), c["rks"][0]) if order == 2 else None
        if model_t is None:                                                    # predictor, fm_solvers_unipc.py:457-485
            if D1 is None:
                return o.sub_s(x_t_, F32(c["c3"] * F32(0)))
            return o.sub(x_t_, o.mul_s(c["c3"], o.mul_t(0.5, D1)))
        rhos = np.array([0.5], dtype=F32) if order == 1 else (_solve2(c["R"], c["b"]) if rhos_c is None else
                                                              np.asarray(rhos_c, dtype=F32))    # fm_solvers_unipc.py:601-605
        res = o.mul_t(rhos[-1], o.sub(model_t, m0))
        if D1 is not None:
            res = o.add(o.mul_t(rhos[0], D1), res)
        return o.sub(x_t_, o.mul_s(c["c3"], res))

    def step(self, model_output: np.ndarray, sample: np.ndarray, rhos_c=None) -> np.ndarray:
        """One ``scheduler.step``.  ``rhos_c``: the order-2 corrector weights to use instead of this
        file's own 2 x 2 solve (the last bit of the reference's LAPACK solve depends on the library)."""
        o, k, sg = self.ops, self.k, self.sigmas
        v, x = o.r(model_output), o.r(sample)
        x0 = o.sub(x, o.mul_s(sg[k], v))                                       # fm_solvers_unipc.py:320-323
        if k > 0 and self.last_sample is not None:                             # fm_solvers_unipc.py:689-701
            x = self._update(self.last_sample, self.m[1], self.m[0], sg[k], sg[k - 1], [sg[k - 2]] if k >= 2 else [],
                             self.this_order, model_t=x0, rhos_c=rhos_c)
        self.m = [self.m[1], x0]
        this_order = min(self.order, len(self.timesteps) - k)                  # lower_order_final
        self.this_order = min(this_order, self.lower_order_nums + 1)
        self.last_sample = x
        out = self._update(x, self.m[1], self.m[0], sg[k + 1], sg[k], [sg[k - 1]] if k >= 1 else [], self.this_order)
        if self.lower_order_nums < self.order:
            self.lower_order_nums += 1
        self.k += 1
        return out
