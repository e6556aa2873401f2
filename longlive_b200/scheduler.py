"""Flow-matching UniPC scheduler with the step as one CUDA kernel.

Same class name, constructor arguments, ``set_timesteps`` / ``step`` signatures and state
(``timesteps``, ``sigmas``, ``step_index``) as the reference's ``FlowUniPCMultistepScheduler``
(wan_5b/utils/fm_solvers_unipc.py:22-135, 162-229, 657-741) in the configuration the chunk loop
uses (pipeline/causal_diffusion_inference.py:892-899): solver order <= 2, ``bh2``, x0 prediction
from a flow prediction, ``lower_order_final``, final sigma zero, no thresholding, no dynamic
shifting.  Anything else raises ``NotImplementedError`` instead of running something different.

The scalar coefficients of a step are computed here, on the host, with the same fp32 PyTorch CPU
operations the reference uses for its 0-dim sigma tensors (log, expm1, the 2 x 2
``torch.linalg.solve`` of the order-2 corrector), once per ``set_timesteps``; the tensor work of a
step -- about twenty PyTorch calls in the reference -- is one launch of ``llnv_unipc_step``, whose
rounding reproduces what those calls do on a GPU.  The x0 history and the last sample live in
buffers owned by the scheduler and rotate in place.
"""
from __future__ import annotations

import ctypes as C

import numpy as np
import torch

from . import _lib
from .ops import _check, _require_cuda, _stream


def _lam(sigma: torch.Tensor) -> torch.Tensor:
    return torch.log(1 - sigma) - torch.log(sigma)


def _update_scalars(sigmas: torch.Tensor, t: int, s0: int, older: int | None, order: int, corrector: bool, round_to) -> dict:
    """Scalars of one UniP / UniC update from sigma[s0] to sigma[t] (fm_solvers_unipc.py:407-455, 550-605).
    ``older``: index of the sigma behind the second history entry (order 2).  Every value is a 0-dim
    fp32 CPU tensor until the final ``float()``, as in the reference."""
    sigma_t, sigma_s0 = sigmas[t], sigmas[s0]
    alpha_t = 1 - sigma_t
    lambda_s0 = _lam(sigma_s0)
    h = _lam(sigma_t) - lambda_s0
    rks = []
    if order == 2:
        rks.append((_lam(sigmas[older]) - lambda_s0) / h)
    rks.append(1.0)
    rks_t = torch.tensor(rks)
    hh = -h
    h_phi_1 = torch.expm1(hh)
    B_h = torch.expm1(hh)
    out = {"c1": float(sigma_t / sigma_s0), "c2": float(alpha_t * h_phi_1), "c3": float(alpha_t * B_h),
           "inv_rk": float(torch.tensor(1.0) / rks[0]) if order == 2 else 0.0, "zero": float(alpha_t * B_h * 0)}
    if corrector:
        if order == 1:
            rhos = torch.tensor([0.5])
        else:
            h_phi_k = h_phi_1 / hh - 1
            R, b, fact = [], [], 1
            for i in range(1, order + 1):
                R.append(torch.pow(rks_t, i - 1))
                b.append(h_phi_k * fact / B_h)
                fact *= i + 1
                h_phi_k = h_phi_k / hh - 1 / fact
            rhos = torch.linalg.solve(torch.stack(R), torch.tensor(b))
        rhos = rhos.to(round_to).float()                     # ``.to(x.dtype)``, fm_solvers_unipc.py:603-605
        out["rho0"], out["rho1"] = (float(rhos[0]) if order == 2 else 0.0), float(rhos[-1])
    return out


class FlowUniPCMultistepScheduler:
    order = 1

    def __init__(self, num_train_timesteps: int = 1000, solver_order: int = 2, prediction_type: str = "flow_prediction",
                 shift: float | None = 1.0, use_dynamic_shifting: bool = False, thresholding: bool = False,
                 predict_x0: bool = True, solver_type: str = "bh2", lower_order_final: bool = True,
                 disable_corrector: tuple = (), final_sigmas_type: str = "zero"):
        if solver_order not in (1, 2):
            raise NotImplementedError("solver_order 1 or 2 (the reference's pipelines use 2)")
        if solver_type in ("midpoint", "heun", "logrho"):
            solver_type = "bh2"                               # fm_solvers_unipc.py:99-101
        if (prediction_type != "flow_prediction" or use_dynamic_shifting or thresholding or not predict_x0 or solver_type != "bh2"
                or not lower_order_final or final_sigmas_type != "zero"):
            raise NotImplementedError("only the chunk loop's configuration is built: flow_prediction, bh2, predict_x0, "
                                      "lower_order_final, final sigma zero, no thresholding, no dynamic shifting")
        self.num_train_timesteps = num_train_timesteps
        self.solver_order = solver_order
        self.shift = 1.0 if shift is None else float(shift)
        self.disable_corrector = tuple(disable_corrector)
        alphas = np.linspace(1, 1 / num_train_timesteps, num_train_timesteps)[::-1].copy()
        sigmas = torch.from_numpy(1.0 - alphas).to(dtype=torch.float32)
        sigmas = self.shift * sigmas / (1 + (self.shift - 1) * sigmas)
        self.sigmas = sigmas
        self.timesteps = sigmas * num_train_timesteps
        self.sigma_min = self.sigmas[-1].item()
        self.sigma_max = self.sigmas[0].item()
        self.num_inference_steps = None
        self._coef_cache: dict = {}
        self._buffers = None
        self._reset()

    def _reset(self) -> None:
        self._step_index = None
        self.lower_order_nums = 0
        self.this_order = 0
        self._have_last = False
        self._hist = 0                                        # x0 predictions stored so far

    @property
    def step_index(self):
        return self._step_index

    def set_timesteps(self, num_inference_steps: int, device=None, sigmas=None, mu=None, shift: float | None = None) -> None:
        """Sigma grid and integer timesteps of a run (fm_solvers_unipc.py:162-229); clears the step state."""
        if sigmas is None:
            sigmas = np.linspace(self.sigma_max, self.sigma_min, num_inference_steps + 1).copy()[:-1]
        else:
            sigmas = np.asarray(sigmas, dtype=np.float64)
        if shift is None:
            shift = self.shift
        sigmas = shift * sigmas / (1 + (shift - 1) * sigmas)
        timesteps = sigmas * self.num_train_timesteps
        new_sigmas = torch.from_numpy(np.concatenate([sigmas, [0]]).astype(np.float32))
        if self.num_inference_steps is None or not torch.equal(new_sigmas, self.sigmas):
            self._coef_cache = {}                             # same grid as the last run: its coefficients stand
        self.sigmas = new_sigmas
        self.timesteps = torch.from_numpy(timesteps).to(device=device, dtype=torch.int64)
        self._timesteps_host = [int(t) for t in timesteps.astype(np.int64)]
        self.num_inference_steps = len(timesteps)
        self._reset()

    def _orders(self, k: int) -> tuple[int, int]:
        """(order of the corrector, order of the predictor) at step k: the warm-up and
        ``lower_order_final`` rules of fm_solvers_unipc.py:714-722, 732-733 as a function of k."""
        def pred(j):
            return min(self.solver_order, self.num_inference_steps - j, j + 1)
        return (pred(k - 1) if k > 0 else 0), pred(k)

    def coefficients(self, k: int, dtype: torch.dtype) -> _lib.UniPCCoef:
        """The ``llnv_unipc_coef`` of step k for latents of ``dtype``."""
        key = (k, dtype)
        c = self._coef_cache.get(key)
        if c is None:
            co, po = self._orders(k)
            use_corr = k > 0 and (k - 1) not in self.disable_corrector
            c = _lib.UniPCCoef()
            c.sigma = float(self.sigmas[k])
            c.use_corrector, c.corrector_order, c.predictor_order = int(use_corr), co, po
            if use_corr:
                s = _update_scalars(self.sigmas, k, k - 1, k - 2 if co == 2 else None, co, True, dtype)
                c.cc1, c.cc2, c.cc3, c.c_inv_rk, c.c_rho0, c.c_rho1 = s["c1"], s["c2"], s["c3"], s["inv_rk"], s["rho0"], s["rho1"]
            s = _update_scalars(self.sigmas, k + 1, k, k - 1 if po == 2 else None, po, False, dtype)
            c.pc1, c.pc2, c.pc3, c.p_inv_rk, c.p_zero = s["c1"], s["c2"], s["c3"], s["inv_rk"], s["zero"]
            self._coef_cache[key] = c
        return c

    def index_for_timestep(self, timestep) -> int:
        """Position of ``timestep`` in the schedule (fm_solvers_unipc.py:630-643: the second match if it
        occurs twice, the last position if it does not occur)."""
        t = int(timestep)
        hits = [i for i, v in enumerate(self._timesteps_host) if v == t]
        if not hits:
            return self.num_inference_steps - 1
        return hits[1] if len(hits) > 1 else hits[0]

    def step(self, model_output: torch.Tensor, timestep, sample: torch.Tensor, return_dict: bool = True, generator=None):
        """One ``scheduler.step`` (fm_solvers_unipc.py:657-741): returns ``(prev_sample,)`` (or an object
        with ``prev_sample``).  ``model_output`` and ``sample``: CUDA tensors of one shape, bf16 or fp32."""
        if self.num_inference_steps is None:
            raise ValueError("Number of inference steps is 'None', you need to run 'set_timesteps' after creating the scheduler")
        _require_cuda(sample, "sample")
        if model_output.shape != sample.shape or model_output.dtype != sample.dtype or model_output.device != sample.device:
            raise RuntimeError("model_output and sample must have one shape, dtype and device")
        if sample.dtype not in (torch.bfloat16, torch.float32):
            raise RuntimeError("latents must be bfloat16 or float32")
        if self._step_index is None:
            self._step_index = self.index_for_timestep(timestep)
        k = self._step_index
        if k >= self.num_inference_steps:
            raise IndexError("the schedule has no step left: call set_timesteps for a new run")
        key = (tuple(sample.shape), sample.dtype, sample.device)
        if self._buffers is None or self._buffers[0] != key:
            self._buffers = (key, [torch.empty_like(sample, memory_format=torch.contiguous_format) for _ in range(3)])
            self._have_last, self._hist = False, 0
        older, prev, last = self._buffers[1]
        coef = self.coefficients(k, sample.dtype)
        if coef.use_corrector and not self._have_last:        # ``self.last_sample is not None``, fm_solvers_unipc.py:692
            coef = _lib.UniPCCoef.from_buffer_copy(coef)
            coef.use_corrector = 0
        need_prev = coef.use_corrector or coef.predictor_order == 2
        need_older = coef.use_corrector and coef.corrector_order == 2
        if (need_prev and self._hist < 1) or (need_older and self._hist < 2):
            raise RuntimeError("step() was entered in the middle of a schedule without the earlier steps' history")
        v, x = model_output.contiguous(), sample.contiguous()
        out = torch.empty_like(x)
        with torch.cuda.device(x.device):
            _check(_lib.lib().llnv_unipc_step(v.data_ptr(), x.data_ptr(), prev.data_ptr(), older.data_ptr(), last.data_ptr(),
                                              older.data_ptr(), last.data_ptr(), out.data_ptr(), x.numel(),
                                              0 if x.dtype == torch.bfloat16 else 1, C.byref(coef), _stream(x)))
        self._buffers[1][0], self._buffers[1][1] = prev, older   # the new x0 went where the oldest one was
        self._hist = min(2, self._hist + 1)
        self._have_last = True
        self.this_order = coef.predictor_order
        if self.lower_order_nums < self.solver_order:
            self.lower_order_nums += 1
        self._step_index += 1
        if not return_dict:
            return (out,)
        return SchedulerOutput(out)

    @property
    def last_sample(self):
        return self._buffers[1][2] if self._have_last else None

    @property
    def model_outputs(self):
        """The stored x0 predictions, oldest first (``None`` where the history is still empty)."""
        if self._buffers is None:
            return [None] * self.solver_order
        older, prev, _ = self._buffers[1]
        full = [older if self._hist >= 2 else None, prev if self._hist >= 1 else None]
        return full[-self.solver_order:]

    def scale_model_input(self, sample: torch.Tensor, *args, **kwargs) -> torch.Tensor:
        return sample

    def __len__(self) -> int:
        return self.num_train_timesteps


class SchedulerOutput:
    def __init__(self, prev_sample: torch.Tensor):
        self.prev_sample = prev_sample
