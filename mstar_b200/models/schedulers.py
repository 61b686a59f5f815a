"""Samplers of the flow-matching generators. Coefficients are host floats computed from the sigma ladder once per
request; the updates are a handful of axpy-style tensor ops on the device, so a step never synchronises.

``FlowEulerSchedule``: x <- x + (sigma_next - sigma) * v with the time-shifted ladder (BAGEL: shift 3.0;
mstar/model/bagel/submodules.py:1005-1100 computes the same dt inline).
``FlowUniPC``: UniPC multistep predictor-corrector (order 2, B(h) = expm1(h), data prediction from a flow
output), the sampler of Wan2.2 and Cosmos3 (mstar/model/wan22/components/unipc.py:117-192; diffusers'
UniPCMultistepScheduler in mstar/model/cosmos3/submodules.py:911).
"""
from __future__ import annotations

import math

import torch


def shifted_sigmas(num_steps: int, shift: float) -> list[float]:
    """num_steps + 1 values from 1 down to 0: linear ladder, then s -> shift * s / (1 + (shift - 1) * s)."""
    base = [1.0 - i / num_steps for i in range(num_steps)]
    return [shift * s / (1 + (shift - 1) * s) for s in base] + [0.0]


class FlowEulerSchedule:
    def __init__(self, num_steps: int, shift: float = 3.0):
        self.sigmas = shifted_sigmas(num_steps, shift)
        self.num_steps = num_steps

    def timestep(self, i: int) -> float:
        return self.sigmas[i]

    def dt(self, i: int) -> float:
        return self.sigmas[i + 1] - self.sigmas[i]

    def step(self, x: torch.Tensor, v: torch.Tensor, i: int) -> torch.Tensor:
        return x + self.dt(i) * v


class FlowUniPC:
    """One instance per request. ``step(v, x)`` consumes the model's flow output at ``timestep(i)`` and returns
    the next sample; keeps the last two data predictions and the last sample."""

    def __init__(self, num_steps: int, shift: float = 5.0, order: int = 2, num_train_timesteps: int = 1000):
        lin = [1.0 - (1.0 - 1.0 / num_train_timesteps) * i / num_steps for i in range(num_steps)]  # 1 .. ~1/N
        self.sigmas = [shift * s / (1 + (shift - 1) * s) for s in lin] + [0.0]
        self.timesteps = [s * num_train_timesteps for s in self.sigmas[:-1]]
        self.num_steps, self.order = num_steps, order
        self.i = 0
        self.lower_order_nums = 0
        self.outputs: list[torch.Tensor | None] = [None] * order      # data predictions, newest last
        self.out_idx: list[int] = [0] * order
        self.last_sample: torch.Tensor | None = None
        self.this_order = 1

    def timestep(self, i: int | None = None) -> float:
        return self.timesteps[self.i if i is None else i]

    @staticmethod
    def _lam(sigma: float) -> float:
        if sigma <= 0.0:
            return math.inf
        return math.log(max(1.0 - sigma, 1e-12)) - math.log(sigma)

    def _coeffs(self, s0: int, t: int, prev: list[int], order: int, corrector: bool):
        """Scalar pieces of one update from ladder index s0 to t; ``prev`` are the ladder indices of the older
        data predictions (newest first)."""
        sig_t, sig_s = self.sigmas[t], self.sigmas[s0]
        alpha_t = 1.0 - sig_t
        h = self._lam(sig_t) - self._lam(sig_s)
        hh = -h
        h_phi_1 = math.expm1(hh) if math.isfinite(hh) else -1.0
        B_h = h_phi_1
        rks = [(self._lam(self.sigmas[si]) - self._lam(sig_s)) / h for si in prev] + [1.0]
        R, b = [], []
        h_phi_k = (h_phi_1 / hh - 1.0) if math.isfinite(hh) else -1.0
        fact = 1.0
        for k in range(1, order + 1):
            R.append([r ** (k - 1) for r in rks])
            b.append(h_phi_k * fact / B_h)
            fact *= k + 1
            h_phi_k = (h_phi_k / hh - 1.0 / fact) if math.isfinite(hh) else -1.0 / fact
        if corrector:
            rhos = [0.5] if order == 1 else torch.linalg.solve(torch.tensor(R, dtype=torch.float64),
                                                               torch.tensor(b, dtype=torch.float64)).tolist()
        else:
            if order == 1:
                rhos = []
            elif order == 2:
                rhos = [0.5]
            else:
                rhos = torch.linalg.solve(torch.tensor([r[:-1] for r in R[:-1]], dtype=torch.float64),
                                          torch.tensor(b[:-1], dtype=torch.float64)).tolist()
        return sig_t / sig_s, alpha_t, h_phi_1, B_h, rks, rhos

    def step(self, v: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        i = self.i
        x = x.float()
        x0_pred = x - self.sigmas[i] * v.float()                      # flow output -> data prediction
        if i > 0 and self.last_sample is not None:                     # corrector on the previous step
            order = self.this_order
            m0 = self.outputs[-1]
            prev = [self.out_idx[-(k + 1)] for k in range(1, order)]
            ratio, alpha_t, h_phi_1, B_h, rks, rhos = self._coeffs(i - 1, i, prev, order, True)
            res = rhos[-1] * (x0_pred - m0)
            for k in range(1, order):
                res = res + rhos[k - 1] * (self.outputs[-(k + 1)] - m0) / rks[k - 1]
            x = ratio * self.last_sample - alpha_t * h_phi_1 * m0 - alpha_t * B_h * res
        self.outputs = self.outputs[1:] + [x0_pred]
        self.out_idx = self.out_idx[1:] + [i]
        order = min(self.order, self.num_steps - i, self.lower_order_nums + 1)
        self.this_order = order
        self.last_sample = x
        m0 = self.outputs[-1]
        prev = [self.out_idx[-(k + 1)] for k in range(1, order)]
        ratio, alpha_t, h_phi_1, B_h, rks, rhos = self._coeffs(i, i + 1, prev, order, False)
        nxt = ratio * x - alpha_t * h_phi_1 * m0
        for k in range(1, order):
            nxt = nxt - alpha_t * B_h * rhos[k - 1] * (self.outputs[-(k + 1)] - m0) / rks[k - 1]
        if self.lower_order_nums < self.order:
            self.lower_order_nums += 1
        self.i += 1
        return nxt
