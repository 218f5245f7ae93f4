"""UniPC multistep sampler for flow-matching models (data prediction, ``bh2`` variant).

The network predicts the velocity ``v = noise - x0`` at noise level sigma (``x_sigma = (1 - sigma) x0 +
sigma n``); the solver works on the data prediction ``x0 = x - sigma v`` in log-SNR time
``lambda = log((1 - sigma) / sigma)``: a UniP predictor of order ``p`` extrapolates from the last ``p``
data predictions, and after the network is evaluated at the new point a UniC corrector of the same
order refines the previous step with it (no extra evaluation).  The sigma grid is the shifted
``linspace(1, 0, N + 1)[:-1]`` grid of the training scheduler followed by 0, pinned at construction;
the last steps fall back to lower order (reference: pinned-grid UniPC used for 50-step validation,
solar/backends/wan22/runtime/scheduler.py:60-112).
"""
from __future__ import annotations

import math
from typing import Callable, List, Optional

import torch


class FlowUniPC:
    def __init__(self, num_steps: int = 50, shift: float = 5.0, order: int = 2, lower_order_final: bool = True):
        if num_steps < 1 or order < 1:
            raise ValueError("num_steps and order must be positive")
        s = torch.linspace(1.0, 0.0, num_steps + 1, dtype=torch.float64)[:-1]
        s = shift * s / (1.0 + (shift - 1.0) * s)
        self.sigmas = torch.cat([s.clamp(max=1.0 - 1e-6), torch.zeros(1, dtype=torch.float64)])
        self.timesteps = (self.sigmas[:-1] * 1000.0).float()
        self.order, self.lower_order_final = order, lower_order_final
        self.reset()

    def reset(self) -> None:
        self.outputs: List[torch.Tensor] = []     # data predictions, newest last
        self.lams: List[float] = []
        self.step_index = 0
        self._last_sample: Optional[torch.Tensor] = None
        self._this_order = 1

    @staticmethod
    def _lam(sigma: float) -> float:
        sigma = min(max(sigma, 1e-12), 1.0 - 1e-12)
        return math.log(1.0 - sigma) - math.log(sigma)

    def _coeffs(self, order: int, h: float, rks: List[float], corrector: bool):
        hh = -h
        h_phi_1 = math.expm1(hh)
        B_h = math.expm1(hh)
        h_phi_k = h_phi_1 / hh - 1.0
        fact = 1
        R, b = [], []
        rks = list(rks) + ([1.0] if corrector else [])
        for i in range(1, len(rks) + 1):
            R.append([rk ** (i - 1) for rk in rks])
            b.append(h_phi_k * fact / B_h)
            fact *= i + 1
            h_phi_k = h_phi_k / hh - 1.0 / fact
        if not rks:
            return h_phi_1, B_h, []
        Rm, bm = torch.tensor(R, dtype=torch.float64), torch.tensor(b, dtype=torch.float64)
        if len(rks) == 1:
            rhos = [0.5]
        else:
            rhos = torch.linalg.solve(Rm, bm).tolist()
        return h_phi_1, B_h, rhos

    def _update(self, x, m0, prev, lam_s0, prev_lams, sigma_s0, sigma_t, order, m_t=None):
        """One UniP (m_t None) or UniC (m_t given) update from sigma_s0 to sigma_t in fp32."""
        lam_t = self._lam(sigma_t)
        h = lam_t - lam_s0
        rks, D1s = [], []
        for mi, li in zip(prev[:order - 1], prev_lams[:order - 1]):
            rk = (li - lam_s0) / h
            rks.append(rk)
            D1s.append((mi - m0) / rk)
        h_phi_1, B_h, rhos = self._coeffs(order, h, rks, corrector=m_t is not None)
        alpha_t = 1.0 - sigma_t
        base = (sigma_t / sigma_s0) * x - alpha_t * h_phi_1 * m0
        res = torch.zeros_like(m0)
        for rho, d in zip(rhos, D1s):
            res = res + rho * d
        if m_t is not None:
            res = res + rhos[-1] * (m_t - m0)
        return base - alpha_t * B_h * res

    def step(self, velocity: torch.Tensor, sample: torch.Tensor) -> torch.Tensor:
        """Consume the network output at ``sigmas[step_index]`` and return the sample at the next sigma."""
        i = self.step_index
        sigma, sigma_next = float(self.sigmas[i]), float(self.sigmas[i + 1])
        x = sample.float()
        m_t = x - sigma * velocity.float()                       # data prediction at the current point
        if i > 0 and self._last_sample is not None:              # UniC: refine the current sample with m_t
            prev = self.outputs[::-1]
            x = self._update(self._last_sample, prev[0], prev[1:], self.lams[-1], self.lams[::-1][1:],
                             float(self.sigmas[i - 1]), sigma, self._this_order, m_t=m_t)
        self.outputs.append(m_t)
        self.lams.append(self._lam(sigma))
        self.outputs, self.lams = self.outputs[-self.order:], self.lams[-self.order:]
        remaining = len(self.sigmas) - 1 - i
        order = min(self.order, len(self.outputs), remaining if self.lower_order_final else self.order)
        self._this_order = max(order, 1)
        self._last_sample = x
        prev = self.outputs[::-1]
        if sigma_next <= 0.0:
            out = prev[0]                                        # the last step lands on the data prediction
        else:
            out = self._update(x, prev[0], prev[1:], self.lams[-1], self.lams[::-1][1:], sigma, sigma_next,
                               self._this_order)
        self.step_index += 1
        return out.to(sample.dtype)


def sample(model_fn: Callable[[torch.Tensor, float], torch.Tensor], noise: torch.Tensor, *, num_steps: int = 50,
           shift: float = 5.0, order: int = 2) -> torch.Tensor:
    """``model_fn(x, timestep)`` -> velocity; integrates from pure noise to data."""
    solver = FlowUniPC(num_steps, shift, order)
    x = noise
    for i in range(num_steps):
        x = solver.step(model_fn(x, float(solver.timesteps[i])), x)
    return x
