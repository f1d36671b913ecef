"""Diffusion schedulers.

* ``FlowMatchEulerScheduler``: ``t_i = 1 - i / N``, ``sigma = s t / (1 + (s - 1) t)``, optional
  Flux dynamic shift ``s = exp(mu)`` with ``mu`` linear in the image sequence length between
  (256, 0.5) and (4096, 1.15), model timestep ``1000 sigma``, step ``x += v (sigma_next - sigma)``,
  img2img noise ``(1 - sigma) x0 + sigma eps``
  (src/HartsyInference.Diffusion/Schedulers/FlowMatchEulerDiscreteScheduler.cs:43-171).
* ``FlowUniPCScheduler``: UniPC multistep (order 2, ``B(h) = expm1(h)``) in data-prediction form
  on the flow parameterisation ``alpha = 1 - sigma``: corrector then predictor every step
  (src/HartsyInference.Diffusion/Schedulers/FlowUniPCMultistepScheduler.cs:17-238). The reference
  runs it on the host; here every update is a handful of device tensor ops.
* ``EulerDiscreteScheduler`` / ``DDIMScheduler`` for epsilon-prediction UNet families.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from ... import ops


def flux_mu(seq_len: int, base_len: int = 256, max_len: int = 4096, base_shift: float = 0.5, max_shift: float = 1.15) -> float:
    m = (max_shift - base_shift) / (max_len - base_len)
    return seq_len * m + (base_shift - m * base_len)


class FlowMatchEulerScheduler:
    def __init__(self, num_steps: int, shift: float = 1.0, mu: Optional[float] = None, terminal: Optional[float] = None):
        t = torch.linspace(1.0, 0.0, num_steps + 1, dtype=torch.float64)[:-1]
        s = math.exp(mu) if mu is not None else shift
        sig = s * t / (1 + (s - 1) * t)
        if terminal is not None:                    # stretch so that the last sigma equals `terminal`
            one_minus = 1 - sig
            sig = 1 - one_minus / (one_minus[-1] / (1 - terminal))
        self.sigmas = torch.cat([sig, torch.zeros(1, dtype=torch.float64)]).float()
        self.num_steps = num_steps

    def timestep(self, i: int) -> float:
        return float(self.sigmas[i]) * 1000.0

    def sigma(self, i: int) -> float:
        return float(self.sigmas[i])

    def dt(self, i: int) -> float:
        return float(self.sigmas[i + 1] - self.sigmas[i])

    def step(self, latents: torch.Tensor, cond: torch.Tensor, i: int, uncond: Optional[torch.Tensor] = None,
             guidance: float = 1.0, renorm_min: Optional[float] = None, row_norm: bool = False) -> torch.Tensor:
        """In-place CFG combine + Euler step on fp32 latents (one fused kernel). With true guidance,
        ``renorm_min`` rescales the guided prediction by clamp(||cond|| / ||guided||, renorm_min, 1) over the
        whole tensor and ``row_norm`` rescales every row of the last dimension to the norm of its
        conditional row (the two guidance normalisations of the reference's CfgHelper)."""
        if uncond is not None and row_norm:
            return ops.cfg_rownorm_euler_step(latents, cond.contiguous(), uncond.contiguous(), guidance, self.dt(i))
        if uncond is not None and renorm_min is not None:
            return ops.cfg_renorm_euler_step(latents, cond.contiguous(), uncond.contiguous(), guidance, self.dt(i), renorm_min)
        return ops.cfg_euler_step(latents, cond, uncond, guidance, self.dt(i))

    def add_noise(self, x0: torch.Tensor, noise: torch.Tensor, i: int) -> torch.Tensor:
        s = self.sigma(i)
        return (1 - s) * x0 + s * noise


class FlowUniPCScheduler:
    def __init__(self, num_steps: int, shift: float = 5.0, order: int = 2, num_train_timesteps: int = 1000):
        sig = torch.linspace(1.0, 1.0 / num_train_timesteps, num_steps, dtype=torch.float64)
        sig = shift * sig / (1 + (shift - 1) * sig)
        self.sigmas = torch.cat([sig, torch.zeros(1, dtype=torch.float64)])
        self.num_steps = num_steps
        self.order = order
        self.model_outputs: list[Optional[torch.Tensor]] = [None] * order
        self.lower_order_nums = 0
        self.last_sample: Optional[torch.Tensor] = None
        self.this_order = 1
        self.step_index = 0

    def timestep(self, i: int) -> float:
        return float(self.sigmas[i]) * 1000.0

    @staticmethod
    def _lambda(sigma: float) -> float:
        if sigma <= 0:
            return math.inf
        return math.log(1 - sigma) - math.log(sigma) if sigma < 1 else -math.inf

    def _coeffs(self, order: int, step_from: int, step_to: int, outputs_back: int):
        """Shared set-up of the UniP / UniC updates: returns (h_phi_1, B_h, rks, R, b, alpha_t, ratio)."""
        sigma_t, sigma_s0 = float(self.sigmas[step_to]), float(self.sigmas[step_from])
        alpha_t = 1 - sigma_t
        lam_t, lam_s0 = self._lambda(sigma_t), self._lambda(sigma_s0)
        h = lam_t - lam_s0
        rks = []
        for i in range(1, order):
            si = step_from - i
            lam_si = self._lambda(float(self.sigmas[si]))
            rks.append((lam_si - lam_s0) / h)
        rks.append(1.0)
        hh = -h
        h_phi_1 = math.expm1(hh) if hh > -700 else -1.0
        B_h = h_phi_1
        h_phi_k = (h_phi_1 / hh - 1) if math.isfinite(hh) else -1.0
        fact = 1
        R, b = [], []
        for i in range(1, order + 1):
            R.append([rk ** (i - 1) for rk in rks])
            b.append(h_phi_k * fact / B_h)
            fact *= i + 1
            h_phi_k = (h_phi_k / hh - 1 / fact) if math.isfinite(hh) else -1.0 / fact
        ratio = sigma_t / sigma_s0
        return h_phi_1, B_h, rks, R, b, alpha_t, ratio

    def _predict(self, sample: torch.Tensor, order: int) -> torch.Tensor:
        m0 = self.model_outputs[-1]
        i = self.step_index
        h_phi_1, B_h, rks, R, b, alpha_t, ratio = self._coeffs(order, i, i + 1, 0)
        # x = ratio sample - alpha h_phi_1 m0 - alpha B_h / 2 (m1 - m0) / r, gathered per tensor so that the
        # update is one pass over the latents (ops.lincomb: one kernel on the device)
        c0 = -alpha_t * h_phi_1
        terms = [(ratio, sample)]
        if order >= 2:
            k = -alpha_t * B_h * 0.5 / rks[0]
            terms += [(c0 - k, m0), (k, self.model_outputs[-2])]
        else:
            terms += [(c0, m0)]
        return _combine(terms)

    def _correct(self, this_x0: torch.Tensor, last_sample: torch.Tensor, order: int) -> torch.Tensor:
        m0 = self.model_outputs[-1]
        i = self.step_index
        h_phi_1, B_h, rks, R, b, alpha_t, ratio = self._coeffs(order, i - 1, i, 0)
        c0 = -alpha_t * h_phi_1
        if order == 1:
            k_t = -alpha_t * B_h * 0.5
            return _combine([(ratio, last_sample), (c0 - k_t, m0), (k_t, this_x0)])
        rhos = torch.linalg.solve(torch.tensor(R, dtype=torch.float64), torch.tensor(b, dtype=torch.float64)).tolist()
        k1 = -alpha_t * B_h * rhos[0] / rks[0]          # weight of (m1 - m0)
        k_t = -alpha_t * B_h * rhos[-1]                 # weight of (this_x0 - m0)
        return _combine([(ratio, last_sample), (c0 - k1 - k_t, m0), (k1, self.model_outputs[-2]), (k_t, this_x0)])

    def step(self, velocity: torch.Tensor, sample: torch.Tensor) -> torch.Tensor:
        """velocity: model output at the current step (fp32 or bf16), sample fp32 -> next sample."""
        i = self.step_index
        sigma = float(self.sigmas[i])
        x0 = sample - sigma * velocity.float()
        if i > 0 and self.last_sample is not None:
            sample = self._correct(x0, self.last_sample, self.this_order)
        self.model_outputs = self.model_outputs[1:] + [x0]
        order = min(self.order, self.num_steps - i)           # lower order for the final steps
        self.this_order = min(order, self.lower_order_nums + 1)
        self.last_sample = sample
        nxt = self._predict(sample, self.this_order)
        if self.lower_order_nums < self.order:
            self.lower_order_nums += 1
        self.step_index += 1
        return nxt


def _combine(terms: list) -> torch.Tensor:
    """sum of coef * tensor; fp32 device tensors go through the one-pass kernel."""
    from ... import ops
    xs = [t for _, t in terms]
    if xs[0].is_cuda and all(t.dtype == torch.float32 and t.is_contiguous() for t in xs):
        return ops.lincomb(terms)
    acc = terms[0][0] * terms[0][1]
    for c, t in terms[1:]:
        acc = acc + c * t
    return acc


class EulerDiscreteScheduler:
    """Epsilon-prediction Euler sampler over a scaled-linear beta schedule (SD 1.5 / SDXL)."""

    def __init__(self, num_steps: int, beta_start: float = 0.00085, beta_end: float = 0.012, train_steps: int = 1000):
        betas = torch.linspace(beta_start ** 0.5, beta_end ** 0.5, train_steps, dtype=torch.float64) ** 2
        ac = torch.cumprod(1 - betas, 0)
        sig_all = ((1 - ac) / ac) ** 0.5
        ts = torch.linspace(train_steps - 1, 0, num_steps, dtype=torch.float64)
        lo, hi = ts.floor().long(), ts.ceil().long()
        w = ts - lo
        self.sigmas = torch.cat([(1 - w) * sig_all[lo] + w * sig_all[hi], torch.zeros(1, dtype=torch.float64)]).float()
        self.timesteps = ts.float()
        self.init_noise_sigma = float((self.sigmas.max() ** 2 + 1) ** 0.5)

    def scale_input(self, x: torch.Tensor, i: int) -> torch.Tensor:
        return x / ((float(self.sigmas[i]) ** 2 + 1) ** 0.5)

    def step(self, eps: torch.Tensor, i: int, x: torch.Tensor) -> torch.Tensor:
        return x + eps.float() * float(self.sigmas[i + 1] - self.sigmas[i])


class DDIMScheduler:
    def __init__(self, num_steps: int, beta_start: float = 0.00085, beta_end: float = 0.012, train_steps: int = 1000,
                 v_prediction: bool = False):
        betas = torch.linspace(beta_start ** 0.5, beta_end ** 0.5, train_steps, dtype=torch.float64) ** 2
        self.ac = torch.cumprod(1 - betas, 0)
        step = train_steps // num_steps
        self.timesteps = (torch.arange(num_steps) * step).flip(0) + 1
        self.v_prediction = v_prediction

    def step(self, out: torch.Tensor, i: int, x: torch.Tensor) -> torch.Tensor:
        t = int(self.timesteps[i])
        prev = int(self.timesteps[i + 1]) if i + 1 < len(self.timesteps) else -1
        a_t = float(self.ac[min(t, len(self.ac) - 1)])
        a_p = float(self.ac[prev]) if prev >= 0 else 1.0
        o = out.float()
        if self.v_prediction:
            x0 = a_t ** 0.5 * x - (1 - a_t) ** 0.5 * o
            eps = a_t ** 0.5 * o + (1 - a_t) ** 0.5 * x
        else:
            eps = o
            x0 = (x - (1 - a_t) ** 0.5 * eps) / a_t ** 0.5
        return a_p ** 0.5 * x0 + (1 - a_p) ** 0.5 * eps


def make_scheduler(name: str, steps: int, **kw):
    name = name.lower()
    if name in ("flow_match_euler", "euler_flow", "flowmatch"):
        return FlowMatchEulerScheduler(steps, **kw)
    if name in ("unipc", "flow_unipc"):
        return FlowUniPCScheduler(steps, **kw)
    if name in ("euler", "euler_discrete"):
        return EulerDiscreteScheduler(steps, **kw)
    if name == "ddim":
        return DDIMScheduler(steps, **kw)
    if name in ("dpm++2m", "dpmpp_2m", "dpm_solver_multistep"):
        return DPMSolverMultistepScheduler(steps, **kw)
    if name == "lcm":
        return LCMScheduler(steps, **kw)
    raise ValueError(f"unknown scheduler '{name}'")


class DPMSolverMultistepScheduler:
    """DPM-Solver++ (2M) for epsilon- or v-prediction models on the scaled-linear beta schedule:
    data prediction ``x0``, half log-SNR ``lambda = log(alpha / sigma)``, second-order multistep
    update with a first-order first and last step
    (src/HartsyInference.Diffusion/Schedulers/DpmSolverMultistepScheduler.cs)."""

    def __init__(self, num_steps: int, beta_start: float = 0.00085, beta_end: float = 0.012, train_steps: int = 1000,
                 prediction: str = "epsilon"):
        betas = torch.linspace(beta_start ** 0.5, beta_end ** 0.5, train_steps, dtype=torch.float64) ** 2
        ac = torch.cumprod(1 - betas, 0)
        ts = torch.linspace(train_steps - 1, 0, num_steps + 1, dtype=torch.float64).round().long()[:-1]
        self.timesteps = ts
        a = ac[ts] ** 0.5
        s = (1 - ac[ts]) ** 0.5
        self.alpha = torch.cat([a, torch.ones(1, dtype=torch.float64)])
        self.sigma = torch.cat([s, torch.zeros(1, dtype=torch.float64)])
        self.lam = torch.log(self.alpha.clamp_min(1e-20)) - torch.log(self.sigma.clamp_min(1e-20))
        self.prediction = prediction
        self.num_steps = num_steps
        self._prev_x0: Optional[torch.Tensor] = None

    def timestep(self, i: int) -> float:
        return float(self.timesteps[i])

    def _x0(self, out: torch.Tensor, x: torch.Tensor, i: int) -> torch.Tensor:
        a, s = float(self.alpha[i]), float(self.sigma[i])
        if self.prediction == "v_prediction":
            return a * x - s * out
        return (x - s * out) / a

    def step(self, out: torch.Tensor, i: int, x: torch.Tensor) -> torch.Tensor:
        x0 = self._x0(out.float(), x.float(), i)
        a_n, s_n, s_c = float(self.alpha[i + 1]), float(self.sigma[i + 1]), float(self.sigma[i])
        last = i == self.num_steps - 1
        if last:
            self._prev_x0 = None
            return x0.to(x.dtype)                       # sigma_next = 0: the sample is the data prediction
        h = float(self.lam[i + 1] - self.lam[i])
        if self._prev_x0 is None or i == self.num_steps - 2:
            d = x0                                      # first-order (also "lower order final")
        else:
            h0 = float(self.lam[i] - self.lam[i - 1])
            r = h0 / h
            d = x0 + (x0 - self._prev_x0) / (2 * r)
        self._prev_x0 = x0
        return ((s_n / s_c) * x.float() - a_n * math.expm1(-h) * d).to(x.dtype)


class LCMScheduler:
    """Latent-consistency sampling: predict x0, then re-noise to the next timestep (the last step
    returns x0). Boundary-condition scalings ``c_skip`` / ``c_out`` with sigma_data 0.5 and
    timestep scaling 10 (src/HartsyInference.Diffusion/Schedulers/LcmScheduler.cs)."""

    def __init__(self, num_steps: int, beta_start: float = 0.00085, beta_end: float = 0.012, train_steps: int = 1000,
                 original_steps: int = 50, seed: int = 0):
        betas = torch.linspace(beta_start ** 0.5, beta_end ** 0.5, train_steps, dtype=torch.float64) ** 2
        self.ac = torch.cumprod(1 - betas, 0)
        k = train_steps // original_steps
        lcm_ts = (torch.arange(1, original_steps + 1) * k - 1).flip(0)
        idx = torch.linspace(0, original_steps, num_steps + 1).floor().long()[:-1]
        self.timesteps = lcm_ts[idx]
        self.num_steps = num_steps
        self.gen = torch.Generator().manual_seed(seed)

    def timestep(self, i: int) -> float:
        return float(self.timesteps[i])

    def step(self, eps: torch.Tensor, i: int, x: torch.Tensor) -> torch.Tensor:
        t = int(self.timesteps[i])
        a_t = float(self.ac[t])
        x0 = (x.float() - (1 - a_t) ** 0.5 * eps.float()) / a_t ** 0.5
        sd, ts = 0.5, t * 10.0
        c_skip = sd * sd / (ts * ts + sd * sd)
        c_out = ts / (ts * ts + sd * sd) ** 0.5
        den = c_out * x0 + c_skip * x.float()
        if i == self.num_steps - 1:
            return den.to(x.dtype)
        a_p = float(self.ac[int(self.timesteps[i + 1])])
        noise = torch.randn(x.shape, generator=self.gen, dtype=torch.float32).to(x.device)
        return (a_p ** 0.5 * den + (1 - a_p) ** 0.5 * noise).to(x.dtype)


class TCDScheduler(LCMScheduler):
    """Trajectory-consistency sampling: like LCM, but each step first jumps to an intermediate
    timestep ``s = (1 - gamma) t_next`` deterministically and only re-noises from there; ``gamma``
    0 is deterministic multi-step consistency, 1 is LCM's full re-noising
    (src/HartsyInference.Diffusion/Schedulers/TcdScheduler.cs)."""

    def __init__(self, num_steps: int, gamma: float = 0.3, **kw):
        super().__init__(num_steps, **kw)
        self.gamma = gamma

    def step(self, eps: torch.Tensor, i: int, x: torch.Tensor) -> torch.Tensor:
        t = int(self.timesteps[i])
        a_t = float(self.ac[t])
        e = eps.float()
        x0 = (x.float() - (1 - a_t) ** 0.5 * e) / a_t ** 0.5
        if i == self.num_steps - 1:
            return x0.to(x.dtype)
        t_next = int(self.timesteps[i + 1])
        s = int((1.0 - self.gamma) * t_next)
        a_s, a_n = float(self.ac[s]), float(self.ac[t_next])
        x_s = a_s ** 0.5 * x0 + (1 - a_s) ** 0.5 * e                      # deterministic jump to s
        if self.gamma <= 0:
            return x_s.to(x.dtype)
        noise = torch.randn(x.shape, generator=self.gen, dtype=torch.float32).to(x.device)
        ratio = a_n / a_s
        return (ratio ** 0.5 * x_s + (1 - ratio) ** 0.5 * noise).to(x.dtype)   # forward diffusion s -> t_next


class FlowDPMSolverMultistepScheduler:
    """DPM-Solver++ (2M) on the flow-matching parameterisation ``x_t = (1 - sigma) x0 + sigma eps``
    with a velocity model: ``x0 = x - sigma v``, half log-SNR ``lambda = log((1 - sigma) / sigma)``
    (src/HartsyInference.Diffusion/Schedulers/FlowDpmPlusPlus2MScheduler.cs)."""

    def __init__(self, num_steps: int, shift: float = 1.0, mu: Optional[float] = None):
        base = FlowMatchEulerScheduler(num_steps, shift=shift, mu=mu)
        self.sigmas = base.sigmas.double()
        self.num_steps = num_steps
        self._prev_x0: Optional[torch.Tensor] = None

    def sigma(self, i: int) -> float:
        return float(self.sigmas[i])

    def timestep(self, i: int) -> float:
        return float(self.sigmas[i]) * 1000.0

    def _lam(self, i: int) -> float:
        s = min(max(float(self.sigmas[i]), 1e-8), 1 - 1e-8)
        return math.log((1 - s) / s)

    def step(self, velocity: torch.Tensor, i: int, x: torch.Tensor) -> torch.Tensor:
        s_c, s_n = float(self.sigmas[i]), float(self.sigmas[i + 1])
        x0 = x.float() - s_c * velocity.float()
        if i == self.num_steps - 1 or s_n <= 0:
            self._prev_x0 = None
            return x0.to(x.dtype)
        h = self._lam(i + 1) - self._lam(i)
        if self._prev_x0 is None or i == self.num_steps - 2:
            d = x0
        else:
            r = (self._lam(i) - self._lam(i - 1)) / h
            d = x0 + (x0 - self._prev_x0) / (2 * r)
        self._prev_x0 = x0
        return ((s_n / s_c) * x.float() - (1 - s_n) * math.expm1(-h) * d).to(x.dtype)


class FlowMatchPingPongScheduler(FlowMatchEulerScheduler):
    """Ping-pong sampling for flow models (the few-step Stable Audio / distilled samplers): denoise
    fully to ``x0 = x - sigma v``, then re-noise to the next sigma with fresh noise
    (src/HartsyInference.Diffusion/Schedulers/FlowMatchPingPongScheduler.cs, StableAudioPingPongScheduler.cs)."""

    def __init__(self, num_steps: int, seed: int = 0, **kw):
        super().__init__(num_steps, **kw)
        self.gen = torch.Generator().manual_seed(seed)

    def step(self, latents: torch.Tensor, cond: torch.Tensor, i: int, uncond: Optional[torch.Tensor] = None,
             guidance: float = 1.0) -> torch.Tensor:
        v = cond.float() if uncond is None else uncond.float() + guidance * (cond.float() - uncond.float())
        s_c, s_n = self.sigma(i), float(self.sigmas[i + 1])
        x0 = latents.float() - s_c * v.reshape(latents.shape)
        if s_n <= 0:
            latents.copy_(x0)
            return latents
        noise = torch.randn(latents.shape, generator=self.gen, dtype=torch.float32).to(latents.device)
        latents.copy_((1 - s_n) * x0 + s_n * noise)
        return latents


class EulerAncestralScheduler(EulerDiscreteScheduler):
    """Euler with ancestral noise: step down to ``sigma_down`` and add ``sigma_up`` of fresh noise,
    ``sigma_up^2 = sigma_next^2 (sigma^2 - sigma_next^2) / sigma^2``
    (the reference's samplers: euler_a)."""

    def __init__(self, num_steps: int, seed: int = 0, eta: float = 1.0, **kw):
        super().__init__(num_steps, **kw)
        self.gen, self.eta = torch.Generator().manual_seed(seed), eta

    def step(self, eps: torch.Tensor, i: int, x: torch.Tensor) -> torch.Tensor:
        s, sn = float(self.sigmas[i]), float(self.sigmas[i + 1])
        up = min(sn, self.eta * (sn ** 2 * (s ** 2 - sn ** 2) / s ** 2) ** 0.5) if s > 0 else 0.0
        down = (sn ** 2 - up ** 2) ** 0.5
        x = x + eps.float() * (down - s)
        if up > 0:
            x = x + torch.randn(x.shape, generator=self.gen, dtype=torch.float32).to(x.device) * up
        return x


class HeunScheduler(EulerDiscreteScheduler):
    """Heun's second-order method on the sigma ODE ``dx / dsigma = eps``: an Euler predictor, a
    second model call at the predicted point, and the trapezoidal corrector (first order on the
    last step, where sigma_next = 0). ``step`` takes a callable for the second evaluation."""

    def step(self, eps: torch.Tensor, i: int, x: torch.Tensor, model=None) -> torch.Tensor:
        s, sn = float(self.sigmas[i]), float(self.sigmas[i + 1])
        x_e = x + eps.float() * (sn - s)
        if model is None or sn == 0:
            return x_e
        eps2 = model(x_e, i + 1).float()
        return x + 0.5 * (eps.float() + eps2) * (sn - s)


def logit_normal_sigmas(num_steps: int, mean: float = 0.0, std: float = 1.0, shift: float = 1.0) -> torch.Tensor:
    """Inference sigmas placed at the quantiles of a logit-normal density (the density SD3-class
    models are trained on), descending from 1 to 0, with the usual resolution shift
    (src/HartsyInference.Diffusion/Schedulers/LogitNormalSchedule.cs)."""
    q = torch.linspace(1.0, 0.0, num_steps + 1, dtype=torch.float64)[1:-1]
    z = mean + std * math.sqrt(2.0) * torch.erfinv(2 * q - 1)
    sig = torch.sigmoid(z)
    sig = torch.cat([torch.ones(1, dtype=torch.float64), sig, torch.zeros(1, dtype=torch.float64)])
    return (shift * sig / (1 + (shift - 1) * sig)).float()


_MORE = {"tcd": TCDScheduler, "flow_dpm++2m": FlowDPMSolverMultistepScheduler, "flow_dpmpp_2m": FlowDPMSolverMultistepScheduler,
         "pingpong": FlowMatchPingPongScheduler, "flow_match_pingpong": FlowMatchPingPongScheduler,
         "euler_a": EulerAncestralScheduler, "euler_ancestral": EulerAncestralScheduler, "heun": HeunScheduler,
         "ddim_v": lambda steps, **kw: DDIMScheduler(steps, v_prediction=True, **kw)}
_make_base = make_scheduler


def make_scheduler(name: str, steps: int, **kw):  # noqa: F811 - the factory, extended with the classes above
    cls = _MORE.get(name.lower())
    return cls(steps, **kw) if cls is not None else _make_base(name, steps, **kw)
