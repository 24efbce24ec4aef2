"""Rectified-flow (flow matching) noise schedule for training and Euler sampling.

Same maths and method names as the reference scheduler (teletron/models/flow_match.py:5-79):
sigmas run linearly from sigma_start to sigma_min and are warped by
``sigma' = shift * sigma / (1 + (shift - 1) * sigma)``; timesteps are ``sigma * 1000``; the
training weights are a Gaussian bump over the timestep index normalised to mean 1;
``add_noise = (1 - sigma) x0 + sigma noise``; the regression target is ``noise - x0``; ``step``
is one Euler step of the learnt velocity.  ``sigma_of`` exposes the per-sample sigma so the
fused noising / loss kernels (``teletron_b200.ops.flow``) can be used.
"""
from __future__ import annotations

import torch


class FlowMatchScheduler:
    def __init__(self, num_inference_steps=100, num_train_timesteps=1000, shift=3.0, sigma_max=1.0,
                 sigma_min=0.003 / 1.002, inverse_timesteps=False, extra_one_step=False,
                 reverse_sigmas=False):
        self.num_train_timesteps = num_train_timesteps
        self.shift = shift
        self.sigma_max, self.sigma_min = sigma_max, sigma_min
        self.inverse_timesteps = inverse_timesteps
        self.extra_one_step = extra_one_step
        self.reverse_sigmas = reverse_sigmas
        self.linear_timesteps_weights = None
        self.set_timesteps(num_inference_steps)

    def set_timesteps(self, num_inference_steps=100, denoising_strength=1.0, training=False, shift=None):
        if shift is not None:
            self.shift = shift
        start = self.sigma_min + (self.sigma_max - self.sigma_min) * denoising_strength
        n = num_inference_steps + 1 if self.extra_one_step else num_inference_steps
        sig = torch.linspace(start, self.sigma_min, n)
        if self.extra_one_step:
            sig = sig[:-1]
        if self.inverse_timesteps:
            sig = sig.flip(0)
        sig = self.shift * sig / (1 + (self.shift - 1) * sig)
        if self.reverse_sigmas:
            sig = 1 - sig
        self.sigmas = sig
        self.timesteps = sig * self.num_train_timesteps
        if training:
            t = self.timesteps
            bump = torch.exp(-2 * ((t - num_inference_steps / 2) / num_inference_steps) ** 2)
            bump = bump - bump.min()
            self.linear_timesteps_weights = bump * (num_inference_steps / bump.sum())

    def _index(self, timestep) -> torch.Tensor:
        if isinstance(timestep, torch.Tensor):
            timestep = timestep.detach().float().cpu()
        else:
            timestep = torch.tensor(float(timestep))
        return torch.argmin((self.timesteps - timestep.reshape(-1)[0]).abs())

    def sigma_of(self, timestep) -> torch.Tensor:
        return self.sigmas[self._index(timestep)]

    def step(self, model_output, timestep, sample, to_final=False, **_):
        i = self._index(timestep)
        sigma = self.sigmas[i]
        if to_final or i + 1 >= len(self.timesteps):
            nxt = 1.0 if (self.inverse_timesteps or self.reverse_sigmas) else 0.0
        else:
            nxt = self.sigmas[i + 1]
        return sample + model_output * (nxt - sigma)

    def return_to_timestep(self, timestep, sample, sample_stablized):
        return (sample - sample_stablized) / self.sigma_of(timestep)

    def add_noise(self, original_samples, noise, timestep):
        sigma = self.sigma_of(timestep)
        return (1 - sigma) * original_samples + sigma * noise

    def training_target(self, sample, noise, timestep=None):
        return noise - sample

    def training_weight(self, timestep):
        assert self.linear_timesteps_weights is not None, "call set_timesteps(..., training=True) first"
        return self.linear_timesteps_weights[self._index(timestep)]
