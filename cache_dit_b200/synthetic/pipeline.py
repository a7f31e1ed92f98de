"""A minimal flow-matching denoising loop around a transformer stand-in.

It plays the role of the diffusion pipeline for the hot path: `enable_cache(pipe)` wraps
`__call__` so that every generation starts from fresh cache contexts, the loop calls the
transformer once per step (twice with a separate classifier-free-guidance call), and the scheduler
is the Euler step `x <- x + (sigma_next - sigma) * v`.
"""
from __future__ import annotations

from typing import Callable, Dict, Optional

import torch


class DenoisePipeline:

  def __init__(self, transformer: torch.nn.Module, inputs: Dict[str, torch.Tensor], latent_key: str = "hidden_states",
               separate_cfg: bool = False, guidance_scale: float = 4.0):
    self.transformer = transformer
    self.inputs = inputs
    self.latent_key = latent_key
    self.separate_cfg = separate_cfg
    self.guidance_scale = guidance_scale

  @staticmethod
  def sigmas(num_inference_steps: int, shift: float = 3.0) -> torch.Tensor:
    s = torch.linspace(1.0, 0.0, num_inference_steps + 1)
    return shift * s / (1 + (shift - 1) * s)

  @torch.no_grad()
  def __call__(self, num_inference_steps: int = 28, latents: Optional[torch.Tensor] = None,
               callback: Optional[Callable[[int, torch.Tensor], None]] = None) -> torch.Tensor:
    kw = dict(self.inputs)
    x = kw.pop(self.latent_key) if latents is None else latents
    kw.pop(self.latent_key, None)
    sig = self.sigmas(num_inference_steps)
    for i in range(num_inference_steps):
      t = torch.full((x.shape[0], ), float(sig[i]), device=x.device)
      v = self.transformer(**{self.latent_key: x}, timestep=t, **kw)
      if self.separate_cfg:
        neg = dict(kw)
        if "encoder_hidden_states" in neg:
          neg["encoder_hidden_states"] = torch.zeros_like(neg["encoder_hidden_states"])
        v_neg = self.transformer(**{self.latent_key: x}, timestep=t, **neg)
        v = v_neg + self.guidance_scale * (v - v_neg)
      x = (x.float() + float(sig[i + 1] - sig[i]) * v.float()).to(x.dtype)
      if callback is not None:
        callback(i, x)
    return x


class FluxDenoisePipeline(DenoisePipeline):
  pass


class QwenImageDenoisePipeline(DenoisePipeline):

  def __init__(self, transformer, inputs, **kw):
    super().__init__(transformer, inputs, separate_cfg=kw.pop("separate_cfg", True), **kw)


class WanDenoisePipeline(DenoisePipeline):

  def __init__(self, transformer, inputs, **kw):
    super().__init__(transformer, inputs, separate_cfg=kw.pop("separate_cfg", True), **kw)
