"""Toy transformers for the six block contracts, and seeded runs through `enable_cache`.

The same module classes and the same seeded inputs are run through the reference's
`cache_dit.enable_cache` (by tests/golden/make_golden.py, where the reference exists) and through
`cache_dit_b200.enable_cache` (by the tests); since every cache operation is reproduced with the
reference's rounding, the two trajectories coincide and masks, diffs and outputs can be compared.
"""
from __future__ import annotations

from typing import Dict, List, Tuple

import numpy as np
import torch
from torch import nn

TORCH_DTYPE = {"fp32": torch.float32, "bf16": torch.bfloat16}


class ToyBlock(nn.Module):
  """h <- h + a * tanh(W h) (and the same for the encoder stream), returned per `pattern`."""

  def __init__(self, dim: int, pattern: int, gain: float):
    super().__init__()
    self.lin = nn.Linear(dim, dim)
    self.enc = nn.Linear(dim, dim)
    self.pattern = pattern
    self.gain = gain

  def _mix(self, hidden_states, encoder_hidden_states):
    h = hidden_states + self.gain * torch.tanh(self.lin(hidden_states))
    if encoder_hidden_states is None:  # patterns 4/5 create the encoder stream from the hidden one
      e = self.gain * torch.tanh(self.enc(hidden_states[:, :3]))
    else:
      e = encoder_hidden_states + self.gain * torch.tanh(self.enc(encoder_hidden_states))
    return h, e


class Block01(ToyBlock):

  def forward(self, hidden_states, encoder_hidden_states, scale=1.0):
    h, e = self._mix(hidden_states * scale, encoder_hidden_states)
    return (h, e) if self.pattern == 0 else (e, h)


class Block2(ToyBlock):

  def forward(self, hidden_states, encoder_hidden_states, scale=1.0):
    h, _ = self._mix(hidden_states * scale, encoder_hidden_states)
    return h


class Block345(ToyBlock):

  def forward(self, hidden_states, scale=1.0):
    h, e = self._mix(hidden_states * scale, None)
    if self.pattern == 3:
      return h
    return (h, e) if self.pattern == 4 else (e, h)


class ToyTransformer(nn.Module):

  def __init__(self, pattern: int, dim: int = 32, n_blocks: int = 10, gain: float = 0.05):
    super().__init__()
    cls = Block01 if pattern in (0, 1) else (Block2 if pattern == 2 else Block345)
    self.pattern = pattern
    self.transformer_blocks = nn.ModuleList([cls(dim, pattern, gain) for _ in range(n_blocks)])

  def forward(self, hidden_states, encoder_hidden_states=None, scale=1.0):
    h, e = hidden_states, encoder_hidden_states
    for block in self.transformer_blocks:
      if self.pattern == 0:
        h, e = block(h, e, scale=scale)
      elif self.pattern == 1:
        e, h = block(h, e, scale=scale)
      elif self.pattern == 2:
        h = block(h, e, scale=scale)
      elif self.pattern == 3:
        h = block(h, scale=scale)
      elif self.pattern == 4:
        h, e = block(h, scale=scale)
      else:
        e, h = block(h, scale=scale)
    return h if e is None else (h, e)


# name, pattern, dtype, steps, cache-config kwargs, calibrator kwargs (None: no calibrator), cfg
RUNS: List[dict] = [
  dict(name="p0_fp32_F2B0_o1", pattern=0, dtype="fp32", steps=16, cc=dict(Fn_compute_blocks=2, max_warmup_steps=3),
       cal=dict(taylorseer_order=1)),
  dict(name="p1_bf16_F2B1_o1", pattern=1, dtype="bf16", steps=16,
       cc=dict(Fn_compute_blocks=2, Bn_compute_blocks=1, max_warmup_steps=3), cal=dict(taylorseer_order=1)),
  dict(name="p1_fp32_F1B0_plain", pattern=1, dtype="fp32", steps=14, cc=dict(Fn_compute_blocks=1, max_warmup_steps=2),
       cal=None),
  dict(name="p2_bf16_F1B0_o2", pattern=2, dtype="bf16", steps=18, cc=dict(Fn_compute_blocks=1, max_warmup_steps=4),
       cal=dict(taylorseer_order=2)),
  dict(name="p2_fp32_F3B2_o1_cfg", pattern=2, dtype="fp32", steps=12,
       cc=dict(Fn_compute_blocks=3, Bn_compute_blocks=2, max_warmup_steps=2, enable_separate_cfg=True,
               residual_diff_threshold=0.25),
       cal=dict(taylorseer_order=1)),
  dict(name="p3_bf16_F2B0_o1", pattern=3, dtype="bf16", steps=16, cc=dict(Fn_compute_blocks=2, max_warmup_steps=3),
       cal=dict(taylorseer_order=1)),
  dict(name="p4_fp32_F2B1_o1", pattern=4, dtype="fp32", steps=16,
       cc=dict(Fn_compute_blocks=2, Bn_compute_blocks=1, max_warmup_steps=3), cal=dict(taylorseer_order=1)),
  dict(name="p5_bf16_F2B0_hidden", pattern=5, dtype="bf16", steps=16, cc=dict(Fn_compute_blocks=2, max_warmup_steps=3),
       cal=dict(taylorseer_order=1, calibrator_cache_type="hidden_states")),
  dict(name="p0_bf16_F8B0_default", pattern=0, dtype="bf16", steps=28, cc=dict(), cal=dict(taylorseer_order=1)),
  dict(name="p1_bf16_two_runs", pattern=1, dtype="bf16", steps=10, cc=dict(Fn_compute_blocks=2, max_warmup_steps=2),
       cal=dict(taylorseer_order=1), runs=2),
]
BY_NAME: Dict[str, dict] = {r["name"]: r for r in RUNS}


def build(run: dict) -> ToyTransformer:
  torch.manual_seed(1000 + run["pattern"])
  model = ToyTransformer(run["pattern"])
  return model.to(TORCH_DTYPE[run["dtype"]])


def inputs(run: dict):
  """Per call: (hidden, encoder-or-None, scale).  A slow drift plus a per-step input scale."""
  dt = TORCH_DTYPE[run["dtype"]]
  g = torch.Generator().manual_seed(2000 + run["pattern"])
  branches = 2 if run["cc"].get("enable_separate_cfg") else 1
  h = [torch.randn(1, 12, 32, generator=g) for _ in range(branches)]
  e = [torch.randn(1, 3, 32, generator=g) for _ in range(branches)]
  for step in range(run["steps"]):
    for b in range(branches):
      h[b] = h[b] + 0.012 * torch.randn(1, 12, 32, generator=g)
      e[b] = e[b] + 0.012 * torch.randn(1, 3, 32, generator=g)
      enc = e[b].to(dt) if run["pattern"] in (0, 1, 2) else None
      yield h[b].to(dt), enc, 1.0 + 0.002 * step


def execute(run: dict, cache_dit, device="cpu") -> Tuple[dict, Dict[str, np.ndarray]]:
  """Enable the cache with `cache_dit` (the reference or cache_dit_b200) and run the schedule."""
  model = build(run).to(device)
  cc = dict(run["cc"])
  branches = 2 if cc.get("enable_separate_cfg") else 1
  cc.setdefault("enable_separate_cfg", False)
  cc["num_inference_steps"] = run["steps"]
  pattern = getattr(cache_dit.ForwardPattern, f"Pattern_{run['pattern']}")
  adapter = cache_dit.BlockAdapter(transformer=model, blocks=model.transformer_blocks, forward_pattern=pattern,
                                   check_forward_pattern=False)
  cal = None if run["cal"] is None else cache_dit.TaylorSeerCalibratorConfig(**run["cal"])
  cache_dit.enable_cache(adapter, cache_config=cache_dit.DBCacheConfig(**cc), calibrator_config=cal)
  outs: Dict[str, np.ndarray] = {}
  stats = []
  for r in range(run.get("runs", 1)):
    cache_dit.refresh_context(model, num_inference_steps=run["steps"])
    with torch.no_grad():
      for call, (h, e, scale) in enumerate(inputs(run)):
        y = model(h.to(device), None if e is None else e.to(device), scale=scale)
        y = y if isinstance(y, tuple) else (y, )
        for tag, t in zip("he", y):
          outs[f"r{r}{tag}{call}"] = t.detach().float().cpu().numpy()
    stats.append(dict(
      cached_steps=[int(s) for s in model._cached_steps],
      residual_diffs={str(k): float(v) for k, v in model._residual_diffs.items()},
      cfg_cached_steps=[int(s) for s in model._cfg_cached_steps],
      cfg_residual_diffs={str(k): float(v) for k, v in model._cfg_residual_diffs.items()},
      accumulated_cached_steps=int(model._accumulated_cached_steps),
      accumulated_executed_steps=int(model._accumulated_executed_steps),
      accumulated_transformer_executed_steps=int(model._accumulated_transformer_executed_steps),
    ))
  # the reference flags the (shared) stand-in pipeline class as cached: release it for the next run
  cache_dit.disable_cache(adapter)
  assert not hasattr(model, "_cached_steps") and not getattr(model, "_is_cached", False)
  return dict(name=run["name"], stats=stats, calls=run["steps"] * branches), outs


def run_reference(cache_dit):
  runs, arrays = {}, {}
  for run in RUNS:
    trace, outs = execute(run, cache_dit)
    runs[run["name"]] = trace
    for k, v in outs.items():
      arrays[f"{run['name']}/{k}"] = v
    print(run["name"], trace["stats"][-1]["cached_steps"], trace["stats"][-1]["cfg_cached_steps"])
  return runs, arrays
