"""Per-context DBCache state: counters, cached-step history, buffers and calibrators.

This is the integer bookkeeping of the reference's `CachedContext`
(src/cache_dit/caching/cache_contexts/cache_context.py:26-360) restated around two small helper
objects: `BranchStats` holds what exists once per classifier-free-guidance branch, and the context
picks the active branch from the parity of the transformer call counter.  Attribute names used by
user code and by the statistics read-out (`cached_steps`, `residual_diffs`, `cfg_*`,
`accumulated_*`) are kept as properties.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional, Tuple

import torch

from .cache_config import BasicCacheConfig, ExtraCacheConfig
from .calibrators import Calibrator, CalibratorBase, CalibratorConfig


@dataclasses.dataclass
class BranchStats:
  """History of one branch (conditional, or the separate unconditional/CFG call)."""
  cached_steps: List[int] = dataclasses.field(default_factory=list)
  residual_diffs: Dict[str, float] = dataclasses.field(default_factory=dict)
  accumulated_residual_diff: float = 0.0
  continuous_cached_steps: int = 0
  accumulated_cached_steps: int = 0
  calibrator: Optional[CalibratorBase] = None
  encoder_calibrator: Optional[CalibratorBase] = None

  def start_run(self):
    self.cached_steps.clear()
    self.residual_diffs.clear()
    for c in (self.calibrator, self.encoder_calibrator):
      if c is not None:
        c.reset_cache()

  def begin_step(self):
    for c in (self.calibrator, self.encoder_calibrator):
      if c is not None:
        c.mark_step_begin()

  def record_diff(self, step: int, diff: float):
    key = str(step)
    if key not in self.residual_diffs:  # the first value recorded for a step wins
      self.residual_diffs[key] = diff
      if diff > 0.0:
        self.accumulated_residual_diff += diff

  def record_hit(self, step: int):
    # run length of consecutive cached steps; the first consecutive pair counts as two
    if not self.cached_steps:
      self.continuous_cached_steps += 1
    elif step - self.cached_steps[-1] == 1:
      self.continuous_cached_steps += 2 if self.continuous_cached_steps == 0 else 1
    self.cached_steps.append(step)
    self.accumulated_cached_steps += 1


class CachedContext:
  """Runtime state of one cache-enabled block list."""

  def __init__(self, name: str = "default", cache_config: Optional[BasicCacheConfig] = None,
               extra_cache_config: Optional[ExtraCacheConfig] = None,
               calibrator_config: Optional[CalibratorConfig] = None, **unused):
    self.name = name
    self.cache_config = cache_config if cache_config is not None else BasicCacheConfig()
    self.extra_cache_config = extra_cache_config if extra_cache_config is not None else ExtraCacheConfig()
    self.calibrator_config = calibrator_config
    self.buffers: Dict[str, Any] = {}
    self.executed_steps = 0
    self.transformer_executed_steps = 0
    self.accumulated_executed_steps = 0
    self.accumulated_transformer_executed_steps = 0
    self.main = BranchStats()
    self.cfg = BranchStats()
    cc = self.cache_config
    if cc.enable_separate_cfg and cc.cfg_diff_compute_separate:
      assert cc.cfg_compute_first is False, ("cfg_compute_first must set as False if "
                                             "cfg_diff_compute_separate is enabled.")
    cal = calibrator_config
    if cal is not None:
      branches = [self.main] + ([self.cfg] if cc.enable_separate_cfg else [])
      for branch in branches:
        if cal.enable_calibrator:
          branch.calibrator = Calibrator(cal)
        if cal.enable_encoder_calibrator:
          branch.encoder_calibrator = Calibrator(cal)

  # ---- calibrator switches -----------------------------------------------------------------
  def enable_calibrator(self) -> bool:
    return bool(self.calibrator_config is not None and self.calibrator_config.enable_calibrator)

  def enable_encoder_calibrator(self) -> bool:
    return bool(self.calibrator_config is not None and self.calibrator_config.enable_encoder_calibrator)

  def calibrator_cache_type(self) -> str:
    return self.calibrator_config.calibrator_cache_type if self.calibrator_config is not None else "residual"

  def has_calibrators(self) -> bool:
    return self.enable_calibrator() or self.enable_encoder_calibrator()

  def get_calibrators(self) -> Tuple[Optional[CalibratorBase], Optional[CalibratorBase]]:
    return self.main.calibrator, self.main.encoder_calibrator

  def get_cfg_calibrators(self) -> Tuple[Optional[CalibratorBase], Optional[CalibratorBase]]:
    return self.cfg.calibrator, self.cfg.encoder_calibrator

  # ---- step counters -------------------------------------------------------------------------
  def get_current_step(self) -> int:
    return self.executed_steps - 1

  def get_current_transformer_step(self) -> int:
    return self.transformer_executed_steps - 1

  def is_separate_cfg_step(self) -> bool:
    """Whether the current transformer call is the separate CFG call of its step."""
    cc = self.cache_config
    if not cc.enable_separate_cfg:
      return False
    odd = self.get_current_transformer_step() % 2 != 0
    return (not odd) if cc.cfg_compute_first else odd

  def branch(self) -> BranchStats:
    return self.cfg if self.is_separate_cfg_step() else self.main

  def mark_step_begin(self):
    """Advance the counters for one transformer call (cache_context.py:146-212 of the reference)."""
    cc = self.cache_config
    self.transformer_executed_steps += 1
    self.accumulated_transformer_executed_steps += 1
    # with separate CFG a step is two calls; it is counted on the call that comes first
    if not cc.enable_separate_cfg or (self.is_separate_cfg_step() == bool(cc.cfg_compute_first)):
      self.executed_steps += 1
      self.accumulated_executed_steps += 1
    if self.get_current_transformer_step() == 0:
      self.main.start_run()
      self.cfg.start_run()
    if self.has_calibrators():
      (self.branch() if cc.enable_separate_cfg else self.main).begin_step()

  @property
  def warmup_steps(self) -> List[int]:
    cc = self.cache_config
    limit = cc.max_warmup_steps
    if cc.steps_computation_mask is not None:
      lead = 0
      for m in cc.steps_computation_mask:
        if m != 1:
          break
        lead += 1
      limit = min(limit, lead)
    return list(range(0, limit, cc.warmup_interval))

  def is_in_warmup(self) -> bool:
    return self.get_current_step() in self.warmup_steps

  def is_in_full_compute_steps(self) -> bool:
    mask = self.cache_config.steps_computation_mask
    step = self.get_current_step()
    return mask is not None and step < len(mask) and mask[step] == 1

  def get_steps_computation_policy(self) -> str:
    return self.cache_config.steps_computation_policy

  def get_force_refresh_step_hint(self) -> Optional[int]:
    return self.cache_config.force_refresh_step_hint

  def get_residual_diff_threshold(self) -> float:
    threshold = self.cache_config.residual_diff_threshold
    if self.extra_cache_config.l1_hidden_states_diff_threshold is not None:
      threshold = self.extra_cache_config.l1_hidden_states_diff_threshold
    if isinstance(threshold, torch.Tensor):
      threshold = threshold.item()
    return threshold

  # ---- history -------------------------------------------------------------------------------
  def add_residual_diff(self, diff):
    if isinstance(diff, torch.Tensor):
      diff = diff.item()
    self.branch().record_diff(self.get_current_step(), diff)

  def add_cached_step(self):
    self.branch().record_hit(self.get_current_step())

  # ---- buffers -------------------------------------------------------------------------------
  def get_buffer(self, name):
    return self.buffers.get(name)

  def set_buffer(self, name, buffer):
    self.buffers[name] = buffer

  def remove_buffer(self, name):
    self.buffers.pop(name, None)

  def clear_buffers(self):
    self.buffers.clear()

  # ---- names the statistics read-out and user code rely on --------------------------------------
  cached_steps = property(lambda s: s.main.cached_steps, lambda s, v: setattr(s.main, "cached_steps", v))
  residual_diffs = property(lambda s: s.main.residual_diffs, lambda s, v: setattr(s.main, "residual_diffs", v))
  accumulated_residual_diff = property(lambda s: s.main.accumulated_residual_diff,
                                       lambda s, v: setattr(s.main, "accumulated_residual_diff", v))
  continuous_cached_steps = property(lambda s: s.main.continuous_cached_steps,
                                     lambda s, v: setattr(s.main, "continuous_cached_steps", v))
  accumulated_cached_steps = property(lambda s: s.main.accumulated_cached_steps,
                                      lambda s, v: setattr(s.main, "accumulated_cached_steps", v))
  cfg_cached_steps = property(lambda s: s.cfg.cached_steps, lambda s, v: setattr(s.cfg, "cached_steps", v))
  cfg_residual_diffs = property(lambda s: s.cfg.residual_diffs,
                                lambda s, v: setattr(s.cfg, "residual_diffs", v))
  cfg_accumulated_residual_diff = property(lambda s: s.cfg.accumulated_residual_diff,
                                           lambda s, v: setattr(s.cfg, "accumulated_residual_diff", v))
  cfg_continuous_cached_steps = property(lambda s: s.cfg.continuous_cached_steps,
                                         lambda s, v: setattr(s.cfg, "continuous_cached_steps", v))
  cfg_accumulated_cached_steps = property(lambda s: s.cfg.accumulated_cached_steps,
                                          lambda s, v: setattr(s.cfg, "accumulated_cached_steps", v))
  calibrator = property(lambda s: s.main.calibrator)
  encoder_calibrator = property(lambda s: s.main.encoder_calibrator)
  cfg_calibrator = property(lambda s: s.cfg.calibrator)
  cfg_encoder_calibrator = property(lambda s: s.cfg.encoder_calibrator)

  def get_cached_steps(self):
    return list(self.main.cached_steps)

  def get_cfg_cached_steps(self):
    return list(self.cfg.cached_steps)

  def get_residual_diffs(self):
    return dict(self.main.residual_diffs)

  def get_cfg_residual_diffs(self):
    return dict(self.cfg.residual_diffs)

  def get_accumulated_residual_diff(self):
    return self.main.accumulated_residual_diff

  def get_cfg_accumulated_residual_diff(self):
    return self.cfg.accumulated_residual_diff

  def get_accumulated_cached_steps(self):
    return self.main.accumulated_cached_steps

  def get_cfg_accumulated_cached_steps(self):
    return self.cfg.accumulated_cached_steps

  def get_accumulated_executed_steps(self):
    return self.accumulated_executed_steps

  def get_accumulated_transformer_executed_steps(self):
    return self.accumulated_transformer_executed_steps
