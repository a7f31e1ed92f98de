"""Scenario backends that need nothing but the numpy oracle (see tests/scenarios.py)."""
from __future__ import annotations

import numpy as np

from oracle import cache_oracle as O

PREFIX = "blocks"


def stats_dict(cached_steps, residual_diffs, cfg_cached_steps, cfg_residual_diffs,
               accumulated_cached_steps, cfg_accumulated_cached_steps,
               accumulated_executed_steps, accumulated_transformer_executed_steps) -> dict:
  """The statistics the reference attaches to modules (cache_blocks/pattern_utils.py:23-31)."""
  return dict(
    cached_steps=[int(s) for s in cached_steps],
    residual_diffs={str(k): float(v) for k, v in residual_diffs.items()},
    cfg_cached_steps=[int(s) for s in cfg_cached_steps],
    cfg_residual_diffs={str(k): float(v) for k, v in cfg_residual_diffs.items()},
    accumulated_cached_steps=int(accumulated_cached_steps),
    cfg_accumulated_cached_steps=int(cfg_accumulated_cached_steps),
    accumulated_executed_steps=int(accumulated_executed_steps),
    accumulated_transformer_executed_steps=int(accumulated_transformer_executed_steps),
  )


class OracleBackend:

  def __init__(self, sc: dict, shards=None):
    self.ctx = O.OracleContext(sc["cache_config"], sc["calibrator_config"], sc["dtype"], shards,
                               sc.get("extra_config"))

  def _p(self, encoder=False):
    kind = "residual" if self.ctx.is_cache_residual(encoder) else "hidden_states"
    return f"{PREFIX}_Bn_{kind}"

  def begin_call(self):
    self.ctx.set_context()

  def mark_step_begin(self):
    self.ctx.mark_step_begin()

  def current_step(self):
    return self.ctx.current_step()

  def can_cache(self, r):
    return self.ctx.can_cache(r, prefix=f"{PREFIX}_Fn_residual")

  def add_cached_step(self):
    self.ctx.add_cached_step()

  def apply_cache(self, h, e):
    return self.ctx.apply_cache(h, e, self._p(), self._p(True))

  def set_Fn_buffer(self, r):
    self.ctx.set_Fn_buffer(r, f"{PREFIX}_Fn_residual")

  def set_Bn_buffer(self, R):
    self.ctx.set_Bn_buffer(R, self._p())

  def set_Bn_encoder_buffer(self, Re):
    self.ctx.set_Bn_buffer(Re, self._p(True), encoder=True)

  def stats(self):
    c = self.ctx
    return stats_dict(c.cached_steps, c.residual_diffs, c.cfg_cached_steps, c.cfg_residual_diffs,
                      c.accumulated_cached_steps, c.cfg_accumulated_cached_steps,
                      c.accumulated_executed_steps, c.accumulated_transformer_executed_steps)

  @staticmethod
  def from_torch(t):
    return t.float().numpy()

  @staticmethod
  def to_numpy(a):
    return np.asarray(a, dtype=np.float32)


class ProductBackend:
  """tests/scenarios.py backend over cache_dit_b200's own CachedContextManager (any device)."""

  def __init__(self, sc: dict, device="cpu", parallelized: bool = False):
    import cache_dit_b200 as cd
    cc = dict(sc["cache_config"])
    cc.setdefault("enable_separate_cfg", False)
    cal = sc["calibrator_config"]
    self.device = device
    self.parallelized = parallelized
    self.mgr = cd.CachedContextManager("scenario", persistent_context=True)
    extra = {"extra_cache_config": cd.ExtraCacheConfig(**sc["extra_config"])} if sc.get("extra_config") else {}
    self.mgr.new_context(name="ctx", cache_config=cd.DBCacheConfig(**cc),
                         calibrator_config=None if cal is None else cd.TaylorSeerCalibratorConfig(**cal), **extra)

  def _p(self, encoder=False):
    res = self.mgr.is_encoder_cache_residual() if encoder else self.mgr.is_cache_residual()
    return f"{PREFIX}_Bn_{'residual' if res else 'hidden_states'}"

  def begin_call(self):
    self.mgr.set_context("ctx")

  def mark_step_begin(self):
    self.mgr.mark_step_begin()

  def current_step(self):
    return self.mgr.get_current_step()

  def can_cache(self, r):
    return self.mgr.can_cache(r, parallelized=self.parallelized, prefix=f"{PREFIX}_Fn_residual")

  def add_cached_step(self):
    self.mgr.add_cached_step()

  def apply_cache(self, h, e):
    return self.mgr.apply_cache(h, e, prefix=self._p(), encoder_prefix=self._p(True))

  def set_Fn_buffer(self, r):
    self.mgr.set_Fn_buffer(r, prefix=f"{PREFIX}_Fn_residual")

  def set_Bn_buffer(self, R):
    self.mgr.set_Bn_buffer(R, prefix=self._p())

  def set_Bn_encoder_buffer(self, Re):
    self.mgr.set_Bn_encoder_buffer(Re, prefix=self._p(True))

  def stats(self):
    m = self.mgr
    return stats_dict(m.get_cached_steps(), m.get_residual_diffs(), m.get_cfg_cached_steps(),
                      m.get_cfg_residual_diffs(), m.get_accumulated_cached_steps(),
                      m.get_cfg_accumulated_cached_steps(), m.get_accumulated_executed_steps(),
                      m.get_accumulated_transformer_executed_steps())

  def from_torch(self, t):
    return t.to(self.device)

  @staticmethod
  def to_numpy(t):
    return t.detach().float().cpu().numpy()
