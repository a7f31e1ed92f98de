"""Context registry and per-step decisions of DBCache.

`CachedContextManager` keeps the method names the reference's block runner and adapters call
(src/cache_dit/caching/cache_contexts/cache_manager.py:20-956: `set_context`, `mark_step_begin`,
`can_cache`, `add_cached_step`, `apply_cache`, `set_Fn_buffer`, `set_Bn_buffer`,
`set_Bn_encoder_buffer`, ...), so third-party block runners written against it keep working.
What differs is how the tensor work is done: every tensor operation is one launch of an sm_100a
kernel (see step_ops.py), and a `LazyResidual` lets the caller hand over "after - before" without
materialising it, so residual formation is fused into the kernel that consumes it.

Host-side order of the gates in `can_cache`, the special threshold values, CFG diff sharing and
the refresh rules are those of the reference; they are integer / float bookkeeping and must match
bit for bit.
"""
from __future__ import annotations

import contextlib
import copy
import logging
from typing import Dict, List, Optional, Tuple, Union

import torch

from .cache_context import CachedContext
from .calibrators import CalibratorBase
from .step_ops import get_ops, ratio_in_dtype, round_to_dtype

logger = logging.getLogger("cache_dit_b200")


class ContextNotExistError(Exception):
  pass


class LazyResidual:
  """`after - before`, formed inside whichever kernel first needs it.

  The block runner passes this instead of a tensor; `value` is filled by the first consumer
  (the relative-L1 kernel writes it as a by-product) and re-used by later ones."""

  def __init__(self, after: torch.Tensor, before: torch.Tensor):
    assert after.shape == before.shape and after.dtype == before.dtype
    self.after = after if after.is_contiguous() else after.contiguous()
    self.before = before if before.is_contiguous() else before.contiguous()
    self.value: Optional[torch.Tensor] = None

  shape = property(lambda self: self.after.shape)
  dtype = property(lambda self: self.after.dtype)
  device = property(lambda self: self.after.device)

  def materialize(self, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    if self.value is None:
      ops = get_ops()
      self.value = ops.residual(self.after, self.before, out if out is not None else ops.empty_like(self.after))
    return self.value


TensorLike = Union[torch.Tensor, LazyResidual]


def _contig(t: torch.Tensor) -> torch.Tensor:
  return t if t.is_contiguous() else t.contiguous()


class CachedContextManager:

  def __init__(self, name: str = None, persistent_context: bool = False):
    self.name = name
    self._current_context: Optional[CachedContext] = None
    self._cached_context_manager: Dict[str, CachedContext] = {}
    self._persistent_context = persistent_context
    self._current_step_refreshed = False

  # ---------------------------------------------------------------- registry / refresh
  @property
  def persistent_context(self) -> bool:
    return self._persistent_context

  @property
  def current_context(self) -> Optional[CachedContext]:
    return self._current_context

  @property
  def current_step_refreshed(self) -> bool:
    return self._current_step_refreshed

  def _ctx(self) -> CachedContext:
    assert self._current_context is not None, "cached_context must be set before"
    return self._current_context

  def new_context(self, *args, **kwargs) -> CachedContext:
    ctx = CachedContext(*args, **kwargs)
    ctx._init_args, ctx._init_kwargs = args, kwargs  # remembered for implicit refresh
    self._cached_context_manager[ctx.name] = ctx
    return ctx

  def _resolve(self, ctx_or_name) -> CachedContext:
    if isinstance(ctx_or_name, CachedContext):
      return ctx_or_name
    if ctx_or_name not in self._cached_context_manager:
      raise ContextNotExistError("Context not exist!")
    return self._cached_context_manager[ctx_or_name]

  def get_context(self, name: str = None) -> Optional[CachedContext]:
    return self._resolve(name) if name is not None else self._current_context

  def is_pre_refreshed(self) -> bool:
    """True on the last step of a run (statistics are published then for persistent contexts)."""
    ctx = self._current_context
    if ctx is None:
      return False
    n = ctx.cache_config.num_inference_steps
    return True if n is None else ctx.get_current_step() == n - 1

  def maybe_refresh(self, cached_context=None) -> Tuple[bool, str]:
    ctx = self._ctx() if cached_context is None else self._resolve(cached_context)
    n = ctx.cache_config.num_inference_steps
    # NOTE: evaluated before this call's mark_step_begin, i.e. on the previous call's index
    if n is not None and ctx.get_current_step() >= n:
      return True, "num_inference_steps"
    hint = ctx.get_force_refresh_step_hint()
    if hint is not None and ctx.get_current_transformer_step() == hint - 1:
      return True, "force_refresh_step_hint"
    return False, ""

  def set_context(self, cached_context, *args, **kwargs) -> CachedContext:
    if isinstance(cached_context, CachedContext):
      self._current_context = cached_context
    elif cached_context in self._cached_context_manager:
      self._current_context = self._cached_context_manager[cached_context]
    elif not self._persistent_context:
      raise ContextNotExistError("Context not exist and persistent_context is False. Please "
                                 "create new context first or set persistent_context=True.")
    elif args or kwargs:
      kwargs["name"] = cached_context
      self._current_context = self.new_context(*args, **kwargs)
    else:
      raise ValueError("To create new context, please provide args and kwargs.")

    should_refresh, reason = self.maybe_refresh(self._current_context)
    self._current_step_refreshed = should_refresh
    if not should_refresh:
      return self._current_context

    old = self._current_context
    if not (args or kwargs):
      args, kwargs = old._init_args, dict(old._init_kwargs)
    new = self.reset_context(old, *args, **kwargs)
    if reason == "force_refresh_step_hint":
      # the steps before and after a forced refresh belong to one inference: keep its history
      new.main.cached_steps = list(old.main.cached_steps)
      new.cfg.cached_steps = list(old.cfg.cached_steps)
      new.main.residual_diffs = dict(old.main.residual_diffs)
      new.cfg.residual_diffs = dict(old.cfg.residual_diffs)
      new.main.accumulated_cached_steps = old.main.accumulated_cached_steps
      new.cfg.accumulated_cached_steps = old.cfg.accumulated_cached_steps
      new.accumulated_executed_steps = old.accumulated_executed_steps
      new.accumulated_transformer_executed_steps = old.accumulated_transformer_executed_steps
      new.cache_config = copy.deepcopy(new.cache_config)  # the config may be shared between users
      if new.cache_config.force_refresh_step_policy == "once":
        new.cache_config.force_refresh_step_hint = None
    self._current_context = new
    return new

  def reset_context(self, cached_context, *args, **kwargs) -> CachedContext:
    name = cached_context.name if isinstance(cached_context, CachedContext) else cached_context
    self.remove_context(name)
    kwargs["name"] = name
    return self.new_context(*args, **kwargs)

  def remove_context(self, cached_context):
    name = cached_context.name if isinstance(cached_context, CachedContext) else cached_context
    if isinstance(cached_context, CachedContext):
      cached_context.clear_buffers()
    ctx = self._cached_context_manager.pop(name, None)
    if ctx is not None:
      ctx.clear_buffers()

  def clear_contexts(self):
    for name in list(self._cached_context_manager):
      self.remove_context(name)

  @contextlib.contextmanager
  def enter_context(self, cached_context):
    previous = self._current_context
    self._current_context = self._resolve(cached_context)
    try:
      yield
    finally:
      self._current_context = previous

  # ---------------------------------------------------------------- thin accessors
  def mark_step_begin(self):
    self._ctx().mark_step_begin()

  def add_cached_step(self):
    self._ctx().add_cached_step()

  def add_residual_diff(self, diff):
    self._ctx().add_residual_diff(diff)

  def get_current_step(self) -> int:
    return self._ctx().get_current_step()

  def get_current_transformer_step(self) -> int:
    return self._ctx().get_current_transformer_step()

  def get_residual_diff_threshold(self) -> float:
    return self._ctx().get_residual_diff_threshold()

  def get_force_refresh_step_hint(self):
    return self._ctx().get_force_refresh_step_hint()

  def get_buffer(self, name):
    return self._ctx().get_buffer(name)

  def set_buffer(self, name, buffer):
    self._ctx().set_buffer(name, buffer)

  def remove_buffer(self, name):
    self._ctx().remove_buffer(name)

  def get_cached_steps(self) -> List[int]:
    return self._ctx().get_cached_steps()

  def get_cfg_cached_steps(self) -> List[int]:
    return self._ctx().get_cfg_cached_steps()

  def get_residual_diffs(self) -> Dict[str, float]:
    return self._ctx().get_residual_diffs()

  def get_cfg_residual_diffs(self) -> Dict[str, float]:
    return self._ctx().get_cfg_residual_diffs()

  def get_current_step_residual_diff(self):
    return self._ctx().main.residual_diffs.get(str(self.get_current_step()))

  def get_current_step_cfg_residual_diff(self):
    return self._ctx().cfg.residual_diffs.get(str(self.get_current_step()))

  def get_max_cached_steps(self) -> int:
    return self._ctx().cache_config.max_cached_steps

  def get_max_continuous_cached_steps(self) -> int:
    return self._ctx().cache_config.max_continuous_cached_steps

  def get_continuous_cached_steps(self) -> int:
    return self._ctx().main.continuous_cached_steps

  def get_cfg_continuous_cached_steps(self) -> int:
    return self._ctx().cfg.continuous_cached_steps

  def get_accumulated_cached_steps(self) -> int:
    return self._ctx().main.accumulated_cached_steps

  def get_cfg_accumulated_cached_steps(self) -> int:
    return self._ctx().cfg.accumulated_cached_steps

  def get_accumulated_executed_steps(self) -> int:
    return self._ctx().accumulated_executed_steps

  def get_accumulated_transformer_executed_steps(self) -> int:
    return self._ctx().accumulated_transformer_executed_steps

  def get_accumulated_residual_diff(self) -> float:
    return self._ctx().main.accumulated_residual_diff

  def get_cfg_accumulated_residual_diff(self) -> float:
    return self._ctx().cfg.accumulated_residual_diff

  def max_accumulated_residual_diff_threshold(self):
    return self._ctx().cache_config.max_accumulated_residual_diff_threshold

  def is_calibrator_enabled(self) -> bool:
    return self._ctx().enable_calibrator()

  def is_encoder_calibrator_enabled(self) -> bool:
    return self._ctx().enable_encoder_calibrator()

  def get_calibrator(self):
    return self._ctx().get_calibrators()

  def get_cfg_calibrator(self):
    return self._ctx().get_cfg_calibrators()

  def is_calibrator_cache_residual(self) -> bool:
    return self._ctx().calibrator_cache_type() == "residual"

  def is_cache_residual(self) -> bool:
    return self.is_calibrator_cache_residual() if self.is_calibrator_enabled() else True

  def is_encoder_cache_residual(self) -> bool:
    return self.is_calibrator_cache_residual() if self.is_encoder_calibrator_enabled() else True

  def is_in_warmup(self) -> bool:
    return self._ctx().is_in_warmup()

  def is_in_full_compute_steps(self) -> bool:
    return self._ctx().is_in_full_compute_steps()

  def is_steps_computation_mask_enabled(self) -> bool:
    return self._ctx().cache_config.steps_computation_mask is not None

  def get_steps_computation_policy(self) -> str:
    return self._ctx().get_steps_computation_policy()

  def is_l1_diff_enabled(self) -> bool:
    t = self._ctx().extra_cache_config.l1_hidden_states_diff_threshold
    return t is not None and t > 0.0

  def get_important_condition_threshold(self) -> float:
    return self._ctx().extra_cache_config.important_condition_threshold

  def get_downsample_factor(self) -> int:
    return self._ctx().extra_cache_config.downsample_factor

  def Fn_compute_blocks(self) -> int:
    n = self._ctx().cache_config.Fn_compute_blocks
    assert n >= 1, "Fn_compute_blocks must be >= 1"
    return n

  def Bn_compute_blocks(self) -> int:
    n = self._ctx().cache_config.Bn_compute_blocks
    assert n >= 0, "Bn_compute_blocks must be >= 0"
    return n

  def enable_separate_cfg(self) -> bool:
    return self._ctx().cache_config.enable_separate_cfg

  def is_separate_cfg_step(self) -> bool:
    return self._ctx().is_separate_cfg_step()

  def cfg_diff_compute_separate(self) -> bool:
    return self._ctx().cache_config.cfg_diff_compute_separate

  # ---------------------------------------------------------------- buffers
  def _key(self, prefix: str, encoder: bool = False) -> str:
    key = f"{prefix}_encoder_buffer" if encoder else f"{prefix}_buffer"
    return key + "_cfg" if self.is_separate_cfg_step() else key

  def _downsample(self, t: torch.Tensor) -> torch.Tensor:
    k = self.get_downsample_factor()
    return t[..., ::k].contiguous() if k > 1 else t

  def set_Fn_buffer(self, buffer: Optional[TensorLike], prefix: str = "Fn"):
    """Store the indicator of the last computed step. A `LazyResidual` is stored as the tensor the
    check kernel already wrote (or is formed now); the buffer it replaces is recycled."""
    if buffer is None:
      return
    ctx = self._ctx()
    key = self._key(prefix)
    if isinstance(buffer, LazyResidual):
      spare_key = key + "/spare"
      value = buffer.materialize(self._take_spare(spare_key, buffer))
      value = self._downsample(value)
      old = ctx.buffers.get(key)
      if old is not None and key in ctx.buffers.get("/owned", ()) and old is not value:
        ctx.buffers[spare_key] = old
      ctx.buffers.setdefault("/owned", set()).add(key)
      ctx.buffers[key] = value
    else:
      ctx.buffers.get("/owned", set()).discard(key)
      ctx.buffers[key] = self._downsample(buffer)

  def _take_spare(self, spare_key: str, like) -> Optional[torch.Tensor]:
    spare = self._ctx().buffers.pop(spare_key, None)
    if spare is not None and (spare.shape != like.shape or spare.dtype != like.dtype
                              or spare.device != like.device):
      spare = None
    return spare

  def get_Fn_buffer(self, prefix: str = "Fn"):
    return self.get_buffer(self._key(prefix))

  def set_Fn_encoder_buffer(self, buffer, prefix: str = "Fn"):
    if buffer is not None:
      self.set_buffer(self._key(prefix, encoder=True), _as_tensor(buffer))

  def get_Fn_encoder_buffer(self, prefix: str = "Fn"):
    return self.get_buffer(self._key(prefix, encoder=True))

  def _calibrator_for(self, encoder: bool) -> Optional[CalibratorBase]:
    ctx = self._ctx()
    if not (ctx.enable_encoder_calibrator() if encoder else ctx.enable_calibrator()):
      return None
    branch = ctx.branch()
    return branch.encoder_calibrator if encoder else branch.calibrator

  def _set_Bn(self, buffer: Optional[TensorLike], prefix: str, encoder: bool):
    if buffer is None:
      return
    cal = self._calibrator_for(encoder)
    if cal is not None:
      if isinstance(buffer, LazyResidual) and buffer.value is None and hasattr(cal, "update_residual"):
        cal.update_residual(buffer.after, buffer.before, name=prefix)  # residual fused into the ladder
      else:
        cal.update(_as_tensor(buffer), name=prefix)
    else:
      self.set_buffer(self._key(prefix, encoder), _as_tensor(buffer))

  def _get_Bn(self, prefix: str, encoder: bool):
    cal = self._calibrator_for(encoder)
    if cal is not None:
      return cal.approximate(name=prefix)
    return self.get_buffer(self._key(prefix, encoder))

  def set_Bn_buffer(self, buffer, prefix: str = "Bn"):
    self._set_Bn(buffer, prefix, encoder=False)

  def get_Bn_buffer(self, prefix: str = "Bn"):
    return self._get_Bn(prefix, encoder=False)

  def set_Bn_encoder_buffer(self, buffer, prefix: str = "Bn"):
    self._set_Bn(buffer, prefix, encoder=True)

  def get_Bn_encoder_buffer(self, prefix: str = "Bn"):
    return self._get_Bn(prefix, encoder=True)

  # ---------------------------------------------------------------- the decision
  def similarity(self, t1: torch.Tensor, t2: TensorLike, *, threshold: float, parallelized: bool = False,
                 prefix: str = "Fn") -> bool:
    """diff = mean|t1 - t2| / mean|t1| < threshold, with t1 the stored and t2 the current tensor."""
    if threshold <= 0.0:
      self.add_residual_diff(-0.0)  # disabled
      return False
    if threshold >= 1.0:
      self.add_residual_diff(-1.0)  # always similar
      return True
    if t1.shape != t2.shape:
      self.add_residual_diff(-2.0)  # shape changed
      return False
    shared = None
    if (self.enable_separate_cfg() and self.is_separate_cfg_step() and not self.cfg_diff_compute_separate()):
      shared = self.get_current_step_residual_diff()
    if shared is not None:
      diff = shared  # the CFG call re-uses the diff of the non-CFG call of the same step
    elif self.get_important_condition_threshold() > 0.0:
      diff = self._important_token_diff(t1, _as_tensor(t2), parallelized)
    else:
      ops = get_ops()
      if isinstance(t2, LazyResidual) and t2.value is None:
        spare_key = self._key(prefix) + "/spare"
        out = self._take_spare(spare_key, t2) if self.get_downsample_factor() <= 1 else None
        out = out if out is not None else ops.empty_like(t2.after)
        md, mp, world = ops.rel_l1_means(t2.after, t2.before, t1, out, group=True if parallelized else None)
        t2.value = out
      else:
        md, mp, world = ops.rel_l1_means(_contig(_as_tensor(t2)), None, _contig(t1), None,
                                         group=True if parallelized else None)
      if world > 1:  # ReduceOp.AVG of the local means, in the tensor dtype
        md = round_to_dtype(md / world, t1.dtype)
        mp = round_to_dtype(mp / world, t1.dtype)
      diff = ratio_in_dtype(md, mp, t1.dtype)
    self.add_residual_diff(diff)
    return diff < threshold

  def _important_token_diff(self, t1, t2, parallelized) -> float:
    """Rarely used token-selective variant (extra config); plain tensor ops, not a hot path."""
    raw = (t1 - t2).abs()
    token_diff = raw.mean(dim=-1) / t1.abs().mean(dim=-1)
    cond = token_diff > self.get_important_condition_threshold()
    if cond.sum() > 0:
      cond = cond.unsqueeze(-1).expand_as(raw)
      mean_diff, mean_t1 = raw[cond].mean(), t1[cond].abs().mean()
    else:
      mean_diff, mean_t1 = raw.mean(), t1.abs().mean()
    if parallelized:
      import torch.distributed as dist
      dist.all_reduce(mean_diff, op=dist.ReduceOp.AVG)
      dist.all_reduce(mean_t1, op=dist.ReduceOp.AVG)
    return (mean_diff / mean_t1).item()

  def can_cache(self, states_tensor: TensorLike, parallelized: bool = False,
                threshold: Optional[float] = None, prefix: str = "Fn") -> bool:
    ctx = self._ctx()
    cc = ctx.cache_config
    if ctx.is_in_warmup():
      return False
    if cc.steps_computation_mask is not None:
      if ctx.is_in_full_compute_steps():
        return False
      if cc.steps_computation_policy == "static":
        return True
    branch = ctx.branch()
    if cc.max_cached_steps >= 0 and len(branch.cached_steps) >= cc.max_cached_steps:
      return False
    if cc.max_continuous_cached_steps >= 0 and branch.continuous_cached_steps >= cc.max_continuous_cached_steps:
      branch.continuous_cached_steps = 0  # a forced compute step ends the run of cached steps
      return False
    cap = cc.max_accumulated_residual_diff_threshold
    if cap is not None and cap > 0.0 and branch.accumulated_residual_diff >= cap:
      return False
    if threshold is None or threshold <= 0.0:
      threshold = ctx.get_residual_diff_threshold()
    if threshold <= 0.0:
      return False
    k = self.get_downsample_factor()
    if k > 1 and "Bn" not in prefix:
      states_tensor = _as_tensor(states_tensor)[..., ::k].contiguous()
    prev = self.get_Bn_buffer(prefix) if "Bn" in prefix else self.get_Fn_buffer(prefix)
    return prev is not None and self.similarity(prev, states_tensor, threshold=threshold,
                                                parallelized=parallelized, prefix=prefix)

  # ---------------------------------------------------------------- hit path
  def _apply_one(self, hidden: torch.Tensor, prefix: str, encoder: bool, residual: bool):
    hidden = _contig(hidden)
    source_is_Bn = "Bn" in prefix
    cal = self._calibrator_for(encoder) if source_is_Bn else None
    if cal is not None and hasattr(cal, "approximate_add"):
      if prefix not in getattr(cal, "states", {prefix: None}):
        raise AssertionError(f"State '{prefix}' not found.")
      return cal.approximate_add(hidden, name=prefix, add_hidden=residual)
    if source_is_Bn:
      prev = self._get_Bn(prefix, encoder)
    else:
      prev = self.get_Fn_encoder_buffer(prefix) if encoder else self.get_Fn_buffer(prefix)
    if prev is None:
      return None
    if not residual:
      return _contig(prev)
    ops = get_ops()
    return ops.taylor_apply(hidden, [_contig(prev)], 1, True, ops.empty_like(hidden))

  def apply_cache(self, hidden_states: torch.Tensor, encoder_hidden_states: torch.Tensor = None,
                  prefix: str = "Bn", encoder_prefix: str = "Bn_encoder"):
    """hidden <- forecast (+ hidden): Taylor series and the add in a single pass per stream."""
    out = self._apply_one(hidden_states, prefix, False, self.is_cache_residual())
    assert out is not None, f"{prefix}_buffer must be set before"
    enc_out = encoder_hidden_states
    if encoder_hidden_states is not None:
      e = self._apply_one(encoder_hidden_states, encoder_prefix, True, self.is_encoder_cache_residual())
      enc_out = _contig(encoder_hidden_states) if e is None else e
    return out, enc_out


def _as_tensor(t: TensorLike) -> torch.Tensor:
  return t.materialize() if isinstance(t, LazyResidual) else t
