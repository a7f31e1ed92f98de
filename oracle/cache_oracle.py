"""CPU restatement of cache-dit's DBCache + TaylorSeer step logic (numpy only).

TEST INFRASTRUCTURE, NOT PRODUCT CODE.  Only the test-suite, the smoke check and
the CPU-baseline leg of the benchmark may import this file; the shipped package
never does.  It restates, in independent numpy code, what the reference computes
for one denoising step so that the CUDA path can be checked value-for-value.

Pinning: every function below was checked against the live reference imported on
CPU (the script next to the golden fixtures drives the reference's own
`CachedContextManager` / `enable_cache` and stores masks, counters, diffs and
small output tensors); the fixtures are re-checked against this file by the
CPU-only tests.

Reference map (paths inside the reference project):
  * relative-L1 similarity ........ src/cache_dit/caching/cache_contexts/cache_manager.py:552-626
  * gate order in can_cache ....... src/cache_dit/caching/cache_contexts/cache_manager.py:862-956
  * counters / CFG parity ......... src/cache_dit/caching/cache_contexts/cache_context.py:146-317
  * cached-residual apply ......... src/cache_dit/caching/cache_contexts/cache_manager.py:814-854
  * Taylor derivative / series .... src/cache_dit/caching/cache_contexts/calibrators/taylorseer.py:68-127
  * block runner (Fn/Mn/Bn) ....... src/cache_dit/caching/cache_blocks/pattern_base.py:198-321
  * persistent-context refresh .... src/cache_dit/caching/cache_contexts/cache_manager.py:79-199

Arithmetic model.  Tensors are float32 numpy arrays whose values are always
representable in the *storage dtype* ("fp32", "bf16" or "fp16").  Every
elementwise torch op in the reference produces a tensor in the storage dtype, so
each op here is computed in float32 and then rounded to the storage dtype with
round-to-nearest-even (`rnd`).  Reductions accumulate wider and round once, as
torch does for low-precision means.
"""
from __future__ import annotations

import copy
import math
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import numpy as np

# --------------------------------------------------------------------------- #
# dtype emulation
# --------------------------------------------------------------------------- #


def round_bf16(x: np.ndarray) -> np.ndarray:
  """Round float32 values to the nearest bfloat16 (ties to even), keep float32 storage."""
  a = np.ascontiguousarray(x, dtype=np.float32)
  u = a.view(np.uint32)
  # NaN stays NaN: adding the rounding bias could carry into the exponent.
  nan = np.isnan(a)
  bias = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
  r = ((u + bias) & np.uint32(0xFFFF0000)).view(np.float32)
  if nan.any():
    r = np.where(nan, np.float32(np.nan), r)
  return r.reshape(a.shape)


def rnd(x, dtype: str) -> np.ndarray:
  """Round to the storage dtype; the result is float32 holding representable values."""
  if dtype == "fp32":
    return np.asarray(x, dtype=np.float32)
  if dtype == "bf16":
    return round_bf16(np.asarray(x, dtype=np.float32))
  if dtype == "fp16":
    with np.errstate(over="ignore"):
      return np.asarray(x, dtype=np.float32).astype(np.float16).astype(np.float32)
  raise ValueError(f"unknown storage dtype {dtype!r}")


def _scalar(x, dtype: str) -> np.float32:
  return np.float32(rnd(np.asarray([x], dtype=np.float32), dtype)[0])


# --------------------------------------------------------------------------- #
# the four tensor operations of the step
# --------------------------------------------------------------------------- #


def residual(after: np.ndarray, before: np.ndarray, dtype: str) -> np.ndarray:
  """`after - before` as one elementwise op in the storage dtype.

  Fn residual: pattern_base.py:195.  Mn residual: pattern_base.py:414,418.
  """
  return rnd(np.float32(after) - np.float32(before), dtype)


def local_means(prev: np.ndarray, cur: np.ndarray, dtype: str) -> Tuple[np.float32, np.float32]:
  """The two 0-dim tensors of cache_manager.py:609-610, each rounded to the storage dtype.

  mean(|prev - cur|) where the subtraction is itself rounded elementwise, and mean(|prev|).
  Sums are taken in float64 (torch accumulates low-precision means in float32 with a
  cascade; both agree far inside the bf16 rounding step and to ~1e-7 in fp32).
  """
  d = np.abs(rnd(np.float32(prev) - np.float32(cur), dtype))
  n = d.size
  mean_diff = np.float32(np.sum(d, dtype=np.float64) / n)
  mean_prev = np.float32(np.sum(np.abs(prev), dtype=np.float64) / n)
  return _scalar(mean_diff, dtype), _scalar(mean_prev, dtype)


def combine_means(pairs: Sequence[Tuple[float, float]], dtype: str) -> Tuple[np.float32, np.float32]:
  """Cross-rank average of the local means (ReduceOp.AVG, cache_manager.py:612-614)."""
  w = len(pairs)
  md = np.float32(sum(np.float64(p[0]) for p in pairs) / w)
  mp = np.float32(sum(np.float64(p[1]) for p in pairs) / w)
  return _scalar(md, dtype), _scalar(mp, dtype)


def rel_l1(prev: np.ndarray, cur: np.ndarray, dtype: str,
           shards: Optional[int] = None) -> float:
  """`(mean_diff / mean_t1).item()` of cache_manager.py:619.

  With `shards=W` the token axis (axis 1) is split like torch.tensor_split and the
  per-shard means are averaged first, as W context-parallel ranks would do.
  """
  if shards is None or shards <= 1:
    md, mp = local_means(prev, cur, dtype)
  else:
    ps = np.array_split(prev, shards, axis=1)
    cs = np.array_split(cur, shards, axis=1)
    md, mp = combine_means([local_means(p, c, dtype) for p, c in zip(ps, cs)], dtype)
  with np.errstate(divide="ignore", invalid="ignore"):
    q = np.float32(md) / np.float32(mp)
  return float(_scalar(q, dtype))


def rel_l1_important_tokens(prev: np.ndarray, cur: np.ndarray, condition: float, dtype: str) -> float:
  """The token-selective distance of cache_manager.py:588-606 (`important_condition_threshold > 0`).

  Per token, mean|prev - cur| / mean|prev| over the channels; when any token exceeds `condition` the two
  means of the relative L1 distance are taken over those tokens only, else over everything.
  """
  raw = np.abs(rnd(np.float32(prev) - np.float32(cur), dtype))
  c = raw.shape[-1]
  token_df = rnd(np.float32(np.sum(raw, axis=-1, dtype=np.float64) / c), dtype)
  token_t1 = rnd(np.float32(np.sum(np.abs(prev), axis=-1, dtype=np.float64) / c), dtype)
  with np.errstate(divide="ignore", invalid="ignore"):
    token_diff = rnd(np.float32(token_df) / np.float32(token_t1), dtype)
  chosen = token_diff > np.float32(condition)
  if chosen.sum() > 0:
    d, p = raw[chosen], np.abs(prev)[chosen]
  else:
    d, p = raw, np.abs(prev)
  md = _scalar(np.float32(np.sum(d, dtype=np.float64) / d.size), dtype)
  mp = _scalar(np.float32(np.sum(p, dtype=np.float64) / p.size), dtype)
  with np.errstate(divide="ignore", invalid="ignore"):
    q = np.float32(md) / np.float32(mp)
  return float(_scalar(q, dtype))


def taylor_series(derivs: Sequence[Optional[np.ndarray]], elapsed: int, dtype: str):
  """TaylorSeerState.approximate, taylorseer.py:91-104, with its per-op rounding.

  `output = 0; output += (1/i!) * dY[i] * elapsed**i` — three rounded elementwise
  ops per term (scale by 1/i!, scale by elapsed**i, accumulate).
  """
  out = None
  for i, d in enumerate(derivs):
    if d is None:
      break
    term = rnd(np.float32(1.0 / math.factorial(i)) * np.float32(d), dtype)
    term = rnd(term * np.float32(elapsed**i), dtype)
    out = term if out is None else rnd(out + term, dtype)
  return 0 if out is None else out


def taylor_derivatives(y: np.ndarray, prev: Sequence[Optional[np.ndarray]], window: int,
                       step_gt_1: bool, dtype: str) -> List[Optional[np.ndarray]]:
  """TaylorSeerState.derivative, taylorseer.py:68-89: finite-difference ladder.

  dY[0] = Y; dY[i+1] = (dY[i] - dY_prev[i]) / window — a rounded subtraction then a
  rounded division — while the previous entry exists and the state's step is > 1.
  """
  order = len(prev)
  cur: List[Optional[np.ndarray]] = [None] * order
  cur[0] = y
  for i in range(order - 1):
    if prev[i] is not None and step_gt_1:
      diff = rnd(np.float32(cur[i]) - np.float32(prev[i]), dtype)
      cur[i + 1] = rnd(diff / np.float32(window), dtype)
    else:
      break
  return cur


def apply_add(approx: np.ndarray, hidden: np.ndarray, dtype: str) -> np.ndarray:
  """`hidden_states_prev + hidden_states`, cache_manager.py:831."""
  return rnd(np.float32(approx) + np.float32(hidden), dtype)


# --------------------------------------------------------------------------- #
# TaylorSeer bookkeeping
# --------------------------------------------------------------------------- #


class TaylorState:
  """One named stream of a TaylorSeer calibrator (taylorseer.py:14-127)."""

  def __init__(self, n_derivatives: int, dtype: str):
    self.n = n_derivatives
    self.order = n_derivatives + 1
    self.dtype = dtype
    self.reset()

  def reset(self):
    self.prev: List[Optional[np.ndarray]] = [None] * self.order
    self.cur: List[Optional[np.ndarray]] = [None] * self.order
    self.current_step = -1
    self.last_step = -1

  def update(self, y: np.ndarray):
    self.prev = self.cur
    window = self.current_step - self.last_step
    if self.prev[0] is not None and self.prev[0].shape != y.shape:
      # shape change drops everything, including the step counters (taylorseer.py:80-82)
      self.reset()
    self.cur = taylor_derivatives(y, self.prev, window, self.current_step > 1, self.dtype)
    self.last_step = self.current_step

  def approximate(self):
    return taylor_series(self.cur, self.current_step - self.last_step, self.dtype)


class TaylorCalibrator:
  """Name-keyed states; a state is created by its first update (taylorseer.py:144-265)."""

  def __init__(self, n_derivatives: int, dtype: str):
    self.n = n_derivatives
    self.dtype = dtype
    self.states: Dict[str, TaylorState] = {}

  def reset_cache(self):
    for s in self.states.values():
      s.reset()

  def mark_step_begin(self):
    for s in self.states.values():
      s.current_step += 1

  def update(self, y, name):
    if name not in self.states:
      self.states[name] = TaylorState(self.n, self.dtype)
    self.states[name].update(y)

  def approximate(self, name):
    return self.states[name].approximate()


# --------------------------------------------------------------------------- #
# per-context state machine
# --------------------------------------------------------------------------- #

DEFAULT_CACHE_CONFIG = dict(
  Fn_compute_blocks=8,
  Bn_compute_blocks=0,
  residual_diff_threshold=0.08,
  max_accumulated_residual_diff_threshold=None,
  max_warmup_steps=8,
  warmup_interval=1,
  max_cached_steps=-1,
  max_continuous_cached_steps=-1,
  enable_separate_cfg=False,
  cfg_compute_first=False,
  cfg_diff_compute_separate=True,
  num_inference_steps=None,
  steps_computation_mask=None,
  steps_computation_policy="dynamic",
  force_refresh_step_hint=None,
  force_refresh_step_policy="once",
)

DEFAULT_CALIBRATOR_CONFIG = dict(
  enable_calibrator=True,
  enable_encoder_calibrator=True,
  calibrator_cache_type="residual",
  taylorseer_order=1,
)


class OracleContext:
  """Restates CachedContext + the CachedContextManager methods the block runner calls."""

  def __init__(self, cache_config: Optional[dict] = None, calibrator_config: Optional[dict] = None,
               dtype: str = "fp32", shards: Optional[int] = None, extra_config: Optional[dict] = None):
    self._init = (copy.deepcopy(cache_config), copy.deepcopy(calibrator_config), dtype, shards)
    self.cfg = dict(DEFAULT_CACHE_CONFIG)
    self.cfg.update(cache_config or {})
    # ExtraCacheConfig (cache_config.py:188-211): off by default
    self.extra = dict(downsample_factor=1, important_condition_threshold=0.0)
    self.extra.update(extra_config or {})
    self.cal = None
    if calibrator_config is not None:
      self.cal = dict(DEFAULT_CALIBRATOR_CONFIG)
      self.cal.update(calibrator_config)
    self.dtype = dtype
    self.shards = shards
    self._fresh()
    self.accumulated_cached_steps = 0
    self.cfg_accumulated_cached_steps = 0
    self.accumulated_executed_steps = 0
    self.accumulated_transformer_executed_steps = 0
    self.refreshed = False

  # -- construction / refresh ------------------------------------------------
  def _fresh(self):
    self.buffers: Dict[str, np.ndarray] = {}
    self.executed_steps = 0
    self.transformer_executed_steps = 0
    self.cached_steps: List[int] = []
    self.cfg_cached_steps: List[int] = []
    self.residual_diffs: Dict[str, float] = {}
    self.cfg_residual_diffs: Dict[str, float] = {}
    self.accumulated_residual_diff = 0.0
    self.cfg_accumulated_residual_diff = 0.0
    self.continuous_cached_steps = 0
    self.cfg_continuous_cached_steps = 0
    n = self.cal["taylorseer_order"] if self.cal else 0
    sep = bool(self.cfg["enable_separate_cfg"])
    mk = lambda on: TaylorCalibrator(n, self.dtype) if on else None
    self.calibrator = mk(bool(self.cal and self.cal["enable_calibrator"]))
    self.encoder_calibrator = mk(bool(self.cal and self.cal["enable_encoder_calibrator"]))
    self.cfg_calibrator = mk(bool(self.cal and self.cal["enable_calibrator"] and sep))
    self.cfg_encoder_calibrator = mk(bool(self.cal and self.cal["enable_encoder_calibrator"] and sep))

  def set_context(self):
    """The refresh test run at the top of every forward (cache_manager.py:100-122,156-197).

    It looks at the step index of the *previous* call, so with num_inference_steps = N a
    persistent context is rebuilt before call N+1, not before call N.
    """
    self.refreshed = False
    n = self.cfg["num_inference_steps"]
    reason = None
    if n is not None and self.current_step() >= n:
      reason = "num_inference_steps"
    else:
      hint = self.cfg["force_refresh_step_hint"]
      if hint is not None and self.current_transformer_step() == hint - 1:
        reason = "force_refresh_step_hint"
    if reason is None:
      return
    keep = None
    if reason == "force_refresh_step_hint":
      keep = (list(self.cached_steps), list(self.cfg_cached_steps), dict(self.residual_diffs),
              dict(self.cfg_residual_diffs), self.accumulated_cached_steps,
              self.cfg_accumulated_cached_steps, self.accumulated_executed_steps,
              self.accumulated_transformer_executed_steps)
    cache_config, calibrator_config, dtype, shards = self._init
    self.__init__(cache_config, calibrator_config, dtype, shards, dict(self.extra))
    if keep is not None:
      (self.cached_steps, self.cfg_cached_steps, self.residual_diffs, self.cfg_residual_diffs,
       self.accumulated_cached_steps, self.cfg_accumulated_cached_steps,
       self.accumulated_executed_steps, self.accumulated_transformer_executed_steps) = keep
      if self.cfg["force_refresh_step_policy"] == "once":
        self.cfg["force_refresh_step_hint"] = None
    self.refreshed = True

  # -- counters --------------------------------------------------------------
  def current_step(self) -> int:
    return self.executed_steps - 1

  def current_transformer_step(self) -> int:
    return self.transformer_executed_steps - 1

  def is_cfg_step(self) -> bool:
    if not self.cfg["enable_separate_cfg"]:
      return False
    odd = self.current_transformer_step() % 2 != 0
    return (not odd) if self.cfg["cfg_compute_first"] else odd

  def _calibrators(self):
    return [c for c in (self.calibrator, self.encoder_calibrator) if c is not None]

  def _cfg_calibrators(self):
    return [c for c in (self.cfg_calibrator, self.cfg_encoder_calibrator) if c is not None]

  def mark_step_begin(self):
    """cache_context.py:146-212."""
    self.transformer_executed_steps += 1
    self.accumulated_transformer_executed_steps += 1
    if not self.cfg["enable_separate_cfg"]:
      bump = True
    elif not self.cfg["cfg_compute_first"]:
      bump = not self.is_cfg_step()
    else:
      bump = self.is_cfg_step()
    if bump:
      self.executed_steps += 1
      self.accumulated_executed_steps += 1
    if self.current_transformer_step() == 0:
      self.cached_steps.clear()
      self.residual_diffs.clear()
      self.cfg_cached_steps.clear()
      self.cfg_residual_diffs.clear()
      for c in self._calibrators() + self._cfg_calibrators():
        c.reset_cache()
    if self.cfg["enable_separate_cfg"]:
      group = self._cfg_calibrators() if self.is_cfg_step() else self._calibrators()
    else:
      group = self._calibrators()
    for c in group:
      c.mark_step_begin()

  def warmup_steps(self) -> List[int]:
    hi = self.cfg["max_warmup_steps"]
    mask = self.cfg["steps_computation_mask"]
    if mask is not None:
      lead = 0
      for m in mask:
        if m == 1:
          lead += 1
        else:
          break
      hi = min(hi, lead)
    return list(range(0, hi, self.cfg["warmup_interval"]))

  def add_residual_diff(self, diff: float):
    step = str(self.current_step())
    if not self.is_cfg_step():
      if step not in self.residual_diffs:
        self.residual_diffs[step] = diff
        if diff > 0.0:
          self.accumulated_residual_diff += diff
    else:
      if step not in self.cfg_residual_diffs:
        self.cfg_residual_diffs[step] = diff
        if diff > 0.0:
          self.cfg_accumulated_residual_diff += diff

  def add_cached_step(self):
    """cache_context.py:249-276 — note the first consecutive pair counts as two."""
    cur = self.current_step()
    if not self.is_cfg_step():
      if self.cached_steps:
        if cur - self.cached_steps[-1] == 1:
          self.continuous_cached_steps += 2 if self.continuous_cached_steps == 0 else 1
      else:
        self.continuous_cached_steps += 1
      self.cached_steps.append(cur)
      self.accumulated_cached_steps += 1
    else:
      if self.cfg_cached_steps:
        if cur - self.cfg_cached_steps[-1] == 1:
          self.cfg_continuous_cached_steps += 2 if self.cfg_continuous_cached_steps == 0 else 1
      else:
        self.cfg_continuous_cached_steps += 1
      self.cfg_cached_steps.append(cur)
      self.cfg_accumulated_cached_steps += 1

  # -- buffers ---------------------------------------------------------------
  def _key(self, prefix: str, encoder: bool = False) -> str:
    k = f"{prefix}_encoder_buffer" if encoder else f"{prefix}_buffer"
    return k + "_cfg" if self.is_cfg_step() else k

  def set_Fn_buffer(self, buf, prefix):
    """cache_manager.py:641-657: with a down-sampling factor k only every k-th channel is kept."""
    if buf is not None:
      k = self.extra["downsample_factor"]
      self.buffers[self._key(prefix)] = np.ascontiguousarray(buf[..., ::k]) if k > 1 else buf

  def get_Fn_buffer(self, prefix):
    return self.buffers.get(self._key(prefix))

  def _pick(self, encoder: bool):
    if self.is_cfg_step():
      return self.cfg_encoder_calibrator if encoder else self.cfg_calibrator
    return self.encoder_calibrator if encoder else self.calibrator

  def _calibrated(self, encoder: bool) -> bool:
    if self.cal is None:
      return False
    return bool(self.cal["enable_encoder_calibrator"] if encoder else self.cal["enable_calibrator"])

  def set_Bn_buffer(self, buf, prefix, encoder: bool = False):
    if buf is None:
      return
    c = self._pick(encoder) if self._calibrated(encoder) else None
    if c is not None:
      c.update(buf, prefix)
    else:
      self.buffers[self._key(prefix, encoder)] = buf

  def get_Bn_buffer(self, prefix, encoder: bool = False):
    c = self._pick(encoder) if self._calibrated(encoder) else None
    if c is not None:
      return c.approximate(prefix)
    return self.buffers.get(self._key(prefix, encoder))

  def is_cache_residual(self, encoder: bool = False) -> bool:
    if self._calibrated(encoder):
      return self.cal["calibrator_cache_type"] == "residual"
    return True

  # -- decision --------------------------------------------------------------
  def similarity(self, prev, cur, threshold: float) -> bool:
    if threshold <= 0.0:
      self.add_residual_diff(-0.0)
      return False
    if threshold >= 1.0:
      self.add_residual_diff(-1.0)
      return True
    if prev.shape != cur.shape:
      self.add_residual_diff(-2.0)
      return False
    step = str(self.current_step())
    if (self.cfg["enable_separate_cfg"] and self.is_cfg_step()
        and not self.cfg["cfg_diff_compute_separate"] and step in self.residual_diffs):
      diff = self.residual_diffs[step]
    elif self.extra["important_condition_threshold"] > 0.0:
      diff = rel_l1_important_tokens(prev, cur, self.extra["important_condition_threshold"], self.dtype)
    else:
      diff = rel_l1(prev, cur, self.dtype, self.shards)
    self.add_residual_diff(diff)
    return diff < threshold

  def can_cache(self, states, prefix: str, threshold: Optional[float] = None) -> bool:
    if self.current_step() in self.warmup_steps():
      return False
    mask = self.cfg["steps_computation_mask"]
    if mask is not None:
      s = self.current_step()
      if s < len(mask) and mask[s] == 1:
        return False
      if self.cfg["steps_computation_policy"] == "static":
        return True
    cfg_step = self.is_cfg_step()
    cached = self.cfg_cached_steps if cfg_step else self.cached_steps
    if self.cfg["max_cached_steps"] >= 0 and len(cached) >= self.cfg["max_cached_steps"]:
      return False
    cont = self.cfg_continuous_cached_steps if cfg_step else self.continuous_cached_steps
    mc = self.cfg["max_continuous_cached_steps"]
    if mc >= 0 and cont >= mc:
      if cfg_step:
        self.cfg_continuous_cached_steps = 0
      else:
        self.continuous_cached_steps = 0
      return False
    cap = self.cfg["max_accumulated_residual_diff_threshold"]
    if cap is not None and cap > 0.0:
      acc = self.cfg_accumulated_residual_diff if cfg_step else self.accumulated_residual_diff
      if acc >= cap:
        return False
    if threshold is None or threshold <= 0.0:
      threshold = self.cfg["residual_diff_threshold"]
    if threshold <= 0.0:
      return False
    k = self.extra["downsample_factor"]
    if k > 1 and "Bn" not in prefix:  # cache_manager.py:937-940
      states = np.ascontiguousarray(states[..., ::k])
    prev = self.get_Bn_buffer(prefix) if "Bn" in prefix else self.get_Fn_buffer(prefix)
    return prev is not None and self.similarity(prev, states, threshold)

  def apply_cache(self, hidden, encoder, prefix, encoder_prefix):
    """cache_manager.py:814-854."""
    approx = self.get_Bn_buffer(prefix)
    assert approx is not None
    hidden = apply_add(approx, hidden, self.dtype) if self.is_cache_residual() else approx
    if encoder is not None:
      e_approx = self.get_Bn_buffer(encoder_prefix, encoder=True)
      if e_approx is not None:
        if self.is_cache_residual(encoder=True):
          encoder = apply_add(e_approx, encoder, self.dtype)
        else:
          encoder = e_approx
    return hidden, encoder


# --------------------------------------------------------------------------- #
# block runner
# --------------------------------------------------------------------------- #

# block(hidden, encoder) -> (hidden, encoder); the runner itself does not care how a
# model orders its block outputs, that is a host-side unpacking detail.
Block = Callable[[np.ndarray, Optional[np.ndarray]], Tuple[np.ndarray, Optional[np.ndarray]]]


def run_blocks(ctx: OracleContext, blocks: Sequence[Block], hidden: np.ndarray,
               encoder: Optional[np.ndarray], name: str = "blocks"):
  """One call of the cached block list (pattern_base.py:198-321). Returns (hidden, encoder, hit)."""
  ctx.set_context()
  fn = ctx.cfg["Fn_compute_blocks"]
  bn = ctx.cfg["Bn_compute_blocks"]
  n = len(blocks)
  dt = ctx.dtype
  h0 = hidden
  for b in blocks[:fn]:
    hidden, encoder = b(hidden, encoder)
  fn_res = residual(hidden, h0, dt)
  ctx.mark_step_begin()
  hit = ctx.can_cache(fn_res, prefix=f"{name}_Fn_residual")
  tail = blocks[n - bn:] if bn > 0 else []
  if hit:
    ctx.add_cached_step()
    p = f"{name}_Bn_residual" if ctx.is_cache_residual() else f"{name}_Bn_hidden_states"
    pe = f"{name}_Bn_residual" if ctx.is_cache_residual(True) else f"{name}_Bn_hidden_states"
    hidden, encoder = ctx.apply_cache(hidden, encoder, p, pe)
  else:
    ctx.set_Fn_buffer(fn_res, f"{name}_Fn_residual")
    h1, e1 = hidden, encoder
    for b in blocks[fn:n - bn if bn > 0 else n]:
      hidden, encoder = b(hidden, encoder)
    if ctx.is_cache_residual():
      ctx.set_Bn_buffer(residual(hidden, h1, dt), f"{name}_Bn_residual")
    else:
      ctx.set_Bn_buffer(hidden, f"{name}_Bn_hidden_states")
    if encoder is not None and e1 is not None:
      if ctx.is_cache_residual(True):
        ctx.set_Bn_buffer(residual(encoder, e1, dt), f"{name}_Bn_residual", encoder=True)
      else:
        ctx.set_Bn_buffer(encoder, f"{name}_Bn_hidden_states", encoder=True)
  for b in tail:
    hidden, encoder = b(hidden, encoder)
  return hidden, encoder, hit
