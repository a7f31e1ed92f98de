"""Calibrators: how a cached tensor is forecast for a skipped step.

Public names and the calibrator interface (`reset_cache`, `mark_step_begin`, `update`,
`approximate`) follow the reference (src/cache_dit/caching/cache_contexts/calibrators/base.py:8-49,
.../calibrators/__init__.py:14-293).  TaylorSeer (.../calibrators/taylorseer.py) is implemented on
top of two kernels; its state keeps the derivative ladder in two engine-owned buffer sets that swap
roles at every update, so "dY_prev = dY_current" is a pointer swap and no kernel ever reads a buffer
it writes.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional

import torch

from .step_ops import get_ops


# ------------------------------------------------------------------------------ configs
@dataclasses.dataclass
class CalibratorConfig:
  enable_calibrator: bool = False
  enable_encoder_calibrator: bool = False
  calibrator_type: str = "taylorseer"
  calibrator_cache_type: str = "residual"  # "residual" or "hidden_states"
  calibrator_kwargs: Dict[str, Any] = dataclasses.field(default_factory=dict)

  def strify(self, **kwargs) -> str:
    return "CalibratorBase"

  def to_kwargs(self) -> Dict:
    return self.calibrator_kwargs.copy()

  def as_dict(self) -> dict:
    return dataclasses.asdict(self)

  def update(self, **kwargs) -> "CalibratorConfig":
    for key, value in kwargs.items():
      if hasattr(self, key) and value is not None:
        setattr(self, key, value)
    return self

  def empty(self, **kwargs) -> "CalibratorConfig":
    for field in dataclasses.fields(self):
      if field.name != "calibrator_type":
        setattr(self, field.name, None)
    if kwargs:
      self.update(**kwargs)
    return self

  def reset(self, **kwargs) -> "CalibratorConfig":
    return self.empty(**kwargs)


@dataclasses.dataclass
class TaylorSeerCalibratorConfig(CalibratorConfig):
  """TaylorSeer (arXiv 2503.06923): forecast by a Taylor series over finite differences."""
  enable_calibrator: bool = True
  enable_encoder_calibrator: bool = True
  calibrator_type: str = "taylorseer"
  taylorseer_order: int = 1

  def strify(self, **kwargs) -> str:
    if kwargs.get("details", False):
      return f"TaylorSeer_O({self.taylorseer_order})" if self.taylorseer_order else "NONE"
    return f"T1O{self.taylorseer_order}" if self.taylorseer_order else "NONE"

  def to_kwargs(self) -> Dict:
    kwargs = self.calibrator_kwargs.copy()
    kwargs["n_derivatives"] = self.taylorseer_order
    return kwargs


# ------------------------------------------------------------------------------ interface
class CalibratorBase:
  """Extension point: anything with these four methods can forecast cached tensors."""

  def reset_cache(self, *args, **kwargs):
    raise NotImplementedError("reset_cache method is not implemented.")

  def approximate(self, *args, **kwargs):
    raise NotImplementedError("approximate method is not implemented.")

  def mark_step_begin(self, *args, **kwargs):
    raise NotImplementedError("mark_step_begin method is not implemented.")

  def update(self, *args, **kwargs):
    raise NotImplementedError("update method is not implemented.")

  def __repr__(self):
    return "CalibratorBase"


# ------------------------------------------------------------------------------ TaylorSeer
MAX_DERIVATIVES = 4  # the kernels take up to 5 Taylor terms


class TaylorSeerState:
  """Derivative ladder of one named tensor stream."""

  def __init__(self, n_derivatives=1, max_warmup_steps=1, skip_interval_steps=1):
    if not 0 <= n_derivatives <= MAX_DERIVATIVES:
      raise ValueError(f"taylorseer order must be in [0, {MAX_DERIVATIVES}], got {n_derivatives}")
    self.n_derivatives = n_derivatives
    self.order = n_derivatives + 1
    self.max_warmup_steps = max_warmup_steps
    self.skip_interval_steps = skip_interval_steps
    self.reset()

  def reset(self):
    self.current_step = -1
    self.last_non_approximated_step = -1
    self._prev: List[Optional[torch.Tensor]] = [None] * self.order
    self._cur: List[Optional[torch.Tensor]] = [None] * self.order
    self._sets: List[List[Optional[torch.Tensor]]] = [[None] * self.order, [None] * self.order]
    self._parity = 0

  @property
  def state(self) -> Dict[str, List[Optional[torch.Tensor]]]:
    return {"dY_prev": self._prev, "dY_current": self._cur}

  def mark_step_begin(self):
    self.current_step += 1

  def should_compute(self, step=None):
    step = self.current_step if step is None else step
    return (step < self.max_warmup_steps
            or (step - self.max_warmup_steps + 1) % self.skip_interval_steps == 0)

  # -- update ------------------------------------------------------------------------------
  def _slot(self, k: int, like: torch.Tensor) -> torch.Tensor:
    buf = self._sets[self._parity][k]
    if buf is None or buf.shape != like.shape or buf.dtype != like.dtype or buf.device != like.device:
      buf = get_ops().empty_like(like)
      self._sets[self._parity][k] = buf
    return buf

  def _advance(self, after: torch.Tensor, before: Optional[torch.Tensor]):
    """Common part of `update` / `update_residual`: rotate the ladder, launch one kernel."""
    window = self.current_step - self.last_non_approximated_step
    prev = self._cur
    if prev[0] is not None and prev[0].shape != after.shape:
      # a change of shape drops the history, step counters included (taylorseer.py:80-82)
      self.reset()
      prev = self._prev
    self._parity ^= 1
    n_new = 0
    if self.current_step > 1:
      while n_new < self.n_derivatives and prev[n_new] is not None:
        n_new += 1
    cur: List[Optional[torch.Tensor]] = [None] * self.order
    cur[0] = self._slot(0, after) if before is not None else after
    for k in range(n_new):
      cur[k + 1] = self._slot(k + 1, after)
    get_ops().taylor_update(after, before, prev[:n_new], cur[:n_new + 1], n_new, window)
    self._prev = prev
    self._cur = cur
    self.last_non_approximated_step = self.current_step

  def update(self, Y: torch.Tensor):
    """Record a fully computed tensor; `Y` is kept by reference as dY[0] (taylorseer.py:106-127)."""
    self._advance(Y, None)

  def update_residual(self, after: torch.Tensor, before: torch.Tensor):
    """Same as `update(after - before)` with the subtraction fused into the ladder kernel."""
    self._advance(after, before)

  def derivative(self, Y: torch.Tensor) -> List[Optional[torch.Tensor]]:
    """The ladder `update(Y)` would store, without committing it."""
    saved = (self.current_step, self.last_non_approximated_step, self._prev, self._cur,
             [list(s) for s in self._sets], self._parity)
    self._sets = [[None] * self.order, [None] * self.order]
    self._advance(Y, None)
    out = self._cur
    (self.current_step, self.last_non_approximated_step, self._prev, self._cur, self._sets,
     self._parity) = saved
    return out

  # -- approximate ----------------------------------------------------------------------------
  def _terms(self) -> List[torch.Tensor]:
    terms = []
    for d in self._cur:
      if d is None:
        break
      terms.append(d)
    return terms

  def approximate(self) -> torch.Tensor:
    """sum_i dY[i] * elapsed^i / i!  (taylorseer.py:91-104)."""
    terms = self._terms()
    if not terms:
      return 0
    out = get_ops().empty_like(terms[0])
    elapsed = self.current_step - self.last_non_approximated_step
    return get_ops().taylor_apply(None, terms, elapsed, False, out)

  def approximate_add(self, hidden: torch.Tensor, add_hidden: bool = True) -> torch.Tensor:
    """`approximate() + hidden` (or just `approximate()`) in one pass over memory."""
    terms = self._terms()
    assert terms, "approximate called before the first update"
    out = get_ops().empty_like(hidden if add_hidden else terms[0])
    elapsed = self.current_step - self.last_non_approximated_step
    return get_ops().taylor_apply(hidden, terms, elapsed, add_hidden, out)

  def step(self, Y: torch.Tensor):
    self.mark_step_begin()
    if self.should_compute():
      self.update(Y)
      return Y
    return self.approximate()


class TaylorSeerCalibrator(CalibratorBase):
  """Name-keyed TaylorSeer states; a state is created by its first update."""

  def __init__(self, n_derivatives=1, max_warmup_steps=1, skip_interval_steps=1, **kwargs):
    self.n_derivatives = n_derivatives
    self.max_warmup_steps = max_warmup_steps
    self.skip_interval_steps = skip_interval_steps
    self.states: Dict[str, TaylorSeerState] = {}

  def reset_cache(self):
    for state in self.states.values():
      state.reset()

  def maybe_init_state(self, name: str = "default"):
    if name not in self.states:
      self.states[name] = TaylorSeerState(self.n_derivatives, self.max_warmup_steps,
                                          self.skip_interval_steps)

  def mark_step_begin(self, *args, **kwargs):
    for state in self.states.values():
      state.mark_step_begin()

  def derivative(self, Y: torch.Tensor, name: str = "default"):
    self.maybe_init_state(name)
    return self.states[name].derivative(Y)

  def approximate(self, name: str = "default") -> torch.Tensor:
    assert name in self.states, f"State '{name}' not found."
    return self.states[name].approximate()

  def approximate_add(self, hidden: torch.Tensor, name: str = "default", add_hidden: bool = True):
    assert name in self.states, f"State '{name}' not found."
    return self.states[name].approximate_add(hidden, add_hidden)

  def update(self, Y: torch.Tensor, name: str = "default"):
    self.maybe_init_state(name)
    self.states[name].update(Y)

  def update_residual(self, after: torch.Tensor, before: torch.Tensor, name: str = "default"):
    self.maybe_init_state(name)
    self.states[name].update_residual(after, before)

  def step(self, Y: torch.Tensor, name: str = "default"):
    self.maybe_init_state(name)
    return self.states[name].step(Y)

  def __repr__(self):
    return f"TaylorSeerCalibrator_O({self.n_derivatives})"


class Calibrator:
  """Factory keyed on `calibrator_type` (calibrators/__init__.py:264-293 of the reference).

  Only TaylorSeer is built here; other types can be registered through `register`."""

  _registry = {"taylorseer": TaylorSeerCalibrator}
  _supported_calibrators = ["taylorseer"]

  @classmethod
  def register(cls, calibrator_type: str, factory) -> None:
    cls._registry[calibrator_type.lower()] = factory
    if calibrator_type.lower() not in cls._supported_calibrators:
      cls._supported_calibrators.append(calibrator_type.lower())

  def __new__(cls, calibrator_config: CalibratorConfig) -> CalibratorBase:
    kind = calibrator_config.calibrator_type.lower()
    assert kind in cls._registry, f"Calibrator {calibrator_config.calibrator_type} is not supported now!"
    return cls._registry[kind](**calibrator_config.to_kwargs())
