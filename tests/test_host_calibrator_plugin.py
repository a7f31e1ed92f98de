"""The calibrator extension point: anything with `reset_cache / approximate / mark_step_begin / update`
registered under a `calibrator_type` is driven by the cache engine exactly like the built-in TaylorSeer
(the reference's interface: src/cache_dit/caching/cache_contexts/calibrators/base.py:8-49, factory keyed on
`calibrator_type` at calibrators/__init__.py:283-293)."""
import dataclasses

import numpy as np
import pytest
import torch

import cache_dit_b200 as cd
from tests import block_scenarios as B
from tests.fake_ops import OracleStepOps

LOG = []


class HoldLast(cd.CalibratorBase):
  """Forecast = the last value seen (a zeroth-order hold), with a log of every call."""

  def __init__(self, gain=1.0):
    self.gain = gain
    self.values = {}
    LOG.append(("init", gain))

  def reset_cache(self):
    self.values.clear()
    LOG.append(("reset_cache", ))

  def mark_step_begin(self):
    LOG.append(("mark_step_begin", ))

  def update(self, Y, name="default"):
    assert isinstance(Y, torch.Tensor)  # third-party calibrators get a materialised tensor
    self.values[name] = Y.clone()
    LOG.append(("update", name))

  def approximate(self, name="default"):
    LOG.append(("approximate", name))
    return (self.values[name] * self.gain).to(self.values[name].dtype)


@dataclasses.dataclass
class HoldLastConfig(cd.CalibratorConfig):
  enable_calibrator: bool = True  # the base class leaves both streams off
  enable_encoder_calibrator: bool = True
  calibrator_type: str = "hold_last"
  gain: float = 1.0

  def strify(self, **kwargs) -> str:
    return f"Hold({self.gain})"

  def to_kwargs(self):
    return {"gain": self.gain}


@pytest.fixture(autouse=True)
def oracle_ops():
  from cache_dit_b200.caching import step_ops
  saved = step_ops._ops
  step_ops.set_ops(OracleStepOps())
  cd.Calibrator.register("hold_last", HoldLast)
  LOG.clear()
  yield
  step_ops.set_ops(saved)
  cd.Calibrator._registry.pop("hold_last", None)
  cd.Calibrator._supported_calibrators.remove("hold_last")


def run(calibrator_config, steps=10):
  spec = dict(B.BY_NAME["p1_bf16_F2B1_o1"], steps=steps)
  model = B.build(spec)
  adapter = cd.BlockAdapter(transformer=model, blocks=model.transformer_blocks, forward_pattern=cd.Pattern_1,
                            check_forward_pattern=False)
  cd.enable_cache(adapter, cache_config=cd.DBCacheConfig(Fn_compute_blocks=2, Bn_compute_blocks=1, max_warmup_steps=2,
                                                         residual_diff_threshold=0.3, num_inference_steps=steps,
                                                         enable_separate_cfg=False),
                  calibrator_config=calibrator_config)
  outs = []
  try:
    cd.refresh_context(model, num_inference_steps=steps)
    with torch.no_grad():
      for h, e, scale in B.inputs(spec):
        y = model(h, e, scale=scale)
        outs.append([t.float().numpy() for t in (y if isinstance(y, tuple) else (y, ))])
    return outs, list(model._cached_steps)
  finally:
    cd.disable_cache(adapter)


def test_base_config_leaves_calibrators_off():
  run(dataclasses.replace(HoldLastConfig(), enable_calibrator=False, enable_encoder_calibrator=False))
  assert not LOG  # plain buffers hold the residuals, nothing is built


def test_registered_calibrator_is_driven_like_taylorseer():
  outs, cached = run(HoldLastConfig(gain=1.0))
  assert cached, "the schedule must hit the cache for the test to say anything"
  kinds = [entry[0] for entry in LOG]
  assert kinds.count("mark_step_begin") >= 10  # once per step and stream calibrator
  assert "update" in kinds and "approximate" in kinds
  # an approximate is only ever asked of a name that was updated before
  seen = set()
  for entry in LOG:
    if entry[0] == "update":
      seen.add(entry[1])
    if entry[0] == "approximate":
      assert entry[1] in seen
  # hidden and encoder stream each have their own instance (four per context with CFG, two without)
  assert kinds.count("init") >= 2
  # order-0 TaylorSeer-like behaviour: same masks as the built-in calibrator at this threshold
  _, cached_taylor = run(cd.TaylorSeerCalibratorConfig(taylorseer_order=1))
  assert cached == cached_taylor  # the decision does not depend on the calibrator


def test_calibrator_kwargs_reach_the_factory_and_change_the_forecast():
  base, cached = run(HoldLastConfig(gain=1.0))
  LOG.clear()
  scaled, cached2 = run(HoldLastConfig(gain=0.5))
  assert ("init", 0.5) in LOG and cached == cached2
  hit = cached[0]
  assert not np.array_equal(base[hit][0], scaled[hit][0])  # a cached step uses the forecast
  miss = next(i for i in range(len(base)) if i not in cached)
  np.testing.assert_array_equal(base[miss][0], scaled[miss][0])  # a computed step does not


def test_unknown_calibrator_type_is_refused():
  @dataclasses.dataclass
  class Nope(cd.CalibratorConfig):
    calibrator_type: str = "nope"

  with pytest.raises(AssertionError):
    cd.Calibrator(Nope())
