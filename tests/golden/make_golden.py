"""Generate the golden fixtures by running the UNMODIFIED reference on CPU.

Usage (only where a checkout of the reference exists; the fixtures it writes are committed):

    python tests/golden/make_golden.py --reference /path/to/cache-dit [--only NAME ...]

What it does
  * cache-step scenarios (tests/scenarios.py): imports the reference's
    `cache_dit.caching.cache_contexts` (with `cache_dit` and `cache_dit.caching` pre-registered as
    empty packages so that the package __init__ files, which need diffusers, are skipped) and
    drives its `CachedContextManager` exactly as its block runner does
    (src/cache_dit/caching/cache_blocks/pattern_base.py:236-312).
  * block-level scenarios (tests/block_scenarios.py): imports the whole reference package behind
    a stub `diffusers` finder and runs `cache_dit.enable_cache` on toy transformers.
  * TaylorSeer known-answer case.

Outputs: tests/golden/cache_steps.json, tests/golden/cache_outputs.npz,
         tests/golden/block_runs.json, tests/golden/block_outputs.npz, tests/golden/taylor_kat.json,
         tests/golden/host_tables.json, tests/golden/load_configs.json (tests/config_cases.py through the
         reference's `load_cache_config` / `load_parallelism_config`)
"""
from __future__ import annotations

import argparse
import importlib.abc
import importlib.machinery
import json
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from tests import scenarios as S  # noqa: E402
from tests.backends import PREFIX, stats_dict  # noqa: E402


def import_reference(ref_root: str):
  """Import the full reference package with a stand-in for the absent `diffusers`."""
  src = os.path.join(ref_root, "src")

  class _Stub(importlib.abc.MetaPathFinder, importlib.abc.Loader):

    def find_spec(self, name, path, target=None):
      if name == "diffusers" or name.startswith("diffusers."):
        return importlib.machinery.ModuleSpec(name, self, is_package=True)
      return None

    def create_module(self, spec):
      m = types.ModuleType(spec.name)
      m.__path__ = []

      def fabricate(attr):
        if attr.startswith("__"):
          raise AttributeError(attr)
        return type(attr, (object, ), {})

      m.__getattr__ = fabricate
      return m

    def exec_module(self, module):
      pass

  sys.meta_path.insert(0, _Stub())
  import diffusers
  diffusers.__version__ = "0.37.0"
  diffusers.DiffusionPipeline = type("DiffusionPipeline", (object, ), {})
  diffusers.ModelMixin = type("ModelMixin", (torch.nn.Module, ), {})
  import diffusers.models.modeling_utils as mu
  mu.ModelMixin = diffusers.ModelMixin
  sys.path.insert(0, src)
  import cache_dit
  return cache_dit


class ReferenceBackend:
  """tests/scenarios.py backend on top of the reference's CachedContextManager."""

  def __init__(self, cache_dit, sc: dict):
    from cache_dit.caching.cache_contexts.cache_manager import CachedContextManager
    from cache_dit import DBCacheConfig, TaylorSeerCalibratorConfig
    cc = dict(sc["cache_config"])
    cc.setdefault("enable_separate_cfg", False)
    cal = sc["calibrator_config"]
    self.mgr = CachedContextManager("golden", persistent_context=True)
    extra = {}
    if sc.get("extra_config"):
      from cache_dit.caching.cache_contexts.cache_config import ExtraCacheConfig
      extra["extra_cache_config"] = ExtraCacheConfig(**sc["extra_config"])
    self.mgr.new_context(
      name="ctx", cache_config=DBCacheConfig(**cc),
      calibrator_config=None if cal is None else TaylorSeerCalibratorConfig(**cal), **extra)

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
    return self.mgr.can_cache(r, parallelized=False, prefix=f"{PREFIX}_Fn_residual")

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

  @staticmethod
  def from_torch(t):
    return t

  @staticmethod
  def to_numpy(t):
    return t.float().numpy()


def taylor_known_answer(cache_dit) -> dict:
  """Y_t = t^2 constants through set_Bn_buffer at context steps 0..5, read back at step 7."""
  from cache_dit.caching.cache_contexts.cache_manager import CachedContextManager
  from cache_dit import DBCacheConfig, TaylorSeerCalibratorConfig
  mgr = CachedContextManager("kat", persistent_context=True)
  mgr.new_context(name="ctx", cache_config=DBCacheConfig(enable_separate_cfg=False),
                  calibrator_config=TaylorSeerCalibratorConfig(taylorseer_order=1))
  state_steps, d1 = [], []
  for t in range(6):
    mgr.set_context("ctx")
    mgr.mark_step_begin()
    mgr.set_Bn_buffer(torch.full((1, 2, 3), float(t * t)), prefix="b_Bn_residual")
    st = mgr.get_calibrator()[0].states["b_Bn_residual"]
    state_steps.append(int(st.current_step))
    d = st.state["dY_current"][1]
    d1.append(None if d is None else float(d.flatten()[0]))
  for _ in range(2):
    mgr.set_context("ctx")
    mgr.mark_step_begin()
  approx = mgr.get_Bn_buffer("b_Bn_residual")
  return dict(state_steps=state_steps, d1=d1, approx_at_7=float(approx.flatten()[0]))


def steps_mask_table(cache_dit) -> dict:
  """`steps_mask` for every predefined policy over a range of schedule lengths, plus explicit bins."""
  table = {}
  for total in [4, 6] + list(range(8, 61)) + [64, 75, 100, 128]:
    for policy in ("slow", "medium", "fast", "ultra"):
      table[f"{policy}/{total}"] = cache_dit.steps_mask(total_steps=total, mask_policy=policy)
  table["bins/a"] = cache_dit.steps_mask(compute_bins=[4, 2, 1], cache_bins=[3, 5, 2])
  table["bins/b"] = cache_dit.steps_mask(compute_bins=[6, 1, 1, 1], cache_bins=[1, 2, 5], total_steps=14)
  return table


def config_tags(cache_dit) -> dict:
  c = cache_dit
  return {
    "default": c.DBCacheConfig().strify(),
    "scm": c.DBCacheConfig(Fn_compute_blocks=1, max_warmup_steps=4, max_cached_steps=10,
                           max_continuous_cached_steps=3, residual_diff_threshold=0.12,
                           steps_computation_mask=[1, 0, 1, 0], steps_computation_policy="static",
                           num_inference_steps=4, force_refresh_step_hint=2, enable_separate_cfg=True).strify(),
    "taylor": c.TaylorSeerCalibratorConfig(taylorseer_order=2).strify(),
    "taylor_details": c.TaylorSeerCalibratorConfig(taylorseer_order=2).strify(details=True),
  }


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--reference", required=True)
  ap.add_argument("--only", nargs="*", default=None)
  ap.add_argument("--load-configs-only", action="store_true", help="write load_configs.json and nothing else")
  args = ap.parse_args()
  torch.set_num_threads(os.cpu_count() or 1)
  cache_dit = import_reference(args.reference)
  from tests import config_cases
  json.dump(config_cases.run_cases(cache_dit), open(os.path.join(HERE, "load_configs.json"), "w"), indent=1,
            sort_keys=True)
  if args.load_configs_only:
    return

  steps_path = os.path.join(HERE, "cache_steps.json")
  out_path = os.path.join(HERE, "cache_outputs.npz")
  traces = json.load(open(steps_path)) if os.path.exists(steps_path) else {}
  arrays = dict(np.load(out_path)) if os.path.exists(out_path) else {}
  for sc in S.SCENARIOS:
    if args.only and sc["name"] not in args.only:
      continue
    res = S.drive(sc, ReferenceBackend(cache_dit, sc))
    traces[sc["name"]] = res["trace"]
    for k in [k for k in arrays if k.startswith(sc["name"] + "/")]:
      del arrays[k]
    for k, v in res["outputs"].items():
      arrays[f"{sc['name']}/{k}"] = v
    print(sc["name"], "".join(map(str, res["trace"]["hits"])))
  json.dump(traces, open(steps_path, "w"), indent=1, sort_keys=True)
  np.savez_compressed(out_path, **arrays)

  if not args.only:
    json.dump(taylor_known_answer(cache_dit), open(os.path.join(HERE, "taylor_kat.json"), "w"),
              indent=1)
    json.dump(dict(steps_mask=steps_mask_table(cache_dit), tags=config_tags(cache_dit)),
              open(os.path.join(HERE, "host_tables.json"), "w"), sort_keys=True)
    try:
      from tests import block_scenarios as B
    except ImportError:
      B = None
    if B is not None:
      runs, outs = B.run_reference(cache_dit)
      json.dump(runs, open(os.path.join(HERE, "block_runs.json"), "w"), indent=1, sort_keys=True)
      np.savez_compressed(os.path.join(HERE, "block_outputs.npz"), **outs)


if __name__ == "__main__":
  main()
