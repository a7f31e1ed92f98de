"""`enable_cache` + the cached block runner on CPU (checker-backed step-ops double) against the
block-level fixtures produced by the reference's own `enable_cache` on the same toy transformers."""
import numpy as np
import pytest

import cache_dit_b200
from tests import block_scenarios as B
from tests.fake_ops import OracleStepOps
from tests.golden_io import load_arrays, load_json


@pytest.fixture(autouse=True)
def oracle_ops():
  from cache_dit_b200.caching import step_ops
  saved = step_ops._ops
  ops = OracleStepOps()
  step_ops.set_ops(ops)
  yield ops
  step_ops.set_ops(saved)


def compare_block_run(name, trace, outs, diff_rtol=1e-3):
  want = load_json("block_runs.json")[name]
  assert len(trace["stats"]) == len(want["stats"])
  for got_s, want_s in zip(trace["stats"], want["stats"]):
    for k in ("cached_steps", "cfg_cached_steps", "accumulated_cached_steps", "accumulated_executed_steps",
              "accumulated_transformer_executed_steps"):
      assert got_s[k] == want_s[k], (name, k, got_s[k], want_s[k])
    for k in ("residual_diffs", "cfg_residual_diffs"):
      assert sorted(got_s[k]) == sorted(want_s[k]), (name, k)
      for step, w in want_s[k].items():
        assert abs(got_s[k][step] - w) <= diff_rtol * abs(w) + 1e-12, (name, k, step, got_s[k][step], w)
  gold = load_arrays("block_outputs.npz", name)
  assert sorted(gold) == sorted(outs)
  fp32 = B.BY_NAME[name]["dtype"] == "fp32"
  for k, w in gold.items():
    if fp32:
      np.testing.assert_allclose(outs[k], w, rtol=2e-5, atol=2e-6, err_msg=f"{name}/{k}")
    else:
      np.testing.assert_array_equal(outs[k], w, err_msg=f"{name}/{k}")


@pytest.mark.parametrize("name", [r["name"] for r in B.RUNS])
def test_block_runs_match_reference(name, oracle_ops):
  trace, outs = B.execute(B.BY_NAME[name], cache_dit_b200)
  compare_block_run(name, trace, outs)
  # residual formation never runs as a kernel of its own on the hot path: it is fused
  assert "residual" not in oracle_ops.calls or B.BY_NAME[name]["cc"].get("max_warmup_steps", 8) > 0


def test_fused_paths_are_used(oracle_ops):
  run = B.BY_NAME["p1_bf16_F2B1_o1"]
  B.execute(run, cache_dit_b200)
  calls = oracle_ops.calls
  assert any(c == "rel_l1_fused" for c in calls)       # check + Fn residual in one pass
  assert any(c.endswith("_fused") and c.startswith("update") for c in calls)  # Mn residual + ladder
  assert "rel_l1" not in calls


def test_summary_and_strify():
  run = B.BY_NAME["p0_fp32_F2B0_o1"]
  model = B.build(run)
  cd = cache_dit_b200
  adapter = cd.BlockAdapter(transformer=model, blocks=model.transformer_blocks,
                            forward_pattern=cd.ForwardPattern.Pattern_0, check_forward_pattern=False)
  cd.enable_cache(adapter, cache_config=cd.DBCacheConfig(Fn_compute_blocks=2, max_warmup_steps=3,
                                                          num_inference_steps=run["steps"],
                                                          enable_separate_cfg=False),
                  calibrator_config=cd.TaylorSeerCalibratorConfig())
  import torch
  with torch.no_grad():
    for h, e, scale in B.inputs(run):
      model(h, e, scale=scale)
  stats = cd.summary(model, logging=False)
  assert stats[-1].cached_steps == load_json("block_runs.json")[run["name"]]["stats"][0]["cached_steps"]
  assert stats[-1].cache_options["cache_config"].Fn_compute_blocks == 2
  assert cd.strify(model).startswith("DBCache_F2B0_W3I1M0MC0_R0.08_N16_CFG0_T1O1_S")
  cd.disable_cache(adapter)
  assert cd.summary(model, logging=False)[0].cached_steps == []
  assert "forward" not in vars(model)


def test_missing_context_runs_uncached(caplog):
  import torch
  cd = cache_dit_b200
  run = B.BY_NAME["p1_fp32_F1B0_plain"]
  model = B.build(run)
  plain = [model(h, e, scale=s) for h, e, s in list(B.inputs(run))[:2]]
  adapter = cd.BlockAdapter(transformer=model, blocks=model.transformer_blocks,
                            forward_pattern=cd.ForwardPattern.Pattern_1, check_forward_pattern=False)
  cd.enable_cache(adapter, cache_config=cd.DBCacheConfig(Fn_compute_blocks=1, enable_separate_cfg=False))
  model._context_manager.clear_contexts()
  model._context_manager._persistent_context = False
  got = [model(h, e, scale=s) for h, e, s in list(B.inputs(run))[:2]]
  for a, b in zip(plain, got):
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])


def test_bad_block_counts_assert():
  cd = cache_dit_b200
  run = B.BY_NAME["p0_fp32_F2B0_o1"]
  model = B.build(run)
  adapter = cd.BlockAdapter(transformer=model, blocks=model.transformer_blocks,
                            forward_pattern=cd.ForwardPattern.Pattern_0, check_forward_pattern=False)
  cd.enable_cache(adapter, cache_config=cd.DBCacheConfig(Fn_compute_blocks=11, enable_separate_cfg=False))
  h, e, s = next(B.inputs(run))
  with pytest.raises(AssertionError):
    model(h, e, scale=s)
