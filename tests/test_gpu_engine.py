"""The product path on a B200: cache_dit_b200's manager and block runner with the real kernels,
against the reference's fixtures (cache-step scenarios) and against the numpy oracle plugged into
the same runner (block-level runs, whose toy blocks compute on the GPU)."""
import numpy as np
import pytest
import torch

import cache_dit_b200
from tests import block_scenarios as B
from tests import scenarios as S
from tests.backends import ProductBackend
from tests.fake_ops import OracleStepOps
from tests.golden_io import compare_digests, compare_trace, load_arrays, load_json

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def device_ops():
  from cache_dit_b200.caching import step_ops
  step_ops.set_ops(None)  # the default: sm_100a kernels
  ops = step_ops.get_ops()
  assert ops.name == "sm_100a"
  yield ops
  step_ops.set_ops(None)


@pytest.mark.parametrize("name", S.SMALL)
def test_small_scenarios_on_gpu(name):
  sc = S.BY_NAME[name]
  want = load_json("cache_steps.json")[name]
  res = S.drive(sc, ProductBackend(sc, device="cuda"))
  compare_trace(res["trace"], want)  # masks / counters bit-exact, diffs within 1e-3 relative
  gold = load_arrays("cache_outputs.npz", name)
  assert sorted(gold) == sorted(res["outputs"])
  for k, w in gold.items():
    g = res["outputs"][k]
    if sc["dtype"] == "fp32":
      np.testing.assert_allclose(g, w, rtol=1e-6, atol=1e-6, err_msg=k)
    else:
      np.testing.assert_array_equal(g, w, err_msg=k)


@pytest.mark.parametrize("name", S.FULL)
def test_full_size_scenarios_on_gpu(name):
  sc = S.BY_NAME[name]
  want = load_json("cache_steps.json")[name]
  res = S.drive(sc, ProductBackend(sc, device="cuda"))
  compare_trace(res["trace"], want)
  compare_digests(res["trace"]["digests"], want["digests"], rtol={"fp32": 2e-6, "bf16": 2**-7}[sc["dtype"]],
                  atol=1e-6)


@pytest.mark.parametrize("name", [r["name"] for r in B.RUNS])
def test_block_runs_kernels_vs_oracle_on_gpu(name):
  from cache_dit_b200.caching import step_ops
  run = B.BY_NAME[name]
  got_trace, got = B.execute(run, cache_dit_b200, device="cuda")
  step_ops.set_ops(OracleStepOps())
  want_trace, want = B.execute(run, cache_dit_b200, device="cuda")
  for gs, ws in zip(got_trace["stats"], want_trace["stats"]):
    for k in ("cached_steps", "cfg_cached_steps", "accumulated_cached_steps", "accumulated_executed_steps"):
      assert gs[k] == ws[k], (name, k, gs[k], ws[k])
    for k in ("residual_diffs", "cfg_residual_diffs"):
      assert sorted(gs[k]) == sorted(ws[k])
      for step, w in ws[k].items():
        assert abs(gs[k][step] - w) <= 1e-3 * abs(w) + 1e-12
  assert sorted(got) == sorted(want)
  for k in want:
    if run["dtype"] == "fp32":
      np.testing.assert_allclose(got[k], want[k], rtol=2e-5, atol=2e-6, err_msg=k)
    else:
      np.testing.assert_array_equal(got[k], want[k], err_msg=k)


def test_cpu_tensors_are_refused():
  sc = S.BY_NAME["small_bf16_o1"]
  with pytest.raises(RuntimeError):
    S.drive(sc, ProductBackend(sc, device="cpu"))
