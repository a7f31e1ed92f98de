"""Host-side state machine of cache_dit_b200 on CPU (checker-backed step-ops double) against the
fixtures produced by the live reference: masks, counters and step indices bit-exact."""
import numpy as np
import pytest

from tests import scenarios as S
from tests.backends import ProductBackend
from tests.fake_ops import OracleStepOps
from tests.golden_io import compare_digests, compare_trace, load_arrays, load_json


@pytest.fixture(autouse=True)
def oracle_ops():
  from cache_dit_b200.caching import step_ops
  saved = step_ops._ops
  ops = OracleStepOps()
  step_ops.set_ops(ops)
  yield ops
  step_ops.set_ops(saved)


@pytest.mark.parametrize("name", S.SMALL)
def test_small_scenarios(name):
  sc = S.BY_NAME[name]
  want = load_json("cache_steps.json")[name]
  res = S.drive(sc, ProductBackend(sc))
  compare_trace(res["trace"], want)
  gold = load_arrays("cache_outputs.npz", name)
  assert sorted(gold) == sorted(res["outputs"])
  for k, w in gold.items():
    g = res["outputs"][k]
    if sc["dtype"] == "fp32":
      np.testing.assert_allclose(g, w, rtol=1e-6, atol=1e-6, err_msg=k)
    else:
      np.testing.assert_array_equal(g, w, err_msg=k)


def test_config1_full_size_mask_and_counters():
  sc = S.BY_NAME["config1_fp32_full"]
  want = load_json("cache_steps.json")[sc["name"]]
  res = S.drive(sc, ProductBackend(sc))
  compare_trace(res["trace"], want)
  assert "".join(map(str, res["trace"]["hits"])) == "0000000011011011011011011011"
  compare_digests(res["trace"]["digests"], want["digests"], rtol=2e-6, atol=1e-6)


def test_one_kernel_per_operation(oracle_ops):
  """Order-1 TaylorSeer: a miss costs one update launch per stream, a hit one apply per stream."""
  sc = S.BY_NAME["small_bf16_o1"]
  S.drive(sc, ProductBackend(sc))
  calls = oracle_ops.calls
  hits = load_json("cache_steps.json")[sc["name"]]["hits"]
  assert calls.count("apply2") + calls.count("apply1") == 2 * sum(hits)  # hidden + encoder
  assert sum(c.startswith("update") for c in calls) <= 2 * (len(hits) - sum(hits))
  assert calls.count("rel_l1") == sum(1 for _ in load_json("cache_steps.json")[sc["name"]]["stats"]["residual_diffs"])
