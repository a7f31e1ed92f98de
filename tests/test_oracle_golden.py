"""The numpy oracle against the fixtures produced by the live reference (CPU only)."""
import numpy as np
import pytest

from oracle import cache_oracle as O
from tests import scenarios as S
from tests.backends import OracleBackend
from tests.golden_io import compare_digests, compare_trace, load_arrays, load_json

# storage-dtype one-ulp tolerances for elementwise outputs
ULP = {"fp32": 2e-6, "bf16": 2**-7, "fp16": 2**-10}


@pytest.mark.parametrize("name", S.SMALL)
def test_small_scenarios_match_reference(name):
  sc = S.BY_NAME[name]
  want = load_json("cache_steps.json")[name]
  res = S.drive(sc, OracleBackend(sc))
  compare_trace(res["trace"], want)
  gold = load_arrays("cache_outputs.npz", name)
  assert sorted(gold) == sorted(res["outputs"])
  for k, w in gold.items():
    g = res["outputs"][k]
    if sc["dtype"] == "fp32":
      np.testing.assert_allclose(g, w, rtol=1e-6, atol=1e-6, err_msg=k)
    else:
      # same per-op rounding as the reference: results are identical, not merely close
      np.testing.assert_array_equal(g, w, err_msg=k)


@pytest.mark.parametrize("name", S.FULL)
def test_full_size_scenarios_match_reference(name):
  sc = S.BY_NAME[name]
  want = load_json("cache_steps.json")[name]
  res = S.drive(sc, OracleBackend(sc))
  compare_trace(res["trace"], want)
  compare_digests(res["trace"]["digests"], want["digests"], rtol=ULP[sc["dtype"]], atol=1e-6)


def test_taylor_known_answer():
  kat = load_json("taylor_kat.json")
  ctx = O.OracleContext(dict(), dict(taylorseer_order=1), "fp32")
  steps, d1 = [], []
  for t in range(6):
    ctx.set_context()
    ctx.mark_step_begin()
    ctx.set_Bn_buffer(np.full((1, 2, 3), float(t * t), np.float32), "b_Bn_residual")
    st = ctx.calibrator.states["b_Bn_residual"]
    steps.append(st.current_step)
    d1.append(None if st.cur[1] is None else float(st.cur[1].flat[0]))
  for _ in range(2):
    ctx.set_context()
    ctx.mark_step_begin()
  assert steps == kat["state_steps"]
  assert d1 == kat["d1"]
  assert float(ctx.get_Bn_buffer("b_Bn_residual").flat[0]) == kat["approx_at_7"]


def test_bf16_rounding_matches_torch():
  import torch
  g = torch.Generator().manual_seed(0)
  x = torch.randn(100000, generator=g) * torch.exp(4 * torch.randn(100000, generator=g))
  x = torch.cat([x, torch.tensor([0.0, -0.0, 1.0, 3.3895314e38, float("inf"), 1e-40])])
  want = x.to(torch.bfloat16).float().numpy()
  np.testing.assert_array_equal(O.round_bf16(x.numpy()), want)


def test_sharded_mean_of_means_differs_only_for_uneven_shards():
  rng = np.random.RandomState(0)
  prev = rng.randn(1, 6889, 8).astype(np.float32)
  prev[:, :3000] *= 4.0  # make the shards' means unequal
  cur = prev + 0.05 * rng.randn(*prev.shape).astype(np.float32)
  whole = O.rel_l1(prev, cur, "fp32")
  even = O.rel_l1(prev[:, :6888], cur[:, :6888], "fp32", shards=8)
  assert abs(even - O.rel_l1(prev[:, :6888], cur[:, :6888], "fp32")) < 1e-3 * whole
  assert O.rel_l1(prev, cur, "fp32", shards=8) != whole


def test_torch_cpu_ops_equal_the_numpy_restatement():
  """oracle/cache_ops_torch.py (the reference's eager op sequences on CPU tensors, used to time the CPU baseline)
  against oracle/cache_oracle.py on bf16 and fp32 inputs: same bits for every tensor result, same check value."""
  import numpy as np
  import torch
  from oracle import cache_ops_torch as T
  from oracle import cache_oracle as O
  g = torch.Generator().manual_seed(3)
  for dtype, name in ((torch.bfloat16, "bf16"), (torch.float32, "fp32")):
    prev = torch.randn(1, 96, 320, generator=g).to(dtype)
    cur = (prev.float() + 0.05 * torch.randn(1, 96, 320, generator=g)).to(dtype)
    older = (prev.float() - 0.07 * torch.randn(1, 96, 320, generator=g)).to(dtype)
    f = lambda t: t.float().numpy()
    assert T.rel_l1(prev, cur) == float(O.rel_l1(f(prev), f(cur), name))
    np.testing.assert_array_equal(f(T.residual(cur, prev)), O.residual(f(cur), f(prev), name))
    y = T.residual(cur, prev)
    got = T.taylor_derivatives(y, [older, None], 3, True)
    want = O.taylor_derivatives(f(y), [f(older), None], 3, True, name)
    np.testing.assert_array_equal(f(got[1]), want[1])
    np.testing.assert_array_equal(f(T.taylor_series(got, 2)), O.taylor_series(want, 2, name))
    np.testing.assert_array_equal(f(T.apply_add(T.taylor_series(got, 2), cur)),
                                  O.apply_add(O.taylor_series(want, 2, name), f(cur), name))
