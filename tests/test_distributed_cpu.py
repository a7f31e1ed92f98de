"""World-size-2 `gloo` runs on CPU: the cross-rank cache decision and the context-parallel plan."""
import json
import os
import subprocess
import sys

import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def results(tmp_path_factory):
  out = tmp_path_factory.mktemp("dist")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
         "127.0.0.1", "--master-port", "29631", os.path.join(HERE, "dist_worker.py"), str(out)]
  env = dict(os.environ, OMP_NUM_THREADS="2")
  proc = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
  assert proc.returncode == 0, proc.stdout[-3000:]
  return [json.load(open(os.path.join(out, f"rank{r}.json"))) for r in range(2)]


def test_every_rank_takes_the_same_branch(results):
  a, b = results[0]["decision"], results[1]["decision"]
  assert a["hits"] == b["hits"]
  assert a["diffs"] == b["diffs"]


def test_reduced_value_is_the_mean_of_local_means(results):
  d = results[0]["decision"]
  got = d["diffs"]["1"]
  assert abs(got - d["want"]) <= 1e-3 * d["want"]


def test_context_parallel_matches_single_rank(results):
  for r in results:
    f = r["flux"]
    assert f["cached_single"] == f["cached_sharded"]
    assert f["rel"] < 2e-3
    for k, v in f["diffs_single"].items():
      # equal shards: mean of local means equals the global mean up to float rounding
      assert abs(f["diffs_sharded"][k] - v) <= 2e-3 * abs(v) + 1e-9
  assert results[0]["flux"]["cached_sharded"] == results[1]["flux"]["cached_sharded"]


@pytest.mark.parametrize("model", ["qwen", "wan"])
def test_other_model_plans_match_single_rank(results, model):
  """Qwen-Image-shape: uneven token split (25/24 image, 3/2 text); Wan-shape: video sharded, text whole."""
  for r in results:
    f = r[model]
    assert f["cached_single"] == f["cached_sharded"] and f["cached_single"]
    assert f["rel"] < 2e-3
    for k, v in f["diffs_single"].items():
      # mean of local means vs global mean: equal up to float rounding for equal shards, and within
      # the shard-size imbalance (1 token in 25) times the spread of per-token means otherwise
      assert abs(f["diffs_sharded"][k] - v) <= 2e-2 * abs(v) + 1e-9
  assert results[0][model]["cached_sharded"] == results[1][model]["cached_sharded"]


def test_auto_parallel_size_is_the_world_size(results):
  for r in results:
    assert r["config"] == dict(ulysses_size=2, anything=True, backend="CACHE_DIT", exchange="nccl", order=1)
