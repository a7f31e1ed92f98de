"""Two GPUs: the peer-memory Ulysses exchange against the NCCL all-to-all path, eager and under CUDA
graphs (child processes, one per GPU; skipped on a single-GPU machine)."""
import json
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def reports(tmp_path_factory):
  if torch.cuda.device_count() < 2:
    pytest.skip("needs two GPUs")
  out = tmp_path_factory.mktemp("peer")
  cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr",
         "127.0.0.1", "--master-port", "29641", os.path.join(HERE, "peer_worker.py"), str(out)]
  env = dict(os.environ, NCCL_NVLS_ENABLE="0", OMP_NUM_THREADS="2")
  proc = subprocess.run(cmd, env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=600)
  assert proc.returncode == 0, proc.stdout[-3000:]
  return [json.load(open(os.path.join(out, f"rank{r}.json"))) for r in range(2)]


def test_peer_exchange_equals_all_to_all(reports):
  for r in reports:
    assert r["finite"] and r["status_peer"] == 0
    assert r["masks_peer"] == r["masks_nccl"] and r["masks_peer"][0]
    assert r["peer_equals_nccl"]
  assert reports[0]["masks_peer"] == reports[1]["masks_peer"]


def test_peer_exchange_under_cuda_graphs(reports):
  for r in reports:
    assert r["status_graphs"] == 0 and r["replays"] > 0
    assert r["masks_graphs"] == r["masks_peer"]
    assert r["graphs_equal_peer"]


@pytest.mark.parametrize("model", ["qwen", "wan"])
def test_other_models_peer_exchange(reports, model):
  """Qwen-Image-shape with uneven token shards and Wan-shape (row-norm q / k, local cross-attention)."""
  for r in reports:
    o = r["others"][model]
    assert o["finite"] and o["status"] == [0, 0]
    assert o["masks"][0] == o["masks"][1] == o["masks"][2] and o["masks"][0]
    assert o["peer_equals_nccl"] and o["graphs_equal_peer"]
  assert reports[0]["others"][model]["masks"] == reports[1]["others"][model]["masks"]


def test_fp8_on_the_wire(reports):
  """`ulysses_float8`: e4m3 + per-(token, head) scales cross NVLink; lossy, so close to, not equal to, bf16."""
  for r in reports:
    f = r["fp8_wire"]
    assert f["finite"] and f["status"] == 0
    assert f["rel"] < 0.1, f["rel"]
  assert reports[0]["fp8_wire"]["masks"] == reports[1]["fp8_wire"]["masks"]


def test_modulation_bank_equals_per_block_products(reports):
  """All blocks' adaLN modulation vectors as one column-sharded product + all-gather per call (FP8 members in the
  FLUX shape, bf16 members in the Qwen-Image shape) against one product per block and rank: same bits, same masks."""
  for r in reports:
    assert r["bank_equals_per_block"]
    assert r["qwen_bank_equals_per_block"]
