"""Host-side pieces of bench.py that decide what a run checks: the committed hit masks and the workload tables."""
import json
import os

import bench


def test_committed_masks_are_well_formed():
  masks = json.load(open(bench.MASKS_PATH))
  for name, entry in masks.items():
    wl = bench.WORKLOADS[name]
    assert entry["steps_per_generation"] == wl.steps_per_generation
    steps = entry["cached_steps"]
    assert steps == sorted(set(steps)) and steps and steps[0] >= 8 and steps[-1] < wl.steps_per_generation  # 8 warm-up steps


def test_expected_hits_follow_the_generation_boundaries():
  flux = bench.WORKLOADS["flux"]
  one = bench.expected_hits(flux, 0, 28)
  assert bench.mask_string(one) == "0000000011011011010101000000"
  two = bench.expected_hits(flux, 0, 56)
  assert two == one + one  # the timed region runs on into the next generation, which starts with its own warm-up
  assert bench.expected_hits(flux, 20, 10) == one[20:28] + one[:2]
  assert bench.expected_hits(bench.WORKLOADS["wan"], 0, 4) is None or len(bench.expected_hits(bench.WORKLOADS["wan"], 0, 4)) == 4


def test_workload_tables_match_the_stated_shapes():
  flux, qwen, wan = (bench.WORKLOADS[k].cpu_shape() for k in ("flux", "qwen_image", "wan"))
  assert flux["computed"] == {"double": 19, "single": 38} and flux["cached"]["double"] == 8
  assert sum(m * k * n for m, k, n in flux["kinds"]["single"]) == 4608 * (3 * 3072 * 3072 + 3072 * 12288 + 15360 * 3072)
  assert qwen["computed"] == {"double": 60} and qwen["calls_per_step"] == 2 and not qwen["taylor"]
  assert wan["computed"] == {"block": 40} and wan["cached"] == {"block": 1} and wan["cache_tensor"] == (75600, 5120)
  # FLOPs of the FLUX step's linears: 59.5 TFLOP (the figure the reference's own benchmark tables imply)
  per_step = sum(cnt * sum(2 * m * k * n for m, k, n in flux["kinds"][kind]) for kind, cnt in flux["computed"].items())
  assert abs(per_step / 1e12 - 59.5) < 1.0


def test_traffic_file_is_what_the_bench_reads():
  cap = json.load(open(bench.TRAFFIC_PATH))
  assert cap["dram_bytes_read"] > 0 and cap["dram_bytes_write"] > 0 and "case" in cap
  assert os.path.exists(os.path.join(bench.ROOT, cap["source"]))
