"""Seeded cache-step scenarios shared by the golden generator and the parity tests.

A scenario is a plain dict.  `trajectory(sc)` turns it into the per-call input tensors
(torch CPU generator, so every machine regenerates identical values); `drive(sc, backend)`
feeds them through a backend with the calling order the reference's block runner uses
(src/cache_dit/caching/cache_blocks/pattern_base.py:198-321) and returns a trace.

Backends (reference manager, numpy oracle, CUDA engine) implement:
  begin_call(), mark_step_begin(), can_cache(r) -> bool, add_cached_step(),
  apply_cache(h, e) -> (h, e), set_Fn_buffer(r), set_Bn_buffer(R), set_Bn_encoder_buffer(Re),
  current_step() -> int, stats() -> dict, to_numpy(t) -> float32 ndarray, from_torch(t) -> backend tensor
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch

TORCH_DTYPE = {"fp32": torch.float32, "bf16": torch.bfloat16, "fp16": torch.float16}

# name -> scenario.  "noise" is the relative step size of the Fn-residual random walk.
SCENARIOS: List[dict] = [
  # BASELINE config 1 at full size: fp32 [1, 4608, 3072], 28 steps, warmup 8, rdt 0.08, order 1.
  dict(name="config1_fp32_full", shape=(1, 4608, 3072), enc_shape=None, dtype="fp32", steps=28,
       seed=0, noise=0.05, cache_config=dict(num_inference_steps=28),
       calibrator_config=dict(taylorseer_order=1), full_outputs=False),
  # Same walk in bf16 on the FLUX image + text stream shapes, sharded sizes included.
  dict(name="flux_bf16_full", shape=(1, 4096, 3072), enc_shape=(1, 512, 3072), dtype="bf16",
       steps=28, seed=1, noise=0.05, cache_config=dict(num_inference_steps=28),
       calibrator_config=dict(taylorseer_order=1), full_outputs=False),
  # Small ragged shapes (token and channel counts not multiples of any vector width).
  dict(name="small_bf16_o1", shape=(1, 37, 72), enc_shape=(1, 5, 72), dtype="bf16", steps=20,
       seed=2, noise=0.04, cache_config=dict(max_warmup_steps=3),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  dict(name="small_fp32_o2", shape=(2, 19, 50), enc_shape=(2, 3, 50), dtype="fp32", steps=24,
       seed=3, noise=0.03, cache_config=dict(max_warmup_steps=4),
       calibrator_config=dict(taylorseer_order=2), full_outputs=True),
  dict(name="small_fp16_o3", shape=(1, 33, 40), enc_shape=None, dtype="fp16", steps=24, seed=4,
       noise=0.02, cache_config=dict(max_warmup_steps=4),
       calibrator_config=dict(taylorseer_order=3), full_outputs=True),
  dict(name="odd_bf16_o2", shape=(1, 7, 13), enc_shape=(1, 1, 13), dtype="bf16", steps=18,
       seed=5, noise=0.03, cache_config=dict(max_warmup_steps=2),
       calibrator_config=dict(taylorseer_order=2), full_outputs=True),
  # No calibrator: the Bn residual is a plain buffer.
  dict(name="plain_buffer_bf16", shape=(1, 37, 72), enc_shape=(1, 5, 72), dtype="bf16", steps=16,
       seed=6, noise=0.04, cache_config=dict(max_warmup_steps=2), calibrator_config=None,
       full_outputs=True),
  # Calibrator on the hidden stream only.
  dict(name="no_encoder_calibrator", shape=(1, 21, 64), enc_shape=(1, 4, 64), dtype="bf16",
       steps=16, seed=7, noise=0.04, cache_config=dict(max_warmup_steps=2),
       calibrator_config=dict(taylorseer_order=1, enable_encoder_calibrator=False),
       full_outputs=True),
  # Hidden-state (not residual) cache type.
  dict(name="cache_hidden_states", shape=(1, 21, 64), enc_shape=(1, 4, 64), dtype="bf16",
       steps=16, seed=8, noise=0.04, cache_config=dict(max_warmup_steps=2),
       calibrator_config=dict(taylorseer_order=1, calibrator_cache_type="hidden_states"),
       full_outputs=True),
  # Host gates.
  dict(name="gate_max_cached", shape=(1, 16, 32), enc_shape=None, dtype="fp32", steps=20, seed=9,
       noise=0.02, cache_config=dict(max_warmup_steps=2, max_cached_steps=5),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  dict(name="gate_max_continuous", shape=(1, 16, 32), enc_shape=None, dtype="fp32", steps=24,
       seed=10, noise=0.01, cache_config=dict(max_warmup_steps=2, max_continuous_cached_steps=3),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  dict(name="gate_accumulated", shape=(1, 16, 32), enc_shape=None, dtype="fp32", steps=24,
       seed=11, noise=0.02,
       cache_config=dict(max_warmup_steps=2, max_accumulated_residual_diff_threshold=0.3),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  dict(name="gate_warmup_interval", shape=(1, 16, 32), enc_shape=None, dtype="fp32", steps=20,
       seed=12, noise=0.02, cache_config=dict(max_warmup_steps=8, warmup_interval=2),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  dict(name="scm_dynamic", shape=(1, 16, 32), enc_shape=None, dtype="fp32", steps=16, seed=13,
       noise=0.05,
       cache_config=dict(max_warmup_steps=4, num_inference_steps=16,
                         steps_computation_mask=[1, 1, 1, 0, 0, 1, 0, 0, 0, 1, 0, 0, 0, 0, 1, 0],
                         steps_computation_policy="dynamic"),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  dict(name="scm_static", shape=(1, 16, 32), enc_shape=None, dtype="fp32", steps=16, seed=14,
       noise=0.5,
       cache_config=dict(max_warmup_steps=4, num_inference_steps=16,
                         steps_computation_mask=[1, 1, 1, 0, 0, 1, 0, 0, 0, 1, 0, 0, 0, 0, 1, 0],
                         steps_computation_policy="static"),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  dict(name="threshold_always", shape=(1, 8, 16), enc_shape=None, dtype="fp32", steps=10, seed=15,
       noise=0.5, cache_config=dict(max_warmup_steps=2, residual_diff_threshold=1.0),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  dict(name="threshold_never", shape=(1, 8, 16), enc_shape=None, dtype="fp32", steps=10, seed=16,
       noise=0.001, cache_config=dict(max_warmup_steps=2, residual_diff_threshold=0.0),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  # Separate classifier-free-guidance branch: two transformer calls per step.
  dict(name="separate_cfg", shape=(1, 16, 32), enc_shape=(1, 3, 32), dtype="bf16", steps=14,
       seed=17, noise=0.03, cache_config=dict(max_warmup_steps=2, enable_separate_cfg=True),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  dict(name="separate_cfg_shared_diff", shape=(1, 16, 32), enc_shape=None, dtype="fp32", steps=14,
       seed=18, noise=0.03,
       cache_config=dict(max_warmup_steps=2, enable_separate_cfg=True,
                         cfg_diff_compute_separate=False),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  # Persistent context driven for two and a half runs: the refresh comes one call late.
  dict(name="persistent_refresh", shape=(1, 16, 32), enc_shape=None, dtype="fp32", steps=22,
       seed=19, noise=0.03, cache_config=dict(max_warmup_steps=2, num_inference_steps=8),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  dict(name="force_refresh_hint", shape=(1, 16, 32), enc_shape=None, dtype="fp32", steps=20,
       seed=20, noise=0.03, cache_config=dict(max_warmup_steps=2, force_refresh_step_hint=10),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  dict(name="force_refresh_repeat", shape=(1, 16, 32), enc_shape=None, dtype="fp32", steps=24,
       seed=21, noise=0.03,
       cache_config=dict(max_warmup_steps=2, force_refresh_step_hint=7, force_refresh_step_policy="repeat"),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  dict(name="separate_cfg_first", shape=(1, 16, 32), enc_shape=(1, 3, 32), dtype="fp32", steps=14,
       seed=22, noise=0.03,
       cache_config=dict(max_warmup_steps=2, enable_separate_cfg=True, cfg_compute_first=True,
                         cfg_diff_compute_separate=False),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  # The highest order the kernels take.
  dict(name="small_bf16_o4", shape=(1, 21, 64), enc_shape=(1, 4, 64), dtype="bf16", steps=26, seed=23,
       noise=0.02, cache_config=dict(max_warmup_steps=6), calibrator_config=dict(taylorseer_order=4),
       full_outputs=True),
  # Extra options of the similarity check (off by default): channel sub-sampling of the indicator and
  # the token-selective distance.
  dict(name="extra_downsample", shape=(1, 16, 32), enc_shape=None, dtype="fp32", steps=20, seed=24,
       noise=0.03, cache_config=dict(max_warmup_steps=2), extra_config=dict(downsample_factor=4),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  dict(name="extra_important_tokens", shape=(2, 16, 32), enc_shape=None, dtype="fp32", steps=20, seed=25,
       noise=0.03, cache_config=dict(max_warmup_steps=2, residual_diff_threshold=0.1),
       extra_config=dict(important_condition_threshold=0.06),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
  dict(name="extra_important_tokens_none_chosen", shape=(1, 16, 32), enc_shape=None, dtype="fp32", steps=12,
       seed=26, noise=0.01, cache_config=dict(max_warmup_steps=2),
       extra_config=dict(important_condition_threshold=0.9),
       calibrator_config=dict(taylorseer_order=1), full_outputs=True),
]

BY_NAME: Dict[str, dict] = {s["name"]: s for s in SCENARIOS}
SMALL = [s["name"] for s in SCENARIOS if s["full_outputs"]]
FULL = [s["name"] for s in SCENARIOS if not s["full_outputs"]]

# flat element indices sampled from large outputs (in addition to float64 sums)
N_SAMPLES = 64


def calls_per_step(sc: dict) -> int:
  return 2 if sc["cache_config"].get("enable_separate_cfg") else 1


def trajectory(sc: dict):
  """Yield dicts of torch CPU tensors in the storage dtype, one per transformer call.

  r  : Fn residual          (random walk, relative step `noise`)
  h  : hidden after Fn      (slow random walk)
  e  : encoder after Fn     (or None)
  R  : Mn residual payload  (a deterministic function of r)
  Re : encoder Mn residual  (or None)
  """
  dt = TORCH_DTYPE[sc["dtype"]]
  g = torch.Generator().manual_seed(sc["seed"])
  branches = calls_per_step(sc)
  shape, enc_shape = tuple(sc["shape"]), sc["enc_shape"]
  state = []
  for _ in range(branches):
    st = dict(r=torch.randn(shape, generator=g), h=torch.randn(shape, generator=g))
    st["e"] = torch.randn(tuple(enc_shape), generator=g) if enc_shape else None
    state.append(st)
  for step in range(sc["steps"]):
    for b in range(branches):
      st = state[b]
      if step > 0:
        st["r"] = st["r"] + sc["noise"] * torch.randn(shape, generator=g)
        st["h"] = st["h"] + 0.02 * torch.randn(shape, generator=g)
        if st["e"] is not None:
          st["e"] = st["e"] + 0.02 * torch.randn(tuple(enc_shape), generator=g)
      r = st["r"].to(dt)
      out = dict(r=r, h=st["h"].to(dt), R=(0.3 * st["r"] + 0.01 * step).to(dt), e=None, Re=None)
      if st["e"] is not None:
        out["e"] = st["e"].to(dt)
        out["Re"] = (0.1 * st["e"] - 0.02 * step).to(dt)
      yield out


def sample_index(numel: int) -> np.ndarray:
  rng = np.random.RandomState(1234)
  return np.sort(rng.randint(0, numel, size=min(N_SAMPLES, numel)))


def digest(a: np.ndarray) -> dict:
  """Size-independent summary of a large output: float64 sums plus fixed samples."""
  flat = np.asarray(a, dtype=np.float32).reshape(-1)
  return dict(sum=float(np.sum(flat, dtype=np.float64)),
              abs_sum=float(np.sum(np.abs(flat), dtype=np.float64)),
              samples=[float(v) for v in flat[sample_index(flat.size)]])


def drive(sc: dict, backend, keep_outputs: Optional[bool] = None) -> dict:
  """Run a scenario through a backend; return the trace the golden files store."""
  keep = sc["full_outputs"] if keep_outputs is None else keep_outputs
  hits: List[int] = []
  step_index: List[int] = []
  outputs: Dict[str, np.ndarray] = {}
  digests: Dict[str, dict] = {}
  for call, t in enumerate(trajectory(sc)):
    backend.begin_call()
    backend.mark_step_begin()
    step_index.append(int(backend.current_step()))
    r = backend.from_torch(t["r"])
    hit = bool(backend.can_cache(r))
    hits.append(int(hit))
    if hit:
      backend.add_cached_step()
      h, e = backend.apply_cache(backend.from_torch(t["h"]),
                                 None if t["e"] is None else backend.from_torch(t["e"]))
      items = [("h", h)] + ([("e", e)] if e is not None else [])
      for tag, val in items:
        arr = backend.to_numpy(val)
        if keep:
          outputs[f"{tag}{call}"] = arr
        else:
          digests[f"{tag}{call}"] = digest(arr)
    else:
      backend.set_Fn_buffer(r)
      backend.set_Bn_buffer(backend.from_torch(t["R"]))
      if t["Re"] is not None:
        backend.set_Bn_encoder_buffer(backend.from_torch(t["Re"]))
  trace = dict(name=sc["name"], hits=hits, step_index=step_index, stats=backend.stats(), digests=digests)
  return dict(trace=trace, outputs=outputs)
