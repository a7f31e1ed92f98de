"""Benchmark of the per-step DiT hot path: FLUX-shape 1024x1024 denoising steps per second.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (BASELINE config 3): random-init FLUX.1-dev-architecture DiT (19 double + 38 single stream
blocks, hidden 3072, 24 heads x 128), 4096 image + 512 text tokens, 28-step schedule, DBCache F8B0
rdt 0.08 + TaylorSeer order 1, FP8 w8a8 linears, bf16 activations.  A "step" is one denoising step
(one transformer call through `cache_dit_b200.enable_cache`); steps are taken from consecutive
28-step generations, each started with `refresh_context`.

For N > 1 (torchrun, one rank per GPU) the sequence is sharded by Ulysses context parallelism
(head / token exchange by stores into peer memory on one node): total work is fixed, so scaling is
"strong".  The block segments between the cache decisions replay as CUDA graphs unless --no-graphs.
Prints ONE JSON line on rank 0:
  value / e2e ........ steps/s with inputs resident in HBM / with per-step host<->device copies
  roofline ........... every FP8 product of the timed steps (CUDA events, eager repeat) against the
                       library's sustained FP8 rate measured in the same run
  roofline_cache_kernels, fp8_linear_sweep, cpu_baseline ... the other two parts of the metric
                       (cache-check HBM GB/s, FP8 linear TFLOP/s) and the host-core baseline

`--impl reference` times the CPU restatement of the same path (the numpy oracle under oracle/) on
the host cores, on a bounded sample of the step, and prints the same line with "impl": "reference".
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
  sys.path.insert(0, ROOT)

STEPS_PER_GENERATION = 28
METRIC = "flux_1024x1024_denoise_steps_per_s"
WORKLOAD = ("FLUX.1-dev-shape DiT (19 double + 38 single blocks, hidden 3072, 24x128 heads), 4096 image + "
            "512 text tokens, 28-step schedule, DBCache F8B0 rdt=0.08 + TaylorSeer O1, FP8 w8a8")
FP8_NOMINAL_TFLOPS = 4500.0


def load_measured_peaks():
  path = os.path.join(ROOT, "MEASURED_PEAKS.json")
  if os.path.exists(path):
    with open(path) as f:
      return json.load(f), "measured"
  return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


# ------------------------------------------------------------------------------------ clocks
class ClockSampler:
  """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

  QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
           "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
           "clocks_event_reasons.sw_power_cap")

  def __init__(self, index: int):
    self.index = index
    self.proc = None
    self.lines = []

  def start(self):
    try:
      self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                                    "--format=csv,noheader,nounits", "-lms", "100"], stdout=subprocess.PIPE,
                                   stderr=subprocess.DEVNULL, text=True)
      threading.Thread(target=self._pump, daemon=True).start()
    except Exception:
      self.proc = None

  def _pump(self):
    for line in self.proc.stdout:
      self.lines.append(line.strip())

  def stop(self) -> dict:
    if self.proc is None:
      return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
    self.proc.terminate()
    try:
      self.proc.wait(timeout=5)
    except Exception:
      pass
    sm, mx, reasons = [], [], set()
    names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
    for line in self.lines:
      parts = [p.strip() for p in line.split(",")]
      if len(parts) < 7:
        continue
      try:
        sm.append(float(parts[0]))
        mx.append(float(parts[1]))
      except ValueError:
        continue
      for name, flag in zip(names, parts[3:7]):
        if flag.lower().startswith("active"):
          reasons.add(name)
    sm.sort()
    return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
            "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------------------ our arm
def build_model(device, seed=0):
  import cache_dit_b200 as cd
  from cache_dit_b200.synthetic import FluxTransformer2DModel
  torch.manual_seed(seed)
  with torch.device(device):
    # calibrated stand-in: smooth time conditioning and small adaLN weights, so that consecutive
    # steps are as similar as they are for a trained model (hit pattern: two hits, one miss)
    model = FluxTransformer2DModel(time_scale=1.0, modulation_init_std=0.02).to(torch.bfloat16)
  model.eval().requires_grad_(False)
  return cd, model


def host_inputs():
  """One generation's inputs in pinned host memory (what a serving process would hold)."""
  from cache_dit_b200.synthetic import FluxTransformer2DModel
  inp = FluxTransformer2DModel.example_inputs(device="cpu")
  return {k: v.pin_memory() for k, v in inp.items()}


def sigmas(n):
  from cache_dit_b200.synthetic import DenoisePipeline
  return DenoisePipeline.sigmas(n)


class Stepper:
  """Runs denoising steps one at a time across generation boundaries."""

  def __init__(self, cd, model, dev_inputs):
    self.cd, self.model = cd, model
    self.inp = {k: v for k, v in dev_inputs.items() if k != "hidden_states"}
    self.x0 = dev_inputs["hidden_states"]
    self.sig = sigmas(STEPS_PER_GENERATION)
    self.i = STEPS_PER_GENERATION
    self.x = None
    self.masks = []

  def start_generation(self):
    if self.i < STEPS_PER_GENERATION and self.i > 0:
      pass
    self.cd.refresh_context(self.model, num_inference_steps=STEPS_PER_GENERATION)
    self.x = self.x0.clone()
    self.i = 0

  @torch.no_grad()
  def step(self, host=None, host_out=None):
    if self.i >= STEPS_PER_GENERATION:
      self.start_generation()
    kw = self.inp
    x = self.x
    if host is not None:  # end-to-end: this step's inputs come from pinned host memory
      x = host["latents"].to(x.device, non_blocking=True)
      kw = {k: v.to(x.device, non_blocking=True) for k, v in host["cond"].items()}
    t = torch.full((x.shape[0], ), float(self.sig[self.i]), device=x.device)
    v = self.model(hidden_states=x, timestep=t, **kw)
    self.x = (x.float() + float(self.sig[self.i + 1] - self.sig[self.i]) * v.float()).to(x.dtype)
    if host_out is not None:  # ... and its result goes back to the host
      host_out.copy_(self.x, non_blocking=True)
      torch.cuda.current_stream().synchronize()
      host["latents"].copy_(host_out)
    self.i += 1
    if self.i == STEPS_PER_GENERATION:
      self.masks.append(list(getattr(self.model, "_cached_steps", [])))


def timed(fn, steps, barrier):
  barrier()
  torch.cuda.synchronize()
  start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
  start.record()
  for _ in range(steps):
    fn()
  end.record()
  torch.cuda.synchronize()
  barrier()
  return start.elapsed_time(end)  # ms


def fp8_library_peak(device, sustained=True):
  """Dense FP8 throughput of the vendor library on this GPU (8192^3, per-tensor scales, best of 10):
  the measured denominator for the tensor-core roofline, next to the nominal 4.5 PFLOP/s."""
  try:
    n = 8192
    a = torch.randn(n, n, device=device).to(torch.float8_e4m3fn)
    b = torch.randn(n, n, device=device).to(torch.float8_e4m3fn).t()
    one = torch.ones((), device=device)
    best = float("inf")
    for i in range(13):
      s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      s.record()
      torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
      e.record()
      torch.cuda.synchronize()
      if i >= 3:
        best = min(best, s.elapsed_time(e))
    burst = 2.0 * n**3 / (best * 1e-3) / 1e12
    if not sustained:
      return burst, None
    # sustained: the same product back to back for ~2 s (power-capped clocks, like a GEMM inside a long step)
    reps, elapsed, done = 50, 0.0, 0
    while elapsed < 2000.0 and done < 5000:
      s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      s.record()
      for _ in range(reps):
        torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
      e.record()
      torch.cuda.synchronize()
      last = s.elapsed_time(e)
      elapsed += last
      done += reps
    sustained = 2.0 * n**3 * reps / (last * 1e-3) / 1e12  # the last chunk, after the clocks settled
    return burst, sustained
  except Exception:
    return None


def cache_kernel_rooflines(device, hbm_peak, S=4096, C=3072, nsets=8):
  """CUDA-graph timed launches of the three cache kernels on bf16 [1, S, C] tensors (default: the FLUX
  image stream); rotating buffer sets (>= 200 MB in total) so nothing is served from L2."""
  from cache_dit_b200 import _native as nat
  n = S * C
  sets = [dict(h=torch.randn(1, S, C, device=device).bfloat16(), h0=torch.randn(1, S, C, device=device).bfloat16(),
               p=torch.randn(1, S, C, device=device).bfloat16(), d=torch.randn(1, S, C, device=device).bfloat16(),
               o=torch.empty(1, S, C, device=device, dtype=torch.bfloat16),
               o2=torch.empty(1, S, C, device=device, dtype=torch.bfloat16)) for _ in range(nsets)]
  means = torch.zeros(2, device=device)
  kernels = {
    "rel_l1_check": (lambda s: nat.rel_l1(s["h"], None, s["p"], None, means), 2 * n * 2),
    "rel_l1_check_fused_residual": (lambda s: nat.rel_l1(s["h"], s["h0"], s["p"], s["o"], means), 4 * n * 2),
    "taylor_apply_o1": (lambda s: nat.taylor_apply(s["h"], [s["p"], s["d"]], [1.0, 1.0], [1.0, 2.0], True, s["o"]),
                        4 * n * 2),
    "taylor_update_o1": (lambda s: nat.taylor_update(s["h"], s["h0"], [s["p"]], [s["o"], s["o2"]], 1, 3.0),
                         5 * n * 2),
  }
  out = {}
  for name, (fn, nbytes) in kernels.items():
    for s in sets:
      fn(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
      for s in sets:
        fn(s)
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(7):
      a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
      a.record()
      g.replay()
      b.record()
      torch.cuda.synchronize()
      ts.append(a.elapsed_time(b) / len(sets))
    ts.sort()
    ms = ts[len(ts) // 2]
    gbs = nbytes / (ms * 1e-3) / 1e9
    out[name] = {"us": round(ms * 1e3, 2), "achieved": round(gbs, 1), "peak": hbm_peak, "unit": "GB/s",
                 "frac": round(gbs / hbm_peak, 3), "algorithmic_bytes": nbytes}
  return out


def _graph_us(fn, n=4, reps=5):
  """Median time of one call of fn, from a CUDA graph of n back-to-back calls."""
  for _ in range(2):
    fn()
  torch.cuda.synchronize()
  g = torch.cuda.CUDAGraph()
  with torch.cuda.graph(g):
    for _ in range(n):
      fn()
  g.replay()
  torch.cuda.synchronize()
  ts = []
  for _ in range(reps):
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    g.replay()
    b.record()
    torch.cuda.synchronize()
    ts.append(a.elapsed_time(b) / n)
  ts.sort()
  return ts[len(ts) // 2] * 1e3


def fp8_linear_sweep(device):
  """The FP8 w8a8 per-token linear on the sweep shapes (activations N(0,1) with 0.1 % outliers x20,
  weights N(0, 0.02) quantized per output row): TFLOP/s of the whole linear (activation quantization
  + GEMM), of the GEMM alone without and with a bias, and of the library's row-wise `torch._scaled_mm` on the
  same operands."""
  from cache_dit_b200 import _native as nat
  out = {}
  g = torch.Generator(device=device).manual_seed(0)
  for M in (4608, 16384):
    for K, N in ((3072, 3072), (3072, 12288), (12288, 3072), (5120, 13824)):
      x = torch.randn(M, K, device=device, generator=g)
      x = torch.where(torch.rand(M, K, device=device, generator=g) < 1e-3, x * 20.0, x).to(torch.bfloat16)
      w = (0.02 * torch.randn(N, K, device=device, generator=g)).to(torch.bfloat16)
      wq = torch.empty(N, K, device=device, dtype=torch.float8_e4m3fn)
      sw = torch.empty(N, device=device)
      nat.fp8_quant_rows(w, wq, sw)
      aq = torch.empty(M, K, device=device, dtype=torch.float8_e4m3fn)
      sa = torch.empty(M, device=device)
      y = torch.empty(M, N, device=device, dtype=torch.bfloat16)

      def linear():
        nat.fp8_quant_rows(x, aq, sa)
        nat.fp8_gemm_rowscaled(aq, sa, wq, sw, None, y)

      flops = 2.0 * M * N * K
      t_lin = _graph_us(linear)
      t_gemm = _graph_us(lambda: nat.fp8_gemm_rowscaled(aq, sa, wq, sw, None, y))
      bias = (0.1 * torch.randn(N, device=device, generator=g)).to(torch.bfloat16)
      t_bias = _graph_us(lambda: nat.fp8_gemm_rowscaled(aq, sa, wq, sw, bias, y))
      entry = {"linear_tflops": round(flops / t_lin / 1e6, 1), "gemm_tflops": round(flops / t_gemm / 1e6, 1),
               "gemm_with_bias_tflops": round(flops / t_bias / 1e6, 1)}
      try:
        sa2, sw2 = sa.view(M, 1), sw.view(1, N)
        t_lib = _graph_us(lambda: torch._scaled_mm(aq, wq.t(), scale_a=sa2, scale_b=sw2, out_dtype=torch.bfloat16))
        entry["library_scaled_mm_rowwise_tflops"] = round(flops / t_lib / 1e6, 1)
      except Exception:
        entry["library_scaled_mm_rowwise_tflops"] = None
      out[f"M{M}_K{K}_N{N}"] = entry
      del x, w, wq, aq, y
  return out


def eager_cache_ops_us(device, S=4096, C=3072):
  """The reference's eager PyTorch op sequences for the same four steps on the GPU (the kernels to
  beat): similarity = sub, abs, mean, abs, mean (src/cache_dit/caching/cache_contexts/cache_manager.py:609-619);
  Taylor approximate + add (calibrators/taylorseer.py:91-104, cache_manager.py:831); update (taylorseer.py:68-89)."""
  mk = lambda: torch.randn(1, S, C, device=device).bfloat16()
  h, h0, p, d = mk(), mk(), mk(), mk()

  def check():
    return ((p - h).abs().mean() / p.abs().mean())

  def check_fused():
    r = h - h0
    return ((p - r).abs().mean() / p.abs().mean())

  def apply():
    out = torch.zeros_like(p)
    out = out + (1.0 / 1.0) * p * (1.0**0)
    out = out + (1.0 / 1.0) * d * (2.0**1)
    return h + out

  def update():
    y = h - h0
    return y, (y - p) / 3.0

  return {"rel_l1_check": round(_graph_us(check), 2), "rel_l1_check_fused_residual": round(_graph_us(check_fused), 2),
          "taylor_apply_o1": round(_graph_us(apply), 2), "taylor_update_o1": round(_graph_us(update), 2)}


def run_ours(args):
  import torch.distributed as dist
  world = int(os.environ.get("WORLD_SIZE", "1"))
  rank = int(os.environ.get("RANK", "0"))
  local_rank = int(os.environ.get("LOCAL_RANK", "0"))
  if world != args.gpus:
    if world == 1 and args.gpus > 1:
      raise SystemExit("launch with torchrun --nproc-per-node N for --gpus N > 1")
  torch.cuda.set_device(local_rank)
  device = torch.device("cuda", local_rank)
  if world > 1:
    dist.init_process_group("nccl", device_id=device)
  barrier = (lambda: dist.barrier()) if world > 1 else (lambda: None)

  from cache_dit_b200 import _native as nat
  nat.lib()
  cd, model = build_model(device)
  cd.enable_cache(model,
                  cache_config=cd.DBCacheConfig(Fn_compute_blocks=8, Bn_compute_blocks=0, residual_diff_threshold=0.08,
                                                max_warmup_steps=8, num_inference_steps=STEPS_PER_GENERATION,
                                                enable_separate_cfg=False),
                  calibrator_config=cd.TaylorSeerCalibratorConfig(taylorseer_order=1),
                  parallelism_config=cd.ParallelismConfig(ulysses_size=world) if world > 1 else None,
                  quantize_config=cd.QuantizeConfig(quant_type="float8_per_row"))
  if not args.no_graphs:
    cd.enable_cuda_graphs(model)  # block segments between the cache decisions replay as CUDA graphs
  host = host_inputs()
  dev_inputs = {k: v.to(device) for k, v in host.items()}
  stepper = Stepper(cd, model, dev_inputs)

  warmup = max(3, args.warmup)
  for _ in range(warmup):
    stepper.step()
  torch.cuda.synchronize()
  # -------- timed region 1: inputs resident in HBM
  stepper.i = STEPS_PER_GENERATION  # start the timed region at a generation boundary
  stepper.masks.clear()
  sampler = ClockSampler(local_rank)
  if rank == 0:
    sampler.start()
  launches0 = nat.launch_count
  if args.profile_timed_region:
    torch.cuda.profiler.start()
  ms = timed(stepper.step, args.steps, barrier)
  if args.profile_timed_region:
    torch.cuda.profiler.stop()
  launches = nat.launch_count - launches0
  clocks = sampler.stop() if rank == 0 else {}
  masks = [list(m) for m in stepper.masks]
  # -------- timed region 2: end to end with host buffers
  host_state = {"latents": host["hidden_states"].clone().pin_memory(),
                "cond": {k: v for k, v in host.items() if k != "hidden_states"}}
  host_out = torch.empty_like(host_state["latents"]).pin_memory()
  stepper.i = STEPS_PER_GENERATION
  for _ in range(3):
    stepper.step(host_state, host_out)
  stepper.i = STEPS_PER_GENERATION
  host_state["latents"].copy_(host["hidden_states"])
  ms_e2e = timed(lambda: stepper.step(host_state, host_out), args.steps, barrier)
  h2d = sum(v.numel() * v.element_size() for v in host.values())
  d2h = host_out.numel() * host_out.element_size()
  # -------- instrumented repeat of region 1: per-launch durations of the dominant kernel (FP8 GEMM)
  # (eager launches: events cannot bracket single kernels inside a graph replay)
  runners = cd.graph_runners(model)
  for r in runners:
    r.enabled = False
  stepper.i = STEPS_PER_GENERATION
  nat.gemm_timer = []
  instrumented_steps = min(args.steps, STEPS_PER_GENERATION)
  for _ in range(instrumented_steps):
    stepper.step()
  torch.cuda.synchronize()
  records, nat.gemm_timer = nat.gemm_timer, None
  for r in runners:
    r.enabled = True
  gemm_ms = sum(s.elapsed_time(e) for s, e, _ in records)
  gemm_flops = sum(f for _, _, f in records)

  times = torch.tensor([ms, ms_e2e], device=device, dtype=torch.float64)
  if world > 1:
    dist.all_reduce(times, op=dist.ReduceOp.MAX)
  ms, ms_e2e = float(times[0]), float(times[1])
  if rank != 0:
    if world > 1:
      dist.destroy_process_group()
    return
  peaks, peak_kind = load_measured_peaks()
  cache_roof = None
  fp8_burst = fp8_library_peak(device, sustained=False) if not args.skip_extras else None
  if not args.skip_extras:  # before the 2-second GEMM loop below heats the part
    cache_roof = {"flux_image_stream_1x4096x3072": cache_kernel_rooflines(device, peaks["hbm_gbs"]),
                  "wan_rank_shard_1x9450x5120": cache_kernel_rooflines(device, peaks["hbm_gbs"], 9450, 5120, 3),
                  "eager_torch_ops_us_1x4096x3072": eager_cache_ops_us(device)}
    sweep = fp8_linear_sweep(device)
  fp8_lib = fp8_library_peak(device) if not args.skip_extras else None
  if fp8_lib and fp8_burst:
    fp8_lib = (max(fp8_lib[0], fp8_burst[0]), fp8_lib[1])
  achieved = gemm_flops / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else 0.0
  # the GEMM launches are timed inside long steps under the power cap: the sustained library figure
  # is the like-for-like denominator, the burst figure is reported beside it
  peak = fp8_lib[1] if fp8_lib else FP8_NOMINAL_TFLOPS
  line = {
    "metric": METRIC, "value": args.steps / (ms * 1e-3), "unit": "steps/s", "n_gpus": world, "steps": args.steps,
    "warmup": warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "strong",
    "vs_baseline": None, "dtype": "bf16 activations, fp8 e4m3 linears (fp32 accumulate)", "data": "synthetic",
    "config": {"workload": WORKLOAD, "parallelism": f"ulysses{world}" if world > 1 else "single",
               "l2_policy": "inputs larger than L2: ~12 GB of FP8 weights streamed per computed step",
               "cuda_graphs": (not args.no_graphs), "cached_steps_per_generation": masks[:2]},
    "e2e": {"value": args.steps / (ms_e2e * 1e-3), "unit": "steps/s", "h2d_bytes_per_step": h2d,
            "d2h_bytes_per_step": d2h},
    "gpu_launches": launches, "clocks": clocks,
    "roofline": {"bound": "tensor", "kernel": "fp8_gemm_rowscaled_pair_kernel + fp8_gemm_rowscaled_kernel + fp8_gemv_rowscaled_kernel (every cdb_fp8_gemm_rowscaled launch of the step)", "achieved": round(achieved, 1),
                 "peak": round(peak, 1), "unit": "TFLOP/s", "frac": round(achieved / peak, 3),
                 "peak_source": "torch._scaled_mm e4m3 8192^3 per-tensor back to back for 2 s (sustained), "
                 "measured in this run" if fp8_lib else "nominal dense FP8",
                 "peak_burst": round(fp8_lib[0], 1) if fp8_lib else None,
                 "frac_of_burst": round(achieved / fp8_lib[0], 3) if fp8_lib else None,
                 "frac_of_nominal_4500": round(achieved / FP8_NOMINAL_TFLOPS, 3), "launches": len(records),
                 "avg_launch_us": round(1e3 * gemm_ms / max(len(records), 1), 2),
                 # time inside these launches per step / the timed region's time per step (compare with the
                 # kernel's share in the committed ncu launch list)
                 "share_of_step": round((gemm_ms / max(instrumented_steps, 1)) / (ms / args.steps), 3),
                 "timing": "CUDA events around every GEMM launch in an instrumented repeat of the timed steps",
                 # dram__bytes_read + dram__bytes_write of one launch of the dominant shape class from the
                 # committed ncu capture (profiles/kernels_small_case_ncu_set_full.md): 52.1 MB + 67.9 MB for
                 # 165.1 MB of operands and output (part of the output is still in L2 when the kernel ends)
                 "traffic": 120.0e6, "traffic_case": "ncu, pair kernel, M=4608 N=12288 K=3072 (a single-stream MLP-in product)"},
  }
  if not args.skip_extras:
    line["roofline_cache_kernels"] = cache_roof
    line["fp8_linear_sweep"] = sweep
    line["roofline_cache_kernels"]["peak_source"] = f"{peak_kind} copy bandwidth (1 Gi-element copy)"
    line["cpu_baseline"] = cpu_baseline(sample_only=True, hits=len(masks[0]) if masks else None)
  if world > 1:
    dist.destroy_process_group()
  print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------ CPU arm
def cpu_baseline(sample_only=False, hits=None):
  """The reference's path restated on the CPU (numpy oracle), timed on this host's cores.

  Sample: the cache ops of one step at full size (bf16 [1, 4608, 3072]: check, TaylorSeer update,
  TaylorSeer apply) and the FP8 linears of ONE double-stream and ONE single-stream block at 4608
  tokens (dynamic per-token quantization + dequantized fp32 product).  A computed step is then
  19 double + 38 single blocks, a cached step is the first 8 double blocks + apply; attention (a
  library call on both sides) is left out of the CPU figure, which flatters the CPU."""
  import numpy as np
  from oracle import cache_oracle as O
  from oracle import fp8_oracle as F
  cores = os.cpu_count() or 1
  torch.set_num_threads(cores)
  # the launcher of multi-rank runs exports OMP_NUM_THREADS=1, which the BLAS under numpy reads at import:
  # lift its pool back to all host cores for this arm, and report the threads it really has
  try:
    from threadpoolctl import threadpool_info, threadpool_limits
    threadpool_limits(limits=cores)
    blas = [p["num_threads"] for p in threadpool_info() if p.get("user_api") == "blas"]
    cores = max(blas) if blas else cores
  except ImportError:
    cores = int(os.environ.get("OMP_NUM_THREADS", cores))
  rng = np.random.RandomState(0)
  S, C = 4608, 3072
  prev = O.round_bf16(rng.randn(1, S, C).astype(np.float32))
  cur = O.round_bf16(prev + 0.05 * rng.randn(1, S, C).astype(np.float32))
  t0 = time.perf_counter()
  O.rel_l1(prev, cur, "bf16")
  t_check = time.perf_counter() - t0
  t0 = time.perf_counter()
  ladder = O.taylor_derivatives(O.residual(cur, prev, "bf16"), [prev, None], 3, True, "bf16")
  t_update = time.perf_counter() - t0
  t0 = time.perf_counter()
  O.apply_add(O.taylor_series(ladder, 2, "bf16"), cur, "bf16")
  t_apply = time.perf_counter() - t0

  def linear(m, k, n):
    x = O.round_bf16(rng.randn(m, k).astype(np.float32))
    w = O.round_bf16((0.02 * rng.randn(n, k)).astype(np.float32))
    wc, ws = F.quantize_rows(w)  # weights are quantized once at load: not timed
    t = time.perf_counter()
    ac, asc = F.quantize_rows(x)
    F.scaled_mm(ac, asc, wc, ws)
    return time.perf_counter() - t

  # double block: image (4096 tokens) and text (512) streams, each q,k,v,out (3072x3072) + MLP 3072<->12288
  t_double = 0.0
  for m in (4096, 512):
    t_double += 4 * linear(m, 3072, 3072) + linear(m, 3072, 12288) + linear(m, 12288, 3072)
  # single block: q,k,v + MLP-in on 4608 tokens, then 15360 -> 3072
  t_single = 3 * linear(4608, 3072, 3072) + linear(4608, 3072, 12288) + linear(4608, 15360, 3072)
  computed = 19 * t_double + 38 * t_single
  cached = 8 * t_double
  if hits is None:
    hits = 14  # hit count of the reference's synthetic cache-step schedule (2 hits, 1 miss after warm-up)
  per_generation = (STEPS_PER_GENERATION - hits) * (computed + t_update) + hits * (cached + t_apply) \
      + (STEPS_PER_GENERATION - 8) * t_check
  return {"value": STEPS_PER_GENERATION / per_generation, "unit": "steps/s", "cores": cores,
          "kind": "port",
          "sample": ("numpy restatement: cache check/update/apply at [1,4608,3072] bf16 + FP8 linears of one "
                     "double and one single block, extrapolated to 19+38 blocks and a 28-step schedule with the "
                     f"GPU run's hit count ({hits}); attention excluded"),
          "seconds": {"check": t_check, "update": t_update, "apply": t_apply, "double_block_linears": t_double,
                      "single_block_linears": t_single}}


def run_reference(args):
  rank = int(os.environ.get("RANK", "0"))
  if rank != 0:
    return
  base = cpu_baseline()
  line = {
    "impl": "reference", "metric": METRIC, "value": base["value"], "unit": "steps/s", "n_gpus": args.gpus,
    "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 / base["value"], "higher_is_better": True,
    "scaling": "strong", "vs_baseline": None, "dtype": "fp32 arithmetic on e4m3 / bf16 values", "data": "synthetic",
    "config": {"workload": WORKLOAD, "parallelism": "host cores"},
    "cpu_baseline": base,
    "e2e": {"value": base["value"], "unit": "steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    "gpu_launches": 0,
  }
  print(json.dumps(line), flush=True)


def main():
  ap = argparse.ArgumentParser()
  ap.add_argument("--gpus", type=int, default=1)
  ap.add_argument("--steps", type=int, default=2 * STEPS_PER_GENERATION)
  ap.add_argument("--warmup", type=int, default=STEPS_PER_GENERATION)
  ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
  ap.add_argument("--no-graphs", action="store_true", help="issue every kernel from Python instead of replaying CUDA graphs")
  ap.add_argument("--profile-timed-region", action="store_true",
                  help="bracket the first timed region with cudaProfilerStart/Stop (for ncu --profile-from-start off)")
  ap.add_argument("--skip-extras", action="store_true",
                  help="leave out the cache-kernel microbenchmarks, the FP8 library peak and the CPU sample")
  args = ap.parse_args()
  if args.impl == "reference":
    run_reference(args)
  else:
    run_ours(args)


if __name__ == "__main__":
  main()
