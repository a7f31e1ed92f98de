"""Worker for the 2-GPU test of the peer-memory Ulysses exchange (launched by tests/test_gpu_multi.py).

One small FLUX-shape generation per configuration, each rank writing what it saw:
  nccl   - heads exchanged with all-to-all collectives, kernels launched from Python
  peer   - heads exchanged by the scatter / gather kernels over peer memory
  graphs - peer exchange, block segments replayed as CUDA graphs
The three must give the same cached steps and the same latents bit for bit."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import cache_dit_b200 as cd  # noqa: E402


def generation(world, exchange, graphs, steps=10, fp8_wire=False):
  from cache_dit_b200.synthetic import FluxTransformer2DModel
  torch.manual_seed(0)
  with torch.device("cuda"):
    model = FluxTransformer2DModel(num_layers=2, num_single_layers=3, dim=256, heads=4, in_channels=16,
                                   joint_attention_dim=64, pooled_projection_dim=32, axes_dims_rope=(8, 28, 28),
                                   time_scale=1.0, modulation_init_std=0.02).to(torch.bfloat16)
  model.eval().requires_grad_(False)
  cd.enable_cache(model,
                  cache_config=cd.DBCacheConfig(Fn_compute_blocks=2, Bn_compute_blocks=0, residual_diff_threshold=0.13,
                                                max_warmup_steps=3, num_inference_steps=steps),
                  calibrator_config=cd.TaylorSeerCalibratorConfig(taylorseer_order=1),
                  parallelism_config=cd.ParallelismConfig(ulysses_size=world, ulysses_float8=fp8_wire,
                                                          parallel_kwargs={"exchange": exchange}),
                  quantize_config=cd.QuantizeConfig(quant_type="float8_per_row"))
  if graphs:
    cd.enable_cuda_graphs(model, warmup_calls=1)
  inp = FluxTransformer2DModel.example_inputs(height=256, width=256, text_tokens=32, in_channels=16,
                                              joint_attention_dim=64, pooled_projection_dim=32)
  x = inp.pop("hidden_states")
  result = []
  with torch.no_grad():
    for gen in range(2):
      cd.refresh_context(model, num_inference_steps=steps)
      lat = x.clone()
      for i in range(steps):
        t = torch.full((1, ), 1.0 - i / steps, device="cuda")
        v = model(hidden_states=lat, timestep=t, **inp)
        lat = (lat.float() - v.float() / steps).to(lat.dtype)
      result.append((lat.clone(), list(model._cached_steps)))
  torch.cuda.synchronize()
  status = 0
  cp = getattr(model, "_cp", None)
  if cp is not None and cp.exchange is not None:
    status = cp.exchange.status()
  replays = sum(r.replays for r in cd.graph_runners(model))
  cd.disable_cache(model)
  return result, status, replays


def other_model(world, which, exchange, graphs, steps=8):
  """Qwen-Image-shape (289 image + 33 text tokens: uneven shards) or Wan-shape (105 video tokens, text whole)."""
  from cache_dit_b200.synthetic import (QwenImageDenoisePipeline, QwenImageTransformer2DModel, WanDenoisePipeline,
                                        WanTransformer3DModel)
  torch.manual_seed(0)
  if which == "qwen":
    with torch.device("cuda"):
      model = QwenImageTransformer2DModel(num_layers=4, dim=256, heads=4, in_channels=16, joint_attention_dim=64,
                                          axes_dims_rope=(8, 28, 28), time_scale=1.0, modulation_init_std=0.02)
    inputs = QwenImageTransformer2DModel.example_inputs(height=272, width=272, text_tokens=33, in_channels=16,
                                                        joint_attention_dim=64)
    pipe = QwenImageDenoisePipeline(model, inputs)
  else:
    with torch.device("cuda"):
      model = WanTransformer3DModel(num_layers=3, dim=256, heads=2, ffn_dim=512, in_channels=16, text_dim=64,
                                    axes_dims_rope=(44, 42, 42), time_scale=1.0, modulation_init_std=0.02)
    inputs = WanTransformer3DModel.example_inputs(frames=3, height=5, width=7, text_tokens=16, in_channels=16,
                                                  text_dim=64)
    pipe = WanDenoisePipeline(model, inputs)
  model.to(torch.bfloat16).eval().requires_grad_(False)
  cd.enable_cache(pipe, cache_config=cd.DBCacheConfig(Fn_compute_blocks=1, max_warmup_steps=3, residual_diff_threshold=0.15),
                  calibrator_config=cd.TaylorSeerCalibratorConfig(taylorseer_order=1),
                  parallelism_config=cd.ParallelismConfig(ulysses_size=world, parallel_kwargs={"exchange": exchange}),
                  quantize_config=cd.QuantizeConfig(quant_type="float8_per_row"))
  if graphs:
    cd.enable_cuda_graphs(pipe, warmup_calls=1)
  out = pipe(num_inference_steps=steps)
  if graphs:
    out = pipe(num_inference_steps=steps)
  stats = cd.summary(pipe, logging=False)[-1]
  torch.cuda.synchronize()
  cp = getattr(model, "_cp", None)
  status = cp.exchange.status() if cp is not None and cp.exchange is not None else 0
  cd.disable_cache(pipe)
  return out.clone(), list(stats.cached_steps), status


def main():
  out_dir = sys.argv[1]
  rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
  torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
  dist.init_process_group("nccl", device_id=torch.device("cuda", int(os.environ["LOCAL_RANK"])))
  nccl, _, _ = generation(world, "nccl", False)
  peer, st_peer, _ = generation(world, "peer", False)
  graphed, st_graph, replays = generation(world, "peer", True)
  wire8, st_wire8, _ = generation(world, "peer", True, fp8_wire=True)
  # the column-sharded modulation bank (on by default in everything above) against per-block modulation products
  os.environ["CACHE_DIT_B200_MODULATION_BANK"] = "0"
  no_bank, _, _ = generation(world, "peer", False)
  qwen_no_bank, qwen_no_bank_mask, _ = other_model(world, "qwen", "peer", False)
  os.environ["CACHE_DIT_B200_MODULATION_BANK"] = "1"
  rel8 = float((wire8[-1][0].float() - peer[-1][0].float()).norm() / peer[-1][0].float().norm())
  others = {}
  for which in ("qwen", "wan"):
    o_nccl, m_nccl, _ = other_model(world, which, "nccl", False)
    o_peer, m_peer, st = other_model(world, which, "peer", False)
    if which == "qwen":
      qwen_peer_out, qwen_peer_mask = o_peer, m_peer
    o_graph, m_graph, st_g = other_model(world, which, "peer", True)
    others[which] = dict(masks=[m_nccl, m_peer, m_graph], status=[st, st_g],
                         peer_equals_nccl=bool(torch.equal(o_nccl, o_peer)),
                         graphs_equal_peer=bool(torch.equal(o_peer, o_graph)),
                         finite=bool(torch.isfinite(o_peer).all().item()))
  report = dict(others=others, fp8_wire=dict(rel=rel8, status=st_wire8, masks=[m for _, m in wire8],
                                             finite=bool(torch.isfinite(wire8[-1][0]).all().item())),
    masks_nccl=[m for _, m in nccl], masks_peer=[m for _, m in peer], masks_graphs=[m for _, m in graphed],
    peer_equals_nccl=all(torch.equal(a, b) for (a, _), (b, _) in zip(nccl, peer)),
    graphs_equal_peer=all(torch.equal(a, b) for (a, _), (b, _) in zip(peer, graphed)),
    status_peer=st_peer, status_graphs=st_graph, replays=replays,
    bank_equals_per_block=all(torch.equal(a, b) and ma == mb for (a, ma), (b, mb) in zip(peer, no_bank)),
    qwen_bank_equals_per_block=bool(torch.equal(qwen_no_bank, qwen_peer_out)) and qwen_no_bank_mask == qwen_peer_mask,
    finite=bool(torch.isfinite(peer[-1][0]).all().item()))
  with open(os.path.join(out_dir, f"rank{rank}.json"), "w") as f:
    json.dump(report, f)
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
