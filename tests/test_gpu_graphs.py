"""CUDA-graph replay of the block segments: a generation with graphs on must reproduce, bit for bit,
the generation with every kernel launched from Python (same cached steps, same latents)."""
import pytest
import torch

import cache_dit_b200 as cd

pytestmark = pytest.mark.gpu


def _generation(graphs: bool, quantize: bool, steps: int = 12):
  from cache_dit_b200.synthetic import FluxTransformer2DModel
  torch.manual_seed(0)
  with torch.device("cuda"):
    model = FluxTransformer2DModel(num_layers=2, num_single_layers=3, dim=256, heads=4, in_channels=16,
                                   joint_attention_dim=64, pooled_projection_dim=32, axes_dims_rope=(8, 28, 28),
                                   time_scale=1.0, modulation_init_std=0.02).to(torch.bfloat16)
  model.eval().requires_grad_(False)
  cd.enable_cache(model,
                  cache_config=cd.DBCacheConfig(Fn_compute_blocks=2, Bn_compute_blocks=0, residual_diff_threshold=0.2,
                                                max_warmup_steps=3, num_inference_steps=steps),
                  calibrator_config=cd.TaylorSeerCalibratorConfig(taylorseer_order=1),
                  quantize_config=cd.QuantizeConfig(quant_type="float8_per_row") if quantize else None)
  runners = []
  if graphs:
    assert cd.enable_cuda_graphs(model, warmup_calls=1) == 1
    runners = cd.graph_runners(model)
  inp = FluxTransformer2DModel.example_inputs(height=256, width=256, text_tokens=32, in_channels=16,
                                              joint_attention_dim=64, pooled_projection_dim=32)
  x = inp.pop("hidden_states")
  outs = []
  with torch.no_grad():
    for gen in range(2):  # second generation: every segment replays from its first step
      cd.refresh_context(model, num_inference_steps=steps)
      lat = x.clone()
      for i in range(steps):
        t = torch.full((1, ), 1.0 - i / steps, device="cuda")
        v = model(hidden_states=lat, timestep=t, **inp)
        lat = (lat.float() - v.float() / steps).to(lat.dtype)
      outs.append((lat.clone(), list(model._cached_steps)))
  torch.cuda.synchronize()
  stats = [(r.captures, r.replays) for r in runners]
  cd.disable_cache(model)
  return outs, stats


@pytest.mark.parametrize("quantize", [False, True])
def test_graph_replay_reproduces_eager_generation(quantize):
  eager, _ = _generation(False, quantize)
  graphed, stats = _generation(True, quantize)
  assert stats and stats[0][0] >= 2 and stats[0][1] > stats[0][0]  # both segments captured, then replayed
  for (lat_e, mask_e), (lat_g, mask_g) in zip(eager, graphed):
    assert mask_e == mask_g
    assert torch.equal(lat_e, lat_g)


def test_graph_runner_falls_back_when_disabled_or_on_new_shapes():
  from cache_dit_b200.caching.block_graphs import BlockGraphRunner
  r = BlockGraphRunner(warmup_calls=1)
  f = lambda a, b, k: (a * k["s"] + b, )
  a, b = torch.randn(8, 16, device="cuda"), torch.randn(8, 16, device="cuda")
  want = a * 3 + b
  for _ in range(4):
    (got, ) = r.run(("seg", ), f, (a, b, {"s": 3}))
    assert torch.equal(got, want)
  assert r.captures == 1 and r.replays == 3
  a2 = torch.randn(4, 16, device="cuda")
  (got, ) = r.run(("seg", ), f, (a2, a2, {"s": 3}))  # another shape: its own key, eager at first
  assert torch.equal(got, a2 * 3 + a2) and r.captures == 1
  (got, ) = r.run(("seg", ), f, (a, b, {"s": 2}))  # another constant: its own key too
  assert torch.equal(got, a * 2 + b)
  r.enabled = False
  (got, ) = r.run(("seg", ), f, (a, b, {"s": 3}))
  assert torch.equal(got, want) and r.replays == 3
