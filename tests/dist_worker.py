"""Worker for the world-size-2 gloo tests (launched by tests/test_distributed_cpu.py with torchrun)."""
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import cache_dit_b200 as cd  # noqa: E402
from cache_dit_b200.caching import step_ops  # noqa: E402
from oracle import cache_oracle as O  # noqa: E402
from tests.fake_ops import OracleStepOps  # noqa: E402


def decision_case(rank, world):
  """Each rank checks its own (uneven) token shard; the decision must come from the averaged means."""
  g = torch.Generator().manual_seed(5)
  prev = torch.randn(1, 37, 16, generator=g)
  prev[:, :10] *= 5.0
  cur = prev + 0.06 * torch.randn(1, 37, 16, generator=g)
  shard = lambda t: torch.tensor_split(t, world, dim=1)[rank].contiguous().to(torch.bfloat16)
  mgr = cd.CachedContextManager("m", persistent_context=True)
  mgr.new_context(name="c", cache_config=cd.DBCacheConfig(max_warmup_steps=0, enable_separate_cfg=False,
                                                          residual_diff_threshold=0.06))
  out = []
  for step in range(3):
    mgr.set_context("c")
    mgr.mark_step_begin()
    hit = mgr.can_cache(shard(cur if step else prev), parallelized=True, prefix="b_Fn_residual")
    if not hit:
      mgr.set_Fn_buffer(shard(prev), prefix="b_Fn_residual")
    out.append(bool(hit))
  want = O.rel_l1(O.round_bf16(prev.numpy()), O.round_bf16(cur.numpy()), "bf16", shards=world)
  return dict(hits=out, diffs=mgr.get_residual_diffs(), want=want)


def flux_case(rank, world):
  from cache_dit_b200.synthetic import FluxDenoisePipeline, FluxTransformer2DModel
  kw = dict(num_layers=2, num_single_layers=3, dim=64, heads=4, in_channels=8, joint_attention_dim=16,
            pooled_projection_dim=12, axes_dims_rope=(4, 6, 6))
  ikw = dict(height=128, width=128, text_tokens=8, device="cpu", dtype=torch.float32, in_channels=8,
             joint_attention_dim=16, pooled_projection_dim=12)

  def run(parallel):
    torch.manual_seed(0)
    model = FluxTransformer2DModel(time_scale=1.0, **kw)
    pipe = FluxDenoisePipeline(model, FluxTransformer2DModel.example_inputs(**ikw))
    cd.enable_cache(pipe, cache_config=cd.DBCacheConfig(Fn_compute_blocks=1, max_warmup_steps=2,
                                                        residual_diff_threshold=0.2),
                    calibrator_config=cd.TaylorSeerCalibratorConfig(),
                    parallelism_config=cd.ParallelismConfig(ulysses_size=world) if parallel else None)
    out = pipe(num_inference_steps=8)
    stats = cd.summary(pipe, logging=False)[-1]
    cd.disable_cache(pipe)
    return out, stats

  single, s1 = run(False)
  sharded, s2 = run(True)
  return dict(rel=float((single - sharded).norm() / single.norm()), cached_single=s1.cached_steps,
              cached_sharded=s2.cached_steps, diffs_single=s1.residual_diffs, diffs_sharded=s2.residual_diffs)


def _sharded_vs_single(world, build, pipe_cls, threshold):
  def run(parallel):
    torch.manual_seed(0)
    model, inputs = build()
    pipe = pipe_cls(model, inputs, separate_cfg=False)
    cd.enable_cache(pipe, cache_config=cd.DBCacheConfig(Fn_compute_blocks=1, max_warmup_steps=2,
                                                        residual_diff_threshold=threshold, enable_separate_cfg=False),
                    calibrator_config=cd.TaylorSeerCalibratorConfig(),
                    parallelism_config=cd.ParallelismConfig(ulysses_size=world) if parallel else None)
    out = pipe(num_inference_steps=8)
    stats = cd.summary(pipe, logging=False)[-1]
    cd.disable_cache(pipe)
    return out, stats

  single, s1 = run(False)
  sharded, s2 = run(True)
  return dict(rel=float((single - sharded).norm() / single.norm()), cached_single=s1.cached_steps,
              cached_sharded=s2.cached_steps, diffs_single=s1.residual_diffs, diffs_sharded=s2.residual_diffs)


def qwen_case(rank, world):
  """49 image + 5 text tokens on 2 ranks: 25 / 24 and 3 / 2, the uneven split of `ulysses_anything`."""
  from cache_dit_b200.synthetic import QwenImageDenoisePipeline, QwenImageTransformer2DModel

  def build():
    model = QwenImageTransformer2DModel(num_layers=4, dim=64, heads=4, in_channels=8, joint_attention_dim=16,
                                        axes_dims_rope=(4, 6, 6), time_scale=1.0, modulation_init_std=0.02)
    return model, QwenImageTransformer2DModel.example_inputs(height=112, width=112, text_tokens=5, device="cpu",
                                                             dtype=torch.float32, in_channels=8, joint_attention_dim=16)

  return _sharded_vs_single(world, build, QwenImageDenoisePipeline, 0.3)


def wan_case(rank, world):
  """Video tokens sharded, text whole on every rank; blocks return hidden states only (Pattern_2)."""
  from cache_dit_b200.synthetic import WanDenoisePipeline, WanTransformer3DModel

  def build():
    model = WanTransformer3DModel(num_layers=3, dim=64, heads=4, ffn_dim=96, in_channels=8, text_dim=16,
                                  axes_dims_rope=(4, 6, 6), time_scale=1.0, modulation_init_std=0.02)
    return model, WanTransformer3DModel.example_inputs(frames=3, height=4, width=5, text_tokens=6, device="cpu",
                                                       dtype=torch.float32, in_channels=8, text_dim=16)

  return _sharded_vs_single(world, build, WanDenoisePipeline, 0.3)


def config_case(rank, world):
  """A configuration dictionary with `ulysses_size: auto` resolves to the number of ranks."""
  loaded = cd.load_configs({"cache_config": {"Fn_compute_blocks": 1, "enable_taylorseer": True},
                            "parallelism_config": {"ulysses_size": "auto", "ulysses_anything": True}})
  p = loaded["parallelism_config"]
  return dict(ulysses_size=p.ulysses_size, anything=bool(p.ulysses_anything), backend=str(p.backend),
              exchange=p.exchange_mode(), order=loaded["calibrator_config"].taylorseer_order)


def main():
  dist.init_process_group("gloo")
  rank, world = dist.get_rank(), dist.get_world_size()
  step_ops.set_ops(OracleStepOps())
  result = dict(rank=rank, decision=decision_case(rank, world), flux=flux_case(rank, world),
                qwen=qwen_case(rank, world), wan=wan_case(rank, world), config=config_case(rank, world))
  with open(os.path.join(sys.argv[1], f"rank{rank}.json"), "w") as f:
    json.dump(result, f)
  dist.barrier()
  dist.destroy_process_group()


if __name__ == "__main__":
  main()
