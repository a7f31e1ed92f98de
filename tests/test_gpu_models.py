"""Qwen-Image- and Wan-shape stand-ins on a B200: the product path (kernels, FP8 linears, separate CFG)
against the numpy oracle plugged into the same runner, CUDA-graph replay against eager launches,
and the row-norm mode of the head-scatter kernel against eager PyTorch."""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

import cache_dit_b200 as cd
from cache_dit_b200.caching import step_ops
from tests.fake_ops import OracleStepOps

pytestmark = pytest.mark.gpu


def _qwen():
  from cache_dit_b200.synthetic import QwenImageDenoisePipeline, QwenImageTransformer2DModel
  with torch.device("cuda"):
    model = QwenImageTransformer2DModel(num_layers=5, dim=256, heads=4, in_channels=16, joint_attention_dim=64,
                                        axes_dims_rope=(8, 28, 28), time_scale=1.0, modulation_init_std=0.02)
  inputs = QwenImageTransformer2DModel.example_inputs(height=272, width=272, text_tokens=33, in_channels=16,
                                                      joint_attention_dim=64)
  return model, inputs, QwenImageDenoisePipeline


def _wan():
  from cache_dit_b200.synthetic import WanDenoisePipeline, WanTransformer3DModel
  with torch.device("cuda"):
    model = WanTransformer3DModel(num_layers=4, dim=256, heads=2, ffn_dim=512, in_channels=16, text_dim=64,
                                  axes_dims_rope=(44, 42, 42), time_scale=1.0, modulation_init_std=0.02)
  inputs = WanTransformer3DModel.example_inputs(frames=3, height=5, width=7, text_tokens=16, in_channels=16, text_dim=64)
  return model, inputs, WanDenoisePipeline


def _generate(build, ops, graphs=False, threshold=0.15, steps=10):
  step_ops.set_ops(ops)
  try:
    torch.manual_seed(0)
    model, inputs, pipe_cls = build()
    model = model.to(torch.bfloat16).eval().requires_grad_(False)
    pipe = pipe_cls(model, inputs)
    cd.enable_cache(pipe, cache_config=cd.DBCacheConfig(Fn_compute_blocks=1, max_warmup_steps=3,
                                                        residual_diff_threshold=threshold),
                    calibrator_config=cd.TaylorSeerCalibratorConfig(taylorseer_order=1),
                    quantize_config=cd.QuantizeConfig(quant_type="float8_per_row"))
    if graphs:
      assert cd.enable_cuda_graphs(pipe, warmup_calls=1) >= 1
    out = pipe(num_inference_steps=steps)
    if graphs:  # a second generation replays every segment from its first step
      out = pipe(num_inference_steps=steps)
    stats = cd.summary(pipe, logging=False)[-1]
    replays = sum(r.replays for r in cd.graph_runners(pipe))
    fp8 = model._quantize_stats
    cd.disable_cache(pipe)
    return out.float().cpu().numpy(), stats, replays, fp8
  finally:
    step_ops.set_ops(None)


@pytest.mark.parametrize("build", [_qwen, _wan], ids=["qwen_image", "wan"])
def test_model_kernels_vs_oracle_ops(build):
  got, s_k, _, fp8 = _generate(build, None)
  want, s_o, _, _ = _generate(build, OracleStepOps())
  assert fp8["quantized"] > 0
  assert s_k.cached_steps == s_o.cached_steps and s_k.cached_steps  # bit-exact masks, both CFG branches
  assert s_k.cfg_cached_steps == s_o.cfg_cached_steps and s_k.cfg_cached_steps
  for k, v in s_o.residual_diffs.items():
    assert abs(s_k.residual_diffs[k] - v) <= 1e-3 * abs(v) + 1e-12
  rel = np.linalg.norm(got - want) / np.linalg.norm(want)
  assert rel < 2e-2, rel


def test_qwen_modulation_linears_stay_bf16():
  """The name filter of the reference (`mod` is an excluded pattern) keeps img_mod / txt_mod in bf16."""
  model, _, _ = _qwen()
  model = model.to(torch.bfloat16)
  cd.quantize(model, cd.QuantizeConfig(quant_type="float8_per_row"))
  block = model.transformer_blocks[0]
  assert isinstance(block.img_mod[1], torch.nn.Linear) and not isinstance(block.img_mod[1], cd.Float8RowwiseLinear)
  assert isinstance(block.attn.to_q, cd.Float8RowwiseLinear)
  assert isinstance(block.img_mlp.net[0].proj, cd.Float8RowwiseLinear)


@pytest.mark.parametrize("build", [_qwen, _wan], ids=["qwen_image", "wan"])
def test_model_graph_replay_equals_eager(build):
  eager, s_e, _, _ = _generate(build, None)
  graphed, s_g, replays, _ = _generate(build, None, graphs=True)
  assert replays > 0
  assert s_g.cached_steps == s_e.cached_steps
  np.testing.assert_array_equal(graphed, eager)


@pytest.mark.parametrize("heads,d,tokens", [(2, 128, 37), (40, 128, 9), (5, 64, 130)])
def test_row_norm_rope_matches_eager(heads, d, tokens):
  """RMSNorm over the whole row (Wan's q / k normalisation) + rotary embedding in the scatter kernel."""
  from cache_dit_b200 import _native as nat
  g = torch.Generator().manual_seed(heads * d)
  c = heads * d
  wide = torch.randn(1, tokens, 2 * c, generator=g).to("cuda", torch.bfloat16)
  x = wide[..., c:]
  w = (1 + 0.1 * torch.randn(c, generator=g)).to("cuda", torch.bfloat16)
  ang = torch.rand(tokens, d // 2, generator=g) * 6.28
  cos = torch.cos(ang).repeat_interleave(2, dim=-1).to("cuda", torch.bfloat16).contiguous()
  sin = torch.sin(ang).repeat_interleave(2, dim=-1).to("cuda", torch.bfloat16).contiguous()
  out = torch.full((1, tokens, heads, d), float("nan"), device="cuda", dtype=torch.bfloat16)
  nat.scatter_heads(x, w, cos, sin, 0, [out.data_ptr()], out.stride(0), 0, heads, 1e-6, across_heads=True)
  torch.cuda.synchronize()
  y = F.rms_norm(x.float(), (c, ), w.float(), 1e-6).unflatten(-1, (heads, d))
  cs, sn = cos.float()[None, :, None, :], sin.float()[None, :, None, :]
  y1, y2 = y.unflatten(-1, (-1, 2)).unbind(-1)
  ref = y * cs + torch.stack([-y2, y1], dim=-1).flatten(-2) * sn
  assert torch.isfinite(out).all().item()
  assert ((out.float() - ref).abs() <= 3 * 2.0**-8 * ref.abs() + 2e-2).all().item()


def test_flux_full_size_generation_kernels_vs_oracle_ops():
  """The benchmark's own workload at full size (19 + 38 blocks, hidden 3072, 4096 + 512 tokens, 28 steps,
  F8B0, threshold 0.08, TaylorSeer order 1, FP8 linears): hit / miss mask and counters bit-exact, diffs
  within 1e-3, final latents within 2e-2 relative L2 of the run whose cache arithmetic is the numpy oracle."""
  from cache_dit_b200.synthetic import FluxDenoisePipeline, FluxTransformer2DModel
  torch.manual_seed(0)
  with torch.device("cuda"):
    model = FluxTransformer2DModel(time_scale=1.0, modulation_init_std=0.02).to(torch.bfloat16)
  model.eval().requires_grad_(False)
  cd.quantize(model, cd.QuantizeConfig(quant_type="float8_per_row"))
  inputs = FluxTransformer2DModel.example_inputs()
  pipe = FluxDenoisePipeline(model, inputs)

  def run(ops):
    step_ops.set_ops(ops)
    try:
      cd.enable_cache(pipe, cache_config=cd.DBCacheConfig(Fn_compute_blocks=8, Bn_compute_blocks=0,
                                                          residual_diff_threshold=0.08, max_warmup_steps=8),
                      calibrator_config=cd.TaylorSeerCalibratorConfig(taylorseer_order=1))
      out = pipe(num_inference_steps=28)
      stats = cd.summary(pipe, logging=False)[-1]
      cd.disable_cache(pipe)
      return out.float().cpu().numpy(), stats
    finally:
      step_ops.set_ops(None)

  got, s_k = run(None)
  want, s_o = run(OracleStepOps())
  assert s_k.cached_steps == s_o.cached_steps and len(s_k.cached_steps) >= 5
  assert set(s_k.residual_diffs) == set(s_o.residual_diffs)
  for k, v in s_o.residual_diffs.items():
    assert abs(s_k.residual_diffs[k] - v) <= 1e-3 * abs(v) + 1e-12
  rel = np.linalg.norm(got - want) / np.linalg.norm(want)
  assert np.isfinite(got).all() and rel < 2e-2, rel


def test_final_latents_against_library_fp8_linears():
  """Product path (fused producers, this package's quantization + tcgen05 GEMM) against the same model whose
  FP8 linears are PyTorch library ops (`torch._scaled_mm` row-wise on torch-quantized operands) and whose block
  glue is eager PyTorch: same cache decisions, final latents within 2e-2 relative L2 after 24 steps.  Unlike the
  oracle-backed runs, the two arms share no FP8 arithmetic, so the error of the FP8 linears accumulating through
  the blocks is part of what is compared."""
  from cache_dit_b200.synthetic import FluxDenoisePipeline, FluxTransformer2DModel
  from tests.library_fp8 import LibraryFloat8Linear, swap_repeated_block_linears

  def build():
    torch.manual_seed(0)
    with torch.device("cuda"):
      model = FluxTransformer2DModel(num_layers=4, num_single_layers=6, dim=256, heads=4, in_channels=16,
                                     joint_attention_dim=64, pooled_projection_dim=32, axes_dims_rope=(8, 28, 28),
                                     time_scale=1.0, modulation_init_std=0.02).to(torch.bfloat16)
    inputs = FluxTransformer2DModel.example_inputs(height=256, width=256, text_tokens=16, in_channels=16,
                                                   joint_attention_dim=64, pooled_projection_dim=32)
    return model.eval().requires_grad_(False), inputs

  def generate(library: bool):
    model, inputs = build()
    if library:
      assert swap_repeated_block_linears(model) > 0
      assert isinstance(model.transformer_blocks[0].attn.to_q, LibraryFloat8Linear)
    pipe = FluxDenoisePipeline(model, inputs)
    cd.enable_cache(pipe, cache_config=cd.DBCacheConfig(Fn_compute_blocks=2, max_warmup_steps=4,
                                                        residual_diff_threshold=0.13),
                    calibrator_config=cd.TaylorSeerCalibratorConfig(taylorseer_order=1),
                    quantize_config=None if library else cd.QuantizeConfig(quant_type="float8_per_row"))
    if not library:
      assert isinstance(model.transformer_blocks[0].attn.to_q, cd.Float8RowwiseLinear)
      assert model._quantize_stats["quantized"] > 0
    out = pipe(num_inference_steps=24)
    stats = cd.summary(pipe, logging=False)[-1]
    cd.disable_cache(pipe)
    return out.float().cpu().numpy(), stats

  got, s_ours = generate(False)
  want, s_lib = generate(True)
  assert s_ours.cached_steps == s_lib.cached_steps and len(s_ours.cached_steps) >= 4
  for k, v in s_lib.residual_diffs.items():
    # the diffs are bf16 values (steps of 0.4-0.8 %) and now carry the two arms' FP8 / rounding differences too
    assert abs(s_ours.residual_diffs[k] - v) <= 6e-2 * abs(v) + 1e-12
  rel = np.linalg.norm(got - want) / np.linalg.norm(want)
  assert np.isfinite(got).all() and 0.0 < rel < 2e-2, rel


@pytest.mark.parametrize("build", [_qwen, _wan, "flux"], ids=["qwen_image", "wan", "flux"])
def test_gelu_in_the_product_epilogue_equals_gelu_in_the_quantization_kernel(build, monkeypatch):
  """By default an MLP-in projection applies the MLP's tanh-GELU in its own epilogue and the quantization in front
  of the MLP-out projection only quantizes; CACHE_DIT_B200_GELU_IN_PRODUCT=0 keeps the activation in that
  quantization kernel.  Same device function and rounding points: same cache decisions, and final latents that
  differ only by the few FP8 codes the corrected division of the plain quantization kernel decides differently."""
  if build == "flux":
    def build():
      from cache_dit_b200.synthetic import FluxDenoisePipeline, FluxTransformer2DModel
      with torch.device("cuda"):
        model = FluxTransformer2DModel(num_layers=3, num_single_layers=4, dim=256, heads=4, in_channels=16,
                                       joint_attention_dim=64, pooled_projection_dim=32, axes_dims_rope=(8, 28, 28),
                                       time_scale=1.0, modulation_init_std=0.02)
      inputs = FluxTransformer2DModel.example_inputs(height=256, width=256, text_tokens=16, in_channels=16,
                                                     joint_attention_dim=64, pooled_projection_dim=32)
      return model, inputs, FluxDenoisePipeline
  results = {}
  for flag in ("1", "0"):
    monkeypatch.setenv("CACHE_DIT_B200_GELU_IN_PRODUCT", flag)
    results[flag] = _generate(build, None, steps=12)
  (a, sa, _, fa), (b, sb, _, _) = results["1"], results["0"]
  assert fa["quantized"] > 0
  assert sa.cached_steps == sb.cached_steps and len(sa.cached_steps) >= 2
  rel = np.linalg.norm(a - b) / np.linalg.norm(b)
  assert np.isfinite(a).all() and rel < 2e-3, rel


def test_fused_forwards_for_a_foreign_model_with_the_flux_attribute_layout(monkeypatch):
  """`quantize` gives blocks that merely LOOK like the public FLUX blocks (attribute names, calling convention of
  the reference's patched forward) the producer-fused forwards; the result must agree with the same FP8 model run
  through its own eager forwards (separate quantization kernels, eager LayerNorm / GELU / concat / RoPE), and take
  far fewer launches of this package's kernels plus none of the eager glue."""
  from cache_dit_b200 import _native as nat
  from tests.fake_flux_layout import TinyFlux
  dev = torch.device("cuda")
  g = torch.Generator().manual_seed(11)

  def build(fuse: bool):
    monkeypatch.setenv("CACHE_DIT_B200_FUSE_BLOCKS", "1" if fuse else "0")
    torch.manual_seed(4)
    model = TinyFlux().to(torch.bfloat16).to(dev).eval().requires_grad_(False)
    for blk in list(model.transformer_blocks) + list(model.single_transformer_blocks):  # small modulation: a tame residual stream
      for name in ("norm1", "norm1_context", "norm"):
        if hasattr(blk, name):
          torch.nn.init.normal_(getattr(blk, name).linear.weight, std=0.02)
    cd.quantize(model, cd.QuantizeConfig(quant_type="float8_per_row"))
    return model

  n_img, n_txt, dim, d = 192, 24, 256, 128
  x = torch.randn(2, n_img, dim, generator=g).to(dev, torch.bfloat16)
  c = torch.randn(2, n_txt, dim, generator=g).to(dev, torch.bfloat16)
  temb = torch.randn(2, dim, generator=g).to(dev, torch.bfloat16)
  ang = torch.rand(n_txt + n_img, d // 2, generator=g) * 6.28
  rope = (torch.cos(ang).repeat_interleave(2, dim=-1).to(dev), torch.sin(ang).repeat_interleave(2, dim=-1).to(dev))  # fp32, as diffusers passes them

  eager = build(False)
  assert eager._quantize_stats["fused_blocks"] == 0
  l0 = nat.launch_count
  want_c, want_x = eager(x, c, temb, rope)
  eager_launches = nat.launch_count - l0
  fused = build(True)
  assert fused._quantize_stats["fused_blocks"] == 4
  l0 = nat.launch_count
  got_c, got_x = fused(x, c, temb, rope)
  fused_launches = nat.launch_count - l0
  torch.cuda.synchronize()
  for got, want in ((got_x, want_x), (got_c, want_c)):
    rel = float((got.float() - want.float()).norm() / want.float().norm())
    assert torch.isfinite(got).all() and rel < 2e-2, rel
  assert fused_launches < eager_launches, (fused_launches, eager_launches)
  # removing the quantization statistics puts the blocks' own forwards back
  from cache_dit_b200.quantization import remove_quantization_stats
  remove_quantization_stats(fused)
  assert not getattr(fused.transformer_blocks[0], "_cdb_fused_forward", False)
