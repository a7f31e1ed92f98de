"""Random-init stand-in with the architecture of FLUX.1-dev's transformer.

19 double-stream + 38 single-stream blocks, hidden 3072, 24 heads of dim 128, RoPE over
(16, 56, 56) axes, adaLN-Zero modulation, QK RMSNorm, tanh-GELU MLP of ratio 4.  Layer names follow
the public diffusers implementation so that the quantization name filter and the block adapter see
what they would see on the real model.  Both block kinds take
`(hidden_states, encoder_hidden_states, temb, image_rotary_emb)` and return
`(encoder_hidden_states, hidden_states)` (ForwardPattern.Pattern_1), so the two lists can be cached
as one 57-block list, the way the reference adapts FLUX
(src/cache_dit/caching/block_adapters/adapters.py:40-103, patch_functors/functor_flux.py:23-211).
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ..caching.block_adapters import BlockAdapter, BlockAdapterRegister
from ..caching.forward_pattern import ForwardPattern
from .layers import (ModulationBank, RMSNorm, RopeCache, TimestepMLP, UlyssesGroup, concat_gelu_linear, gated_add, gated_add_pair,
                     gelu_in_product, gelu_linear_pair,
                     joint_attention, join_tokens, linear_pair, norm_modulate, norm_modulate_linears,
                     norm_modulate_linears_pair, shared_input_linears, split_tokens, timestep_embedding)


class AdaLayerNormZero(nn.Module):
  """SiLU -> Linear -> n chunks of modulation parameters."""

  def __init__(self, dim: int, chunks: int):
    super().__init__()
    self.chunks = chunks
    self.linear = nn.Linear(dim, chunks * dim)

  def forward(self, temb):
    return self.linear(F.silu(temb)).chunk(self.chunks, dim=-1)


class FeedForward(nn.Module):

  def __init__(self, dim: int, inner: int):
    super().__init__()
    self.proj_in = nn.Linear(dim, inner)
    self.proj_out = nn.Linear(inner, dim)


class FluxAttention(nn.Module):

  def __init__(self, dim: int, heads: int, joint: bool):
    super().__init__()
    self.heads = heads
    self.head_dim = dim // heads
    self.to_q = nn.Linear(dim, dim)
    self.to_k = nn.Linear(dim, dim)
    self.to_v = nn.Linear(dim, dim)
    self.norm_q = RMSNorm(self.head_dim)
    self.norm_k = RMSNorm(self.head_dim)
    if joint:
      self.to_out = nn.Linear(dim, dim)
      self.add_q_proj = nn.Linear(dim, dim)
      self.add_k_proj = nn.Linear(dim, dim)
      self.add_v_proj = nn.Linear(dim, dim)
      self.norm_added_q = RMSNorm(self.head_dim)
      self.norm_added_k = RMSNorm(self.head_dim)
      self.to_add_out = nn.Linear(dim, dim)

  def heads_view(self, t):
    return t.unflatten(-1, (self.heads, self.head_dim))


class FluxTransformerBlock(nn.Module):
  """Double-stream block: image and text tokens have their own weights and attend jointly."""

  def __init__(self, dim: int, heads: int, mlp_ratio: float = 4.0):
    super().__init__()
    self.norm1 = AdaLayerNormZero(dim, 6)
    self.norm1_context = AdaLayerNormZero(dim, 6)
    self.attn = FluxAttention(dim, heads, joint=True)
    self.ff = FeedForward(dim, int(dim * mlp_ratio))
    self.ff_context = FeedForward(dim, int(dim * mlp_ratio))
    self.cp: Optional[UlyssesGroup] = None

  def forward(self, hidden_states, encoder_hidden_states, temb, image_rotary_emb):
    a = self.attn
    bank = getattr(self, "mod_bank", None)
    if bank is not None:  # computed once per step for all blocks, column-sharded over the ranks
      mod, c_mod = bank.outputs((self.norm1.linear, self.norm1_context.linear))
    else:
      # both streams' modulation projections read SiLU(temb): one quantization, one weight-streaming product
      mod, c_mod = shared_input_linears(F.silu(temb), (self.norm1.linear, self.norm1_context.linear))
    shift, scale, gate, shift_mlp, scale_mlp, gate_mlp = mod.chunk(6, dim=-1)
    c_shift, c_scale, c_gate, c_shift_mlp, c_scale_mlp, c_gate_mlp = c_mod.chunk(6, dim=-1)
    (q, k, v), (cq, ck, cv) = norm_modulate_linears_pair(
      (hidden_states, shift, scale, (a.to_q, a.to_k, a.to_v)),
      (encoder_hidden_states, c_shift, c_scale, (a.add_q_proj, a.add_k_proj, a.add_v_proj)))
    o = joint_attention(((cq, a.norm_added_q), (q, a.norm_q)), ((ck, a.norm_added_k), (k, a.norm_k)), (cv, v),
                        image_rotary_emb, a.heads, self.cp)
    n_txt = encoder_hidden_states.shape[1]
    y, cy = linear_pair(o[:, n_txt:], a.to_out, o[:, :n_txt], a.to_add_out)
    hidden_states, encoder_hidden_states = gated_add_pair(hidden_states, gate, y, encoder_hidden_states, c_gate, cy)
    act = gelu_in_product()
    (h, ), (c, ) = norm_modulate_linears_pair((hidden_states, shift_mlp, scale_mlp, (self.ff.proj_in, )),
                                              (encoder_hidden_states, c_shift_mlp, c_scale_mlp, (self.ff_context.proj_in, )),
                                              gelu_last=act)
    y, cy = gelu_linear_pair(h, self.ff.proj_out, c, self.ff_context.proj_out, activated=act)
    hidden_states, encoder_hidden_states = gated_add_pair(hidden_states, gate_mlp, y, encoder_hidden_states, c_gate_mlp, cy)
    return encoder_hidden_states, hidden_states


class FluxSingleTransformerBlock(nn.Module):
  """Single-stream block: text and image tokens share weights; attention and MLP run in parallel."""

  def __init__(self, dim: int, heads: int, mlp_ratio: float = 4.0):
    super().__init__()
    self.norm = AdaLayerNormZero(dim, 3)
    self.proj_mlp = nn.Linear(dim, int(dim * mlp_ratio))
    self.attn = FluxAttention(dim, heads, joint=False)
    self.proj_out = nn.Linear(dim + int(dim * mlp_ratio), dim)
    self.cp: Optional[UlyssesGroup] = None

  def forward(self, hidden_states, encoder_hidden_states, temb, image_rotary_emb):
    a = self.attn
    n_txt = encoder_hidden_states.shape[1]
    x = join_tokens(encoder_hidden_states, hidden_states)
    bank = getattr(self, "mod_bank", None)
    shift, scale, gate = bank.outputs((self.norm.linear, ))[0].chunk(3, dim=-1) if bank is not None else self.norm(temb)
    act = gelu_in_product()
    q, k, v, mlp = norm_modulate_linears(x, shift, scale, (a.to_q, a.to_k, a.to_v, self.proj_mlp), gelu_last=act)
    o = joint_attention(((q, a.norm_q), ), ((k, a.norm_k), ), (v, ), image_rotary_emb, a.heads, self.cp)
    y = concat_gelu_linear(o, mlp, self.proj_out, tail_activated=act)
    return split_tokens(gated_add(x, gate, y), n_txt)


class FluxTransformer2DModel(nn.Module):
  _repeated_blocks = ["FluxTransformerBlock", "FluxSingleTransformerBlock"]

  def __init__(self, num_layers: int = 19, num_single_layers: int = 38, dim: int = 3072, heads: int = 24,
               in_channels: int = 64, joint_attention_dim: int = 4096, pooled_projection_dim: int = 768,
               axes_dims_rope: Tuple[int, int, int] = (16, 56, 56), guidance_embeds: bool = True,
               time_scale: float = 1000.0, modulation_init_std: Optional[float] = None):
    super().__init__()
    self.dim = dim
    self.axes_dims_rope = axes_dims_rope
    # multiplier of the timestep before the sinusoidal embedding (1000 in FLUX); a random-init
    # embedder is smoother in t for smaller values
    self.time_scale = time_scale
    self.x_embedder = nn.Linear(in_channels, dim)
    self.context_embedder = nn.Linear(joint_attention_dim, dim)
    self.time_embedder = TimestepMLP(256, dim)
    self.guidance_embedder = TimestepMLP(256, dim) if guidance_embeds else None
    self.text_embedder = TimestepMLP(pooled_projection_dim, dim)
    self.transformer_blocks = nn.ModuleList([FluxTransformerBlock(dim, heads) for _ in range(num_layers)])
    self.single_transformer_blocks = nn.ModuleList(
      [FluxSingleTransformerBlock(dim, heads) for _ in range(num_single_layers)])
    self.norm_out = AdaLayerNormZero(dim, 2)
    self.proj_out = nn.Linear(dim, in_channels)
    self._cp: Optional[UlyssesGroup] = None
    self._rope_cache = RopeCache()
    if modulation_init_std is not None:
      # small adaLN modulation weights (the trained model starts from adaLN-Zero): with random
      # weights of ordinary scale the residual stream changes by ~45 % between steps and nothing
      # is ever cacheable; with small ones the step-to-step relative L1 walks through 0.06 / 0.07 /
      # 0.08 like the reference's synthetic cache-step configuration
      for block in list(self.transformer_blocks) + list(self.single_transformer_blocks):
        for mod in (getattr(block, "norm1", None), getattr(block, "norm1_context", None), getattr(block, "norm", None)):
          if mod is not None:
            nn.init.normal_(mod.linear.weight, std=modulation_init_std)
            nn.init.zeros_(mod.linear.bias)

  # ---- context parallelism: split tokens and ids at the root, gather after proj_out
  # (the reference's plan for FLUX: src/cache_dit/distributed/transformers/flux.py:49-61)
  def enable_context_parallel(self, config):
    group = getattr(config, "_group", None)
    exchange = None
    if config.exchange_mode() == "peer":
      from ..distributed.peer_exchange import PeerExchange
      exchange = PeerExchange(group, fp8=bool(config.ulysses_float8))
    elif config.ulysses_float8:
      raise NotImplementedError("FP8 head/token exchange is built for the peer-memory exchange only "
                                "(parallel_kwargs={'exchange': 'peer'})")
    self._cp = UlyssesGroup(group, exchange)
    for block in list(self.transformer_blocks) + list(self.single_transformer_blocks):
      block.cp = self._cp
    self._mod_bank = None
    self._mod_bank_wanted = self._cp.world > 1 and os.environ.get("CACHE_DIT_B200_MODULATION_BANK", "1") != "0"
    # the block modules themselves: inside `forward` of a cache-enabled model the two lists hold the cache runner
    self._mod_bank_blocks = (list(self.transformer_blocks), list(self.single_transformer_blocks))

  def disable_context_parallel(self):
    if self._cp is not None and self._cp.exchange is not None:
      self._cp.exchange.close()
    self._cp = None
    self._mod_bank = None
    self._mod_bank_wanted = False
    for block in list(self.transformer_blocks) + list(self.single_transformer_blocks):
      block.cp = None
      block.mod_bank = None
    self._mod_bank_blocks = ([], [])

  def _modulation_for_step(self, temb):
    """Under context parallelism with FP8 modulation linears: all blocks' modulation vectors as one column-sharded
    product + all-gather per step (`ModulationBank`) instead of 57 replicated weight-streaming products."""
    if not getattr(self, "_mod_bank_wanted", False) or not temb.is_cuda:
      return
    if self._mod_bank is None or not self._mod_bank.still_valid():
      from ..quantization.linear import Float8RowwiseLinear
      double, single = self._mod_bank_blocks
      groups = [(b.norm1.linear, b.norm1_context.linear) for b in double] + [(b.norm.linear, ) for b in single]
      if not all(isinstance(l, Float8RowwiseLinear) for g in groups for l in g):
        self._mod_bank_wanted = False
        return
      try:
        self._mod_bank = ModulationBank(groups, self._cp.group)
      except ValueError:
        self._mod_bank_wanted = False
        return
      self._mod_bank_index = {id(b): i for i, b in enumerate(double + single)}
      for b in double + single:
        b.mod_bank = self._mod_bank
    self._mod_bank.begin_call(temb)
    first = self.transformer_blocks
    if not (len(first) == 1 and hasattr(first[0], "context_manager")):  # no cache runner stands in for the block list
      self._mod_bank.prepare(0, len(self._mod_bank_index))

  def prepare_blocks(self, blocks) -> None:
    """Called by the cache runner before it runs `blocks` (a contiguous slice of the 57-block list)."""
    bank = getattr(self, "_mod_bank", None)
    if bank is None or not getattr(self, "_mod_bank_wanted", False):
      return
    index = self._mod_bank_index
    if id(blocks[0]) in index:
      bank.prepare(index[id(blocks[0])], index[id(blocks[-1])] + 1)

  def forward(self, hidden_states, encoder_hidden_states, pooled_projections, timestep, img_ids, txt_ids,
              guidance=None):
    cp = self._cp
    if cp is not None and cp.world > 1:
      hidden_states = hidden_states.chunk(cp.world, dim=1)[cp.rank]
      encoder_hidden_states = encoder_hidden_states.chunk(cp.world, dim=1)[cp.rank]
      img_ids = img_ids.chunk(cp.world, dim=0)[cp.rank]
      txt_ids = txt_ids.chunk(cp.world, dim=0)[cp.rank]
    dt = hidden_states.dtype
    hidden_states = self.x_embedder(hidden_states)
    temb = self.time_embedder(timestep_embedding(timestep * self.time_scale, 256).to(dt))
    if self.guidance_embedder is not None and guidance is not None:
      temb = temb + self.guidance_embedder(timestep_embedding(guidance * 1000.0, 256).to(dt))
    temb = temb + self.text_embedder(pooled_projections)
    self._modulation_for_step(temb)
    encoder_hidden_states = self.context_embedder(encoder_hidden_states)
    rope = self._rope_cache.get((txt_ids, img_ids), self.axes_dims_rope, dt)
    for block in self.transformer_blocks:
      encoder_hidden_states, hidden_states = block(hidden_states, encoder_hidden_states, temb, rope)
    for block in self.single_transformer_blocks:
      encoder_hidden_states, hidden_states = block(hidden_states, encoder_hidden_states, temb, rope)
    shift, scale = self.norm_out(temb)
    out = self.proj_out(norm_modulate(hidden_states, shift, scale))
    if cp is not None and cp.world > 1:
      import torch.distributed as dist
      parts = [torch.empty_like(out) for _ in range(cp.world)]
      dist.all_gather(parts, out.contiguous(), group=cp.group)
      out = torch.cat(parts, dim=1)
    return out

  # ---- synthetic inputs of the 1024 x 1024 configuration: 4096 image + 512 text tokens
  @staticmethod
  def example_inputs(batch: int = 1, height: int = 1024, width: int = 1024, text_tokens: int = 512,
                     device="cuda", dtype=torch.bfloat16, seed: int = 0, in_channels: int = 64,
                     joint_attention_dim: int = 4096, pooled_projection_dim: int = 768):
    g = torch.Generator().manual_seed(seed)
    gh, gw = height // 16, width // 16
    img_ids = torch.zeros(gh, gw, 3)
    img_ids[..., 1] = torch.arange(gh)[:, None]
    img_ids[..., 2] = torch.arange(gw)[None, :]
    return dict(
      hidden_states=torch.randn(batch, gh * gw, in_channels, generator=g).to(device=device, dtype=dtype),
      encoder_hidden_states=torch.randn(batch, text_tokens, joint_attention_dim, generator=g).to(device=device, dtype=dtype),
      pooled_projections=torch.randn(batch, pooled_projection_dim, generator=g).to(device=device, dtype=dtype),
      img_ids=img_ids.reshape(-1, 3).to(device), txt_ids=torch.zeros(text_tokens, 3, device=device),
      guidance=torch.full((batch, ), 3.5, device=device))


@BlockAdapterRegister.register("Flux")
def flux_adapter(pipe_or_transformer, **kwargs) -> BlockAdapter:
  transformer = pipe_or_transformer if isinstance(pipe_or_transformer, nn.Module) else pipe_or_transformer.transformer
  pipe = None if isinstance(pipe_or_transformer, nn.Module) else pipe_or_transformer
  return BlockAdapter(pipe=pipe, transformer=transformer,
                      blocks=transformer.transformer_blocks + transformer.single_transformer_blocks,
                      blocks_name="transformer_blocks", dummy_blocks_names=["single_transformer_blocks"],
                      forward_pattern=ForwardPattern.Pattern_1, check_forward_pattern=False, **kwargs)
