"""Random-init stand-in with the architecture of Wan2.1-14B's video transformer.

40 blocks, hidden 5120, 40 heads of dim 128, FFN 13824: self-attention over the video tokens (q / k
RMSNorm over the whole hidden dimension, rotary embedding over (frame, height, width) axes of
44 + 42 + 42), cross-attention to 512 text tokens, tanh-GELU FFN; adaLN modulation = a learned
`scale_shift_table` plus a 6-way projection of the timestep embedding.  Layer names follow the public
diffusers implementation.  Blocks take `(hidden_states, encoder_hidden_states, temb, rotary_emb)` and
return `hidden_states` only: ForwardPattern.Pattern_2, one 40-block list, separate CFG
(src/cache_dit/caching/block_adapters/adapters.py:178-187).

Context parallelism (src/cache_dit/distributed/transformers/wan.py:52-65): video tokens and their rotary
rows are sharded, the text stays whole on every rank; self-attention exchanges heads for tokens,
cross-attention needs no communication (every query sees the whole text locally).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ..caching.block_adapters import BlockAdapter, BlockAdapterRegister
from ..caching.forward_pattern import ForwardPattern
from .context_parallel import ContextParallelMixin
from .layers import (RMSNorm, TimestepMLP, UlyssesGroup, gated_add, gelu_in_product, gelu_linear, joint_attention, norm_modulate,
                     norm_modulate_linears, RopeCache, timestep_embedding)
from .qwen_image import QwenFeedForward


class WanAttention(nn.Module):

  def __init__(self, dim: int, heads: int):
    super().__init__()
    self.heads = heads
    self.head_dim = dim // heads
    self.to_q, self.to_k, self.to_v = nn.Linear(dim, dim), nn.Linear(dim, dim), nn.Linear(dim, dim)
    self.norm_q, self.norm_k = RMSNorm(dim), RMSNorm(dim)  # across heads
    self.to_out = nn.ModuleList([nn.Linear(dim, dim)])


class WanTransformerBlock(nn.Module):

  def __init__(self, dim: int, ffn_dim: int, heads: int):
    super().__init__()
    self.scale_shift_table = nn.Parameter(torch.randn(1, 6, dim) / dim**0.5)
    self.attn1 = WanAttention(dim, heads)
    self.attn2 = WanAttention(dim, heads)
    self.norm2 = nn.LayerNorm(dim, eps=1e-6, elementwise_affine=True)
    self.ffn = QwenFeedForward(dim, ffn_dim)
    self.cp: Optional[UlyssesGroup] = None

  def forward(self, hidden_states, encoder_hidden_states, temb, rotary_emb):
    mod = (self.scale_shift_table.to(temb.dtype) + temb)  # [B, 6, C]
    shift_msa, scale_msa, gate_msa, c_shift, c_scale, c_gate = mod.unbind(dim=1)
    # 1. self-attention over the video tokens
    a = self.attn1
    q, k, v = norm_modulate_linears(hidden_states, shift_msa, scale_msa, (a.to_q, a.to_k, a.to_v))
    o = joint_attention(((q, a.norm_q), ), ((k, a.norm_k), ), (v, ), rotary_emb, a.heads, self.cp, across_heads=True)
    hidden_states = gated_add(hidden_states, gate_msa, a.to_out[0](o))
    # 2. cross-attention to the text (local under context parallelism)
    a = self.attn2
    q = a.norm_q(a.to_q(self.norm2(hidden_states))).unflatten(-1, (a.heads, a.head_dim))
    k = a.norm_k(a.to_k(encoder_hidden_states)).unflatten(-1, (a.heads, a.head_dim))
    v = a.to_v(encoder_hidden_states).unflatten(-1, (a.heads, a.head_dim))
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2)
    hidden_states = hidden_states + a.to_out[0](o.flatten(2))
    # 3. feed-forward
    act = gelu_in_product()
    (h, ) = norm_modulate_linears(hidden_states, c_shift, c_scale, (self.ffn.net[0].proj, ), gelu_last=act)
    return gated_add(hidden_states, c_gate, gelu_linear(h, self.ffn.net[2], activated=act))


class WanTransformer3DModel(ContextParallelMixin, nn.Module):
  _repeated_blocks = ["WanTransformerBlock"]

  def __init__(self, num_layers: int = 40, dim: int = 5120, heads: int = 40, ffn_dim: int = 13824,
               in_channels: int = 64, text_dim: int = 4096, axes_dims_rope: Tuple[int, int, int] = (44, 42, 42),
               time_scale: float = 1000.0, modulation_init_std: Optional[float] = None):
    super().__init__()
    self.dim = dim
    self.axes_dims_rope = axes_dims_rope
    self.time_scale = time_scale
    self.patch_embedding = nn.Linear(in_channels, dim)  # the 1 x 2 x 2 patch convolution on pre-patchified tokens
    self.time_embedder = TimestepMLP(256, dim)
    self.time_proj = nn.Linear(dim, 6 * dim)
    self.text_embedder = nn.Sequential(nn.Linear(text_dim, dim), nn.GELU(approximate="tanh"), nn.Linear(dim, dim))
    self.blocks = nn.ModuleList([WanTransformerBlock(dim, ffn_dim, heads) for _ in range(num_layers)])
    self.scale_shift_table = nn.Parameter(torch.randn(1, 2, dim) / dim**0.5)
    self.proj_out = nn.Linear(dim, in_channels)
    self._rope_cache = RopeCache()
    if modulation_init_std is not None:  # see FluxTransformer2DModel: makes consecutive steps similar
      nn.init.normal_(self.time_proj.weight, std=modulation_init_std)
      nn.init.zeros_(self.time_proj.bias)

  def _cp_blocks(self):
    return list(self.blocks)

  def forward(self, hidden_states, encoder_hidden_states, timestep, video_ids):
    n_tokens = hidden_states.shape[1]
    hidden_states, video_ids = self.cp_shard(hidden_states, 1), self.cp_shard(video_ids, 0)
    dt = hidden_states.dtype
    hidden_states = self.patch_embedding(hidden_states)
    temb = self.time_embedder(timestep_embedding(timestep * self.time_scale, 256).to(dt))
    temb6 = self.time_proj(F.silu(temb)).unflatten(1, (6, -1))
    encoder_hidden_states = self.text_embedder(encoder_hidden_states)
    rope = self._rope_cache.get((video_ids, ), self.axes_dims_rope, dt)
    for block in self.blocks:
      hidden_states = block(hidden_states, encoder_hidden_states, temb6, rope)
    shift, scale = (self.scale_shift_table.to(dt) + temb[:, None]).unbind(dim=1)
    out = self.proj_out(norm_modulate(hidden_states, shift, scale))
    return self.cp_gather(out, 1, n_tokens)

  # ---- synthetic inputs: 81 frames at 1280 x 720 -> 21 x 45 x 80 = 75600 latent tokens + 512 text tokens
  @staticmethod
  def example_inputs(batch: int = 1, frames: int = 21, height: int = 45, width: int = 80, text_tokens: int = 512,
                     device="cuda", dtype=torch.bfloat16, seed: int = 0, in_channels: int = 64, text_dim: int = 4096):
    g = torch.Generator().manual_seed(seed)
    ids = torch.stack(torch.meshgrid(torch.arange(frames), torch.arange(height), torch.arange(width), indexing="ij"),
                      dim=-1).reshape(-1, 3).float()
    return dict(
      hidden_states=torch.randn(batch, frames * height * width, in_channels, generator=g).to(device=device, dtype=dtype),
      encoder_hidden_states=torch.randn(batch, text_tokens, text_dim, generator=g).to(device=device, dtype=dtype),
      video_ids=ids.to(device))


@BlockAdapterRegister.register("Wan", separate_cfg=True)
def wan_adapter(pipe_or_transformer, **kwargs) -> BlockAdapter:
  transformer = pipe_or_transformer if isinstance(pipe_or_transformer, nn.Module) else pipe_or_transformer.transformer
  pipe = None if isinstance(pipe_or_transformer, nn.Module) else pipe_or_transformer
  return BlockAdapter(pipe=pipe, transformer=transformer, blocks=transformer.blocks, blocks_name="blocks",
                      forward_pattern=ForwardPattern.Pattern_2, check_forward_pattern=False, has_separate_cfg=True,
                      **kwargs)
