"""Random-init stand-in with the architecture of Qwen-Image's transformer.

60 dual-stream MMDiT blocks, hidden 3072, 24 heads of dim 128: image and text tokens keep separate
weights (modulation, q/k/v, output projection, MLP) and attend jointly over [text; image]; QK RMSNorm
per head, rotary embedding over (16, 56, 56) axes, adaLN modulation from the timestep embedding only,
tanh-GELU MLP of ratio 4.  Layer names follow the public diffusers implementation (`img_mod.1`,
`txt_mod.1`, `attn.to_q`, `attn.add_q_proj`, `img_mlp.net.0.proj`, ...), so the FP8 name filter leaves
the modulation linears in bf16 exactly as it does on the real model ("mod" is an excluded pattern).
Blocks take `(hidden_states, encoder_hidden_states, temb, image_rotary_emb)` and return
`(encoder_hidden_states, hidden_states)`: ForwardPattern.Pattern_1, one 60-block list, separate CFG
(src/cache_dit/caching/block_adapters/adapters.py:263-271).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from ..caching.block_adapters import BlockAdapter, BlockAdapterRegister
from ..caching.forward_pattern import ForwardPattern
from .context_parallel import ContextParallelMixin
from .layers import (RMSNorm, RopeCache, TimestepMLP, UlyssesGroup, gated_add_pair, gelu_in_product, gelu_linear_pair, joint_attention,
                     linear_pair, modulation_rows, norm_modulate, norm_modulate_linears_pair, timestep_embedding)


class _GeluProj(nn.Module):

  def __init__(self, dim: int, inner: int):
    super().__init__()
    self.proj = nn.Linear(dim, inner)


class QwenFeedForward(nn.Module):
  """net.0.proj -> tanh-GELU -> net.2, the diffusers FeedForward layout."""

  def __init__(self, dim: int, inner: int):
    super().__init__()
    self.net = nn.ModuleList([_GeluProj(dim, inner), nn.Identity(), nn.Linear(inner, dim)])


class QwenJointAttention(nn.Module):

  def __init__(self, dim: int, heads: int):
    super().__init__()
    self.heads = heads
    self.head_dim = dim // heads
    self.to_q, self.to_k, self.to_v = nn.Linear(dim, dim), nn.Linear(dim, dim), nn.Linear(dim, dim)
    self.add_q_proj, self.add_k_proj, self.add_v_proj = nn.Linear(dim, dim), nn.Linear(dim, dim), nn.Linear(dim, dim)
    self.norm_q, self.norm_k = RMSNorm(self.head_dim), RMSNorm(self.head_dim)
    self.norm_added_q, self.norm_added_k = RMSNorm(self.head_dim), RMSNorm(self.head_dim)
    self.to_out = nn.ModuleList([nn.Linear(dim, dim)])
    self.to_add_out = nn.Linear(dim, dim)


class QwenImageTransformerBlock(nn.Module):

  def __init__(self, dim: int, heads: int, mlp_ratio: float = 4.0):
    super().__init__()
    self.img_mod = nn.Sequential(nn.SiLU(), nn.Linear(dim, 6 * dim))
    self.txt_mod = nn.Sequential(nn.SiLU(), nn.Linear(dim, 6 * dim))
    self.attn = QwenJointAttention(dim, heads)
    self.img_mlp = QwenFeedForward(dim, int(dim * mlp_ratio))
    self.txt_mlp = QwenFeedForward(dim, int(dim * mlp_ratio))
    self.cp: Optional[UlyssesGroup] = None

  def forward(self, hidden_states, encoder_hidden_states, temb, image_rotary_emb):
    a = self.attn
    bank = getattr(self, "mod_bank", None)
    if bank is not None:  # computed once per call for all blocks, column-sharded over the ranks
      img, txt = bank.outputs((self.img_mod[1], self.txt_mod[1]))
    else:
      img, txt = modulation_rows(temb, self.img_mod[1]), modulation_rows(temb, self.txt_mod[1])
    shift1, scale1, gate1, shift2, scale2, gate2 = img.chunk(6, dim=-1)
    c_shift1, c_scale1, c_gate1, c_shift2, c_scale2, c_gate2 = txt.chunk(6, dim=-1)
    (q, k, v), (cq, ck, cv) = norm_modulate_linears_pair(
      (hidden_states, shift1, scale1, (a.to_q, a.to_k, a.to_v)),
      (encoder_hidden_states, c_shift1, c_scale1, (a.add_q_proj, a.add_k_proj, a.add_v_proj)))
    o = joint_attention(((cq, a.norm_added_q), (q, a.norm_q)), ((ck, a.norm_added_k), (k, a.norm_k)), (cv, v),
                        image_rotary_emb, a.heads, self.cp)
    n_txt = encoder_hidden_states.shape[1]
    y, cy = linear_pair(o[:, n_txt:], a.to_out[0], o[:, :n_txt], a.to_add_out)
    hidden_states, encoder_hidden_states = gated_add_pair(hidden_states, gate1, y, encoder_hidden_states, c_gate1, cy)
    act = gelu_in_product()
    (h, ), (c, ) = norm_modulate_linears_pair((hidden_states, shift2, scale2, (self.img_mlp.net[0].proj, )),
                                              (encoder_hidden_states, c_shift2, c_scale2, (self.txt_mlp.net[0].proj, )),
                                              gelu_last=act)
    y, cy = gelu_linear_pair(h, self.img_mlp.net[2], c, self.txt_mlp.net[2], activated=act)
    hidden_states, encoder_hidden_states = gated_add_pair(hidden_states, gate2, y, encoder_hidden_states, c_gate2, cy)
    return encoder_hidden_states, hidden_states


class QwenImageTransformer2DModel(ContextParallelMixin, nn.Module):
  _repeated_blocks = ["QwenImageTransformerBlock"]

  def __init__(self, num_layers: int = 60, dim: int = 3072, heads: int = 24, in_channels: int = 64,
               joint_attention_dim: int = 3584, axes_dims_rope: Tuple[int, int, int] = (16, 56, 56),
               time_scale: float = 1000.0, modulation_init_std: Optional[float] = None):
    super().__init__()
    self.dim = dim
    self.axes_dims_rope = axes_dims_rope
    self.time_scale = time_scale
    self.img_in = nn.Linear(in_channels, dim)
    self.txt_norm = RMSNorm(joint_attention_dim)
    self.txt_in = nn.Linear(joint_attention_dim, dim)
    self.time_text_embed = TimestepMLP(256, dim)
    self.transformer_blocks = nn.ModuleList([QwenImageTransformerBlock(dim, heads) for _ in range(num_layers)])
    self.norm_out_linear = nn.Linear(dim, 2 * dim)
    self.proj_out = nn.Linear(dim, in_channels)
    self._rope_cache = RopeCache()
    if modulation_init_std is not None:  # see FluxTransformer2DModel: makes consecutive steps similar
      for block in self.transformer_blocks:
        for mod in (block.img_mod[1], block.txt_mod[1]):
          nn.init.normal_(mod.weight, std=modulation_init_std)
          nn.init.zeros_(mod.bias)

  def _cp_blocks(self):
    return list(self.transformer_blocks)

  def _modulation_groups(self, blocks):
    return [(b.img_mod[1], b.txt_mod[1]) for b in blocks]

  def _runs_blocks_itself(self) -> bool:
    return not self.is_cache_runner_list(self.transformer_blocks)

  def forward(self, hidden_states, encoder_hidden_states, timestep, img_ids, txt_ids):
    n_img = hidden_states.shape[1]
    hidden_states, encoder_hidden_states = self.cp_shard(hidden_states, 1), self.cp_shard(encoder_hidden_states, 1)
    img_ids, txt_ids = self.cp_shard(img_ids, 0), self.cp_shard(txt_ids, 0)
    dt = hidden_states.dtype
    hidden_states = self.img_in(hidden_states)
    encoder_hidden_states = self.txt_in(self.txt_norm(encoder_hidden_states))
    temb = self.time_text_embed(timestep_embedding(timestep * self.time_scale, 256).to(dt))
    self.modulation_for_call(temb)
    rope = self._rope_cache.get((txt_ids, img_ids), self.axes_dims_rope, dt)
    for block in self.transformer_blocks:
      encoder_hidden_states, hidden_states = block(hidden_states, encoder_hidden_states, temb, rope)
    scale, shift = self.norm_out_linear(F.silu(temb)).chunk(2, dim=-1)
    out = self.proj_out(norm_modulate(hidden_states, shift, scale))
    return self.cp_gather(out, 1, n_img)

  # ---- synthetic inputs of the 1328 x 1328 configuration: 83 x 83 = 6889 image + 256 text tokens
  @staticmethod
  def example_inputs(batch: int = 1, height: int = 1328, width: int = 1328, text_tokens: int = 256,
                     device="cuda", dtype=torch.bfloat16, seed: int = 0, in_channels: int = 64,
                     joint_attention_dim: int = 3584):
    g = torch.Generator().manual_seed(seed)
    gh, gw = height // 16, width // 16
    img_ids = torch.zeros(gh, gw, 3)
    img_ids[..., 1] = torch.arange(gh)[:, None]
    img_ids[..., 2] = torch.arange(gw)[None, :]
    txt_ids = torch.zeros(text_tokens, 3)
    txt_ids[:, 1] = txt_ids[:, 2] = max(gh, gw) + torch.arange(text_tokens)  # text continues the diagonal
    return dict(
      hidden_states=torch.randn(batch, gh * gw, in_channels, generator=g).to(device=device, dtype=dtype),
      encoder_hidden_states=torch.randn(batch, text_tokens, joint_attention_dim, generator=g).to(device=device, dtype=dtype),
      img_ids=img_ids.reshape(-1, 3).to(device), txt_ids=txt_ids.to(device))


@BlockAdapterRegister.register("QwenImage", separate_cfg=True)
def qwen_image_adapter(pipe_or_transformer, **kwargs) -> BlockAdapter:
  transformer = pipe_or_transformer if isinstance(pipe_or_transformer, nn.Module) else pipe_or_transformer.transformer
  pipe = None if isinstance(pipe_or_transformer, nn.Module) else pipe_or_transformer
  return BlockAdapter(pipe=pipe, transformer=transformer, blocks=transformer.transformer_blocks,
                      blocks_name="transformer_blocks", forward_pattern=ForwardPattern.Pattern_1,
                      check_forward_pattern=False, has_separate_cfg=True, **kwargs)
