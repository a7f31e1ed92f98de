"""Modules with the ATTRIBUTE LAYOUT of the public diffusers FLUX blocks and eager forwards of the same data flow,
written for the tests: they stand for "a model this package did not write" when the producer-fused block forwards
are installed by `quantize`.  Calling convention of both blocks: the one the reference patches FLUX to
(src/cache_dit/caching/patch_functors/functor_flux.py:48-80): `(hidden_states, encoder_hidden_states, temb,
image_rotary_emb, joint_attention_kwargs=None) -> (encoder_hidden_states, hidden_states)`."""
import torch
import torch.nn.functional as F
from torch import nn


def _rope(x, rope):  # x [B, S, H, D]; rotate consecutive pairs (cos / sin repeated per pair)
  cos, sin = rope[0][None, :, None, :].to(x.dtype), rope[1][None, :, None, :].to(x.dtype)
  x1, x2 = x.unflatten(-1, (-1, 2)).unbind(-1)
  return x * cos + torch.stack([-x2, x1], dim=-1).flatten(-2) * sin


class AdaLayerNormZero(nn.Module):

  def __init__(self, dim, chunks):
    super().__init__()
    self.chunks = chunks
    self.silu = nn.SiLU()
    self.linear = nn.Linear(dim, chunks * dim)
    self.norm = nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6)

  def forward(self, x, emb):
    parts = self.linear(self.silu(emb)).chunk(self.chunks, dim=1)
    x = self.norm(x) * (1 + parts[1][:, None]) + parts[0][:, None]
    return (x, ) + tuple(parts[2:])


class GELU(nn.Module):

  def __init__(self, dim, inner):
    super().__init__()
    self.proj = nn.Linear(dim, inner)

  def forward(self, x):
    return F.gelu(self.proj(x), approximate="tanh")


class FeedForward(nn.Module):

  def __init__(self, dim, inner):
    super().__init__()
    self.net = nn.ModuleList([GELU(dim, inner), nn.Dropout(0.0), nn.Linear(inner, dim)])

  def forward(self, x):
    for m in self.net:
      x = m(x)
    return x


class Attention(nn.Module):

  def __init__(self, dim, heads, joint):
    super().__init__()
    self.heads, self.head_dim = heads, dim // heads
    self.to_q, self.to_k, self.to_v = nn.Linear(dim, dim), nn.Linear(dim, dim), nn.Linear(dim, dim)
    self.norm_q, self.norm_k = nn.RMSNorm(self.head_dim, eps=1e-6), nn.RMSNorm(self.head_dim, eps=1e-6)
    if joint:
      self.add_q_proj, self.add_k_proj, self.add_v_proj = nn.Linear(dim, dim), nn.Linear(dim, dim), nn.Linear(dim, dim)
      self.norm_added_q, self.norm_added_k = nn.RMSNorm(self.head_dim, eps=1e-6), nn.RMSNorm(self.head_dim, eps=1e-6)
      self.to_out = nn.ModuleList([nn.Linear(dim, dim), nn.Dropout(0.0)])
      self.to_add_out = nn.Linear(dim, dim)

  def forward(self, hidden_states, encoder_hidden_states=None, image_rotary_emb=None):
    h = lambda t: t.unflatten(-1, (self.heads, self.head_dim))
    q, k, v = self.norm_q(h(self.to_q(hidden_states))), self.norm_k(h(self.to_k(hidden_states))), h(self.to_v(hidden_states))
    if encoder_hidden_states is not None:
      cq = self.norm_added_q(h(self.add_q_proj(encoder_hidden_states)))
      ck = self.norm_added_k(h(self.add_k_proj(encoder_hidden_states)))
      cv = h(self.add_v_proj(encoder_hidden_states))
      q, k, v = torch.cat([cq, q], dim=1), torch.cat([ck, k], dim=1), torch.cat([cv, v], dim=1)
    q, k = _rope(q, image_rotary_emb), _rope(k, image_rotary_emb)
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)).transpose(1, 2).flatten(2)
    if encoder_hidden_states is None:
      return o
    n_txt = encoder_hidden_states.shape[1]
    return self.to_out[0](o[:, n_txt:]), self.to_add_out(o[:, :n_txt])


class FluxTransformerBlock(nn.Module):

  def __init__(self, dim, heads):
    super().__init__()
    self.norm1, self.norm1_context = AdaLayerNormZero(dim, 6), AdaLayerNormZero(dim, 6)
    self.attn = Attention(dim, heads, joint=True)
    self.norm2 = nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6)
    self.ff = FeedForward(dim, 4 * dim)
    self.norm2_context = nn.LayerNorm(dim, elementwise_affine=False, eps=1e-6)
    self.ff_context = FeedForward(dim, 4 * dim)

  def forward(self, hidden_states, encoder_hidden_states, temb, image_rotary_emb=None, joint_attention_kwargs=None):
    nh, gate, shift_mlp, scale_mlp, gate_mlp = self.norm1(hidden_states, emb=temb)
    ne, c_gate, c_shift_mlp, c_scale_mlp, c_gate_mlp = self.norm1_context(encoder_hidden_states, emb=temb)
    a, ca = self.attn(hidden_states=nh, encoder_hidden_states=ne, image_rotary_emb=image_rotary_emb)
    hidden_states = hidden_states + gate.unsqueeze(1) * a
    nh = self.norm2(hidden_states) * (1 + scale_mlp[:, None]) + shift_mlp[:, None]
    hidden_states = hidden_states + gate_mlp.unsqueeze(1) * self.ff(nh)
    encoder_hidden_states = encoder_hidden_states + c_gate.unsqueeze(1) * ca
    ne = self.norm2_context(encoder_hidden_states) * (1 + c_scale_mlp[:, None]) + c_shift_mlp[:, None]
    encoder_hidden_states = encoder_hidden_states + c_gate_mlp.unsqueeze(1) * self.ff_context(ne)
    return encoder_hidden_states, hidden_states


class FluxSingleTransformerBlock(nn.Module):

  def __init__(self, dim, heads):
    super().__init__()
    self.norm = AdaLayerNormZero(dim, 3)
    self.proj_mlp = nn.Linear(dim, 4 * dim)
    self.act_mlp = nn.GELU(approximate="tanh")
    self.attn = Attention(dim, heads, joint=False)
    self.proj_out = nn.Linear(5 * dim, dim)

  def forward(self, hidden_states, encoder_hidden_states, temb, image_rotary_emb=None, joint_attention_kwargs=None):
    n_txt = encoder_hidden_states.shape[1]
    x = torch.cat([encoder_hidden_states, hidden_states], dim=1)
    nx, gate = self.norm(x, emb=temb)
    mlp = self.act_mlp(self.proj_mlp(nx))
    o = self.attn(hidden_states=nx, image_rotary_emb=image_rotary_emb)
    x = x + gate.unsqueeze(1) * self.proj_out(torch.cat([o, mlp], dim=2))
    return x[:, :n_txt], x[:, n_txt:]


class TinyFlux(nn.Module):
  _repeated_blocks = ["FluxTransformerBlock", "FluxSingleTransformerBlock"]

  def __init__(self, dim=256, heads=2, double=2, single=2):
    super().__init__()
    self.transformer_blocks = nn.ModuleList([FluxTransformerBlock(dim, heads) for _ in range(double)])
    self.single_transformer_blocks = nn.ModuleList([FluxSingleTransformerBlock(dim, heads) for _ in range(single)])

  def forward(self, hidden_states, encoder_hidden_states, temb, image_rotary_emb):
    for blk in list(self.transformer_blocks) + list(self.single_transformer_blocks):
      encoder_hidden_states, hidden_states = blk(hidden_states, encoder_hidden_states, temb, image_rotary_emb)
    return encoder_hidden_states, hidden_states
