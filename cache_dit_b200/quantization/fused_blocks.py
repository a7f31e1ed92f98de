"""Producer-fused forwards for transformer blocks with the attribute layout of diffusers' FLUX blocks.

`quantize()` swaps `nn.Linear` layers for `Float8RowwiseLinear`, whose own `forward` has to quantize
whatever bf16 tensor it is handed: the adaLN-modulated LayerNorm, the tanh-GELU and the concatenation in
front of it have then already been written to memory by eager PyTorch ops.  For blocks whose attributes are
laid out like the public diffusers FLUX blocks - the layout the reference patches and adapts
(src/cache_dit/caching/patch_functors/functor_flux.py:23-80, block_adapters/adapters.py:40-103):

  double stream   norm1.linear, norm1_context.linear, attn.{to_q, to_k, to_v, add_q_proj, add_k_proj, add_v_proj,
                  norm_q, norm_k, norm_added_q, norm_added_k, to_out[0], to_add_out}, ff.net[0].proj, ff.net[2],
                  ff_context.net[0].proj, ff_context.net[2]
  single stream   norm.linear, proj_mlp, attn.{to_q, to_k, to_v, norm_q, norm_k}, proj_out

this module installs block forwards that keep the reference's calling convention
`(hidden_states, encoder_hidden_states, temb, image_rotary_emb, joint_attention_kwargs=None) ->
(encoder_hidden_states, hidden_states)` (functor_flux.py:48-80) and run the fused path: LayerNorm + modulation
inside the activation-quantization kernel, q/k/v (+ MLP-in) as one product, QK RMSNorm + rotary embedding +
concatenation as one kernel, `[attention | GELU(mlp)]` quantized from its two sources, gated residual adds as one
kernel, the two streams of a double block sharing launches.  A block is only touched when every linear the
fused path needs is FP8 and its norms look as expected; anything else keeps its own forward.
"""
from __future__ import annotations

import logging
import os
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from .linear import Float8RowwiseLinear

logger = logging.getLogger("cache_dit_b200")


def _get(obj, path: str):
  for part in path.split("."):
    if obj is None:
      return None
    obj = obj[int(part)] if part.isdigit() else getattr(obj, part, None)
  return obj


_DOUBLE_FP8 = ("attn.to_q", "attn.to_k", "attn.to_v", "attn.add_q_proj", "attn.add_k_proj", "attn.add_v_proj",
               "attn.to_out.0", "attn.to_add_out", "ff.net.0.proj", "ff.net.2", "ff_context.net.0.proj", "ff_context.net.2")
_DOUBLE_OTHER = ("norm1.linear", "norm1_context.linear", "attn.norm_q", "attn.norm_k", "attn.norm_added_q",
                 "attn.norm_added_k")
_SINGLE_FP8 = ("attn.to_q", "attn.to_k", "attn.to_v", "proj_mlp", "proj_out")
_SINGLE_OTHER = ("norm.linear", "attn.norm_q", "attn.norm_k")


def _plain_layernorms(block, paths) -> bool:
  """The fused LayerNorm has no affine parameters and eps 1e-6 (what the FLUX blocks use): any LayerNorm found at
  `paths` has to agree, a missing one is taken to be applied inside the modulation module in that form."""
  for p in paths:
    m = _get(block, p)
    if m is not None and (getattr(m, "elementwise_affine", False) or abs(getattr(m, "eps", 1e-6) - 1e-6) > 1e-12):
      return False
  return True


def _layout(block) -> Optional[str]:
  def ok(fp8, other):
    return all(isinstance(_get(block, p), Float8RowwiseLinear) for p in fp8) and \
        all(_get(block, p) is not None for p in other) and getattr(_get(block, "attn"), "heads", None) is not None and \
        _plain_layernorms(block, ("norm.norm", "norm1.norm", "norm1_context.norm", "norm2", "norm2_context"))
  if ok(_DOUBLE_FP8, _DOUBLE_OTHER):
    return "double"
  if ok(_SINGLE_FP8, _SINGLE_OTHER) and _get(block, "attn.add_q_proj") is None:
    return "single"
  return None


class _RopeTables:
  """(cos, sin) in the activation dtype, contiguous; converted once per distinct pair of tensors."""

  def __init__(self):
    self._key, self._value = None, None

  def get(self, rope: Tuple[torch.Tensor, torch.Tensor], dtype):
    key = (rope[0].data_ptr(), rope[1].data_ptr(), rope[0]._version, tuple(rope[0].shape), dtype)
    if key != self._key:
      self._value = (rope[0].to(dtype).contiguous(), rope[1].to(dtype).contiguous())
      self._key, self._keep = key, rope
    return self._value


_ROPE = _RopeTables()


def _modulation(linear, temb, chunks):
  return linear(F.silu(temb)).chunk(chunks, dim=-1)


def flux_double_block_forward(self, hidden_states, encoder_hidden_states, temb, image_rotary_emb=None,
                              joint_attention_kwargs=None):
  from ..synthetic.layers import (gated_add_pair, gelu_in_product, gelu_linear_pair, joint_attention, linear_pair,
                                  norm_modulate_linears_pair, shared_input_linears)
  a = self.attn
  rope = _ROPE.get(image_rotary_emb, hidden_states.dtype)
  mod, c_mod = shared_input_linears(F.silu(temb), (self.norm1.linear, self.norm1_context.linear))
  shift, scale, gate, shift_mlp, scale_mlp, gate_mlp = mod.chunk(6, dim=-1)
  c_shift, c_scale, c_gate, c_shift_mlp, c_scale_mlp, c_gate_mlp = c_mod.chunk(6, dim=-1)
  (q, k, v), (cq, ck, cv) = norm_modulate_linears_pair(
    (hidden_states, shift, scale, (a.to_q, a.to_k, a.to_v)),
    (encoder_hidden_states, c_shift, c_scale, (a.add_q_proj, a.add_k_proj, a.add_v_proj)))
  o = joint_attention(((cq, a.norm_added_q), (q, a.norm_q)), ((ck, a.norm_added_k), (k, a.norm_k)), (cv, v), rope,
                      a.heads, getattr(self, "cp", None))
  n_txt = encoder_hidden_states.shape[1]
  y, cy = linear_pair(o[:, n_txt:], a.to_out[0], o[:, :n_txt], a.to_add_out)
  hidden_states, encoder_hidden_states = gated_add_pair(hidden_states, gate, y, encoder_hidden_states, c_gate, cy)
  act = gelu_in_product()
  (h, ), (c, ) = norm_modulate_linears_pair((hidden_states, shift_mlp, scale_mlp, (self.ff.net[0].proj, )),
                                            (encoder_hidden_states, c_shift_mlp, c_scale_mlp, (self.ff_context.net[0].proj, )),
                                            gelu_last=act)
  y, cy = gelu_linear_pair(h, self.ff.net[2], c, self.ff_context.net[2], activated=act)
  hidden_states, encoder_hidden_states = gated_add_pair(hidden_states, gate_mlp, y, encoder_hidden_states, c_gate_mlp, cy)
  return encoder_hidden_states, hidden_states


def flux_single_block_forward(self, hidden_states, encoder_hidden_states, temb, image_rotary_emb=None,
                              joint_attention_kwargs=None):
  from ..synthetic.layers import (concat_gelu_linear, gated_add, gelu_in_product, join_tokens, joint_attention, norm_modulate_linears,
                                  split_tokens)
  a = self.attn
  rope = _ROPE.get(image_rotary_emb, hidden_states.dtype)
  n_txt = encoder_hidden_states.shape[1]
  x = join_tokens(encoder_hidden_states, hidden_states)
  shift, scale, gate = _modulation(self.norm.linear, temb, 3)
  act = gelu_in_product()
  q, k, v, mlp = norm_modulate_linears(x, shift, scale, (a.to_q, a.to_k, a.to_v, self.proj_mlp), gelu_last=act)
  o = joint_attention(((q, a.norm_q), ), ((k, a.norm_k), ), (v, ), rope, a.heads, getattr(self, "cp", None))
  y = concat_gelu_linear(o, mlp, self.proj_out, tail_activated=act)
  return split_tokens(gated_add(x, gate, y), n_txt)


def install_fused_block_forwards(module: torch.nn.Module) -> int:
  """Give every block under `module` that has one of the two layouts (and FP8 linears throughout) its fused
  forward.  Returns how many blocks were changed; `CACHE_DIT_B200_FUSE_BLOCKS=0` leaves everything alone."""
  if os.environ.get("CACHE_DIT_B200_FUSE_BLOCKS", "1") == "0":
    return 0
  count = 0
  for block in module.modules():
    if getattr(block, "_cdb_fused_forward", False):
      continue
    if type(block).__module__.startswith("cache_dit_b200.synthetic"):
      continue  # the in-tree stand-ins are written against the fused helpers already
    kind = _layout(block)
    if kind is None:
      continue
    fn = flux_double_block_forward if kind == "double" else flux_single_block_forward
    block._cdb_original_forward = block.forward
    block.forward = fn.__get__(block)
    block._cdb_fused_forward = True
    count += 1
  if count:
    logger.info(f"installed producer-fused forwards on {count} blocks of {module.__class__.__name__}")
  return count


def remove_fused_block_forwards(module: torch.nn.Module) -> None:
  for block in module.modules():
    if getattr(block, "_cdb_fused_forward", False):
      block.forward = block._cdb_original_forward
      del block._cdb_original_forward
      block._cdb_fused_forward = False
