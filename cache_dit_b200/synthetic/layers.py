"""Building blocks shared by the random-init DiT stand-ins (FLUX-, Qwen-Image-, Wan-shape).

These modules exist so the hot path can be exercised and timed without model weights: same layer
shapes, same data flow, random parameters.  Where a linear layer has been swapped for
`Float8RowwiseLinear`, the producer (adaLN-modulated LayerNorm, tanh-GELU) is fused into the
activation-quantization kernel and the quantized activations are shared by all linears that read
them (q/k/v), so the bf16 intermediate is never written.
"""
from __future__ import annotations

import math
import os
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F
from torch import nn

from .. import _native
from ..quantization.linear import (Float8RowwiseLinear, _members_share_storage, fused_group, grouped_forward_quantized,
                                   quantize_rows_fused, quantize_rows_fused_pair)


def _all_fp8(linears: Sequence[nn.Module]) -> bool:
  return all(isinstance(l, Float8RowwiseLinear) for l in linears)


def gelu_in_product() -> bool:
  """Whether an MLP-in projection applies the MLP's tanh-GELU in its own epilogue (default), so that the
  quantization in front of the MLP-out projection only concatenates / quantizes.
  CACHE_DIT_B200_GELU_IN_PRODUCT=0 keeps the activation in that quantization kernel."""
  return os.environ.get("CACHE_DIT_B200_GELU_IN_PRODUCT", "1") != "0"


def norm_modulate_linears(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor,
                          linears: Sequence[nn.Module], eps: float = 1e-6, gelu_last: bool = False) -> List[torch.Tensor]:
  """[lin(LayerNorm(x) * (1 + scale) + shift) for lin in linears]; shift / scale are [B, C].
  `gelu_last`: the last output is returned as gelu_tanh(lin(...)) (an MLP-in projection)."""
  if _all_fp8(linears) and x.is_cuda:
    # shift / scale are column slices of one modulation matrix: passed as strided views
    a_q, a_scale, lead = quantize_rows_fused(x, _native.PRE_LAYERNORM_MOD, shift, scale, eps)
    if len(linears) > 1:  # one GEMM over the concatenated output rows
      return list(fused_group(linears).forward_quantized(a_q, a_scale, lead, gelu_last))
    return [linears[0].forward_quantized(a_q, a_scale, lead, gelu_last)]
  y = F.layer_norm(x, (x.shape[-1], ), eps=eps) * (1 + scale[:, None]) + shift[:, None]
  outs = [l(y) for l in linears]
  if gelu_last:
    outs[-1] = F.gelu(outs[-1], approximate="tanh")
  return outs


# ---- two streams at once -----------------------------------------------------------------------------
# A double-stream block runs every layer twice: on the image tokens and, with other weights, on the much
# shorter text sequence.  The pair helpers quantize both activations and run both products in ONE GEMM
# launch, where the text product's tiles ride in the tail wave of the image product.
def _pair_ready(xa, xb, linears) -> bool:
  return xa.is_cuda and xb.is_cuda and _all_fp8(linears)


def norm_modulate_linears_pair(a, b, eps: float = 1e-6, gelu_last: bool = False):
  """(x, shift, scale, linears) for each stream -> (outputs of stream a, outputs of stream b); `gelu_last` as in
  `norm_modulate_linears`, for both streams."""
  (xa, sha, sca, la), (xb, shb, scb, lb) = a, b
  if not _pair_ready(xa, xb, tuple(la) + tuple(lb)):
    return (norm_modulate_linears(xa, sha, sca, la, eps, gelu_last),
            norm_modulate_linears(xb, shb, scb, lb, eps, gelu_last))
  qa, qb = quantize_rows_fused_pair(xa, xb, _native.PRE_LAYERNORM_MOD, (sha, sca), (shb, scb), eps)
  items = [(fused_group(lin) if len(lin) > 1 else lin[0], *triple) for lin, triple in ((la, qa), (lb, qb))]
  ra, rb = grouped_forward_quantized(items, gelu_last)
  as_list = lambda r: list(r) if isinstance(r, (tuple, list)) else [r]
  return as_list(ra), as_list(rb)


def linear_pair(xa, lina, xb, linb):
  """(lina(xa), linb(xb)) with one GEMM launch."""
  if not _pair_ready(xa, xb, (lina, linb)):
    return lina(xa), linb(xb)
  qa, qb = quantize_rows_fused_pair(xa, xb, _native.PRE_NONE)
  ra, rb = grouped_forward_quantized([(lina, *qa), (linb, *qb)])
  return ra, rb


def gelu_linear_pair(xa, lina, xb, linb, activated: bool = False):
  """(lina(gelu_tanh(xa)), linb(gelu_tanh(xb))) with one GEMM launch.  `activated`: xa and xb already hold the
  activated values (their producer applied the GELU)."""
  if not _pair_ready(xa, xb, (lina, linb)):
    return gelu_linear(xa, lina, activated), gelu_linear(xb, linb, activated)
  qa, qb = quantize_rows_fused_pair(xa, xb, _native.PRE_NONE if activated else _native.PRE_GELU_TANH)
  ra, rb = grouped_forward_quantized([(lina, *qa), (linb, *qb)])
  return ra, rb


def shared_input_linears(x: torch.Tensor, linears: Sequence[nn.Module]) -> List[torch.Tensor]:
  """[lin(x) for lin in linears]; FP8 linears share one quantization of x and one product."""
  if _all_fp8(linears) and x.is_cuda and len(linears) > 1:
    a_q, a_scale = linears[0].quantize_input(x)
    return list(fused_group(linears).forward_quantized(a_q, a_scale, x.shape[:-1]))
  return [lin(x) for lin in linears]


def norm_modulate(x: torch.Tensor, shift: torch.Tensor, scale: torch.Tensor, eps: float = 1e-6):
  return F.layer_norm(x, (x.shape[-1], ), eps=eps) * (1 + scale[:, None]) + shift[:, None]


def gelu_linear(x: torch.Tensor, linear: nn.Module, activated: bool = False) -> torch.Tensor:
  """linear(gelu_tanh(x)); with `activated`, x already holds gelu_tanh(...)."""
  if isinstance(linear, Float8RowwiseLinear) and x.is_cuda:
    a_q, a_scale, lead = quantize_rows_fused(x, _native.PRE_NONE if activated else _native.PRE_GELU_TANH)
    return linear.forward_quantized(a_q, a_scale, lead)
  return linear(x if activated else F.gelu(x, approximate="tanh"))


def concat_gelu_linear(head: torch.Tensor, tail: torch.Tensor, linear: nn.Module,
                       tail_activated: bool = False) -> torch.Tensor:
  """linear(cat([head, gelu_tanh(tail)], dim=-1)): the output projection of a parallel attention + MLP
  block.  With an FP8 linear neither the activated MLP branch nor the concatenation is written.
  `tail_activated`: tail already holds gelu_tanh(...)."""
  if isinstance(linear, Float8RowwiseLinear) and head.is_cuda:
    h2, t2 = head.reshape(-1, head.shape[-1]), tail.reshape(-1, tail.shape[-1])
    a_q = torch.empty((h2.shape[0], h2.shape[1] + t2.shape[1]), dtype=torch.float8_e4m3fn, device=head.device)
    a_scale = torch.empty(h2.shape[0], dtype=torch.float32, device=head.device)
    _native.fp8_quant_rows_concat_gelu(h2, t2, a_q, a_scale, tail_activated)
    return linear.forward_quantized(a_q, a_scale, head.shape[:-1])
  return linear(torch.cat([head, tail if tail_activated else F.gelu(tail, approximate="tanh")], dim=-1))


def modulation_rows(temb: torch.Tensor, linear: nn.Module) -> torch.Tensor:
  """linear(SiLU(temb)) for the few rows of a timestep embedding.  A bf16 `nn.Linear` on the GPU goes through the
  weight-streaming kernel (`cdb_bf16_gemv`), whose per-column arithmetic is what `ModulationBank` reproduces when
  it shards the columns over the ranks; everything else is the eager call."""
  x = F.silu(temb)
  if type(linear) is nn.Linear and x.is_cuda and x.dtype == torch.bfloat16 and linear.weight.dtype == torch.bfloat16 \
      and x.dim() == 2 and x.shape[0] <= 4 and x.shape[0] * x.shape[1] * 4 <= 48 * 1024 and x.shape[1] % 8 == 0 \
      and linear.weight.is_contiguous():
    out = torch.empty((x.shape[0], linear.out_features), dtype=torch.bfloat16, device=x.device)
    _native.bf16_gemv(x if x.stride(1) == 1 else x.contiguous(), linear.weight, linear.bias, out)
    return out
  return linear(x)


class ModulationBank:
  """Every adaLN modulation projection of a model as ONE weight-streaming product per call, column-sharded over
  the ranks of a context-parallel group.

  The projections read only SiLU(temb), which is known when a call starts and is the same on every rank, so under
  context parallelism each rank would stream all of their weights (2.1 GB of FP8 for the FLUX shape, 13.6 GB of
  bf16 for the Qwen-Image shape: the one part of a step that does not shrink with the number of GPUs).  Here rank
  r computes its 1/W of the columns of the blocks that are about to run (all of them without a cache runner;
  with one, the first blocks at the start of a call and the rest only when the step turns out to be computed) and
  one all-gather hands every rank the whole vector; the blocks then take views of it.  Members are either all FP8 linears (the M <= 4 path of the
  FP8 product) or all bf16 `nn.Linear` (`cdb_bf16_gemv`); both kernels compute a column in a fixed order that
  does not depend on the slice, so results equal the per-block products bit for bit.
  The output lives in one buffer that is overwritten every call, so captured block graphs read it in place."""

  def __init__(self, groups: Sequence[Sequence[nn.Module]], group=None):
    import torch.distributed as dist
    self.group = group
    self.world = dist.get_world_size(group)
    self.rank = dist.get_rank(group)
    self.linears = [l for g in groups for l in g]
    self.fp8 = _all_fp8(self.linears)
    if self.fp8:
      self.fused = fused_group(self.linears)
      self.cols = self.fused.out_features
    else:
      if not all(type(l) is nn.Linear and l.weight.dtype == torch.bfloat16 for l in self.linears):
        raise ValueError("a modulation bank holds FP8 linears or bf16 nn.Linear layers, not a mixture")
      self.weight = torch.cat([l.weight.detach() for l in self.linears], dim=0)  # [cols, K]; members become views
      has_bias = [l.bias is not None for l in self.linears]
      self.bias = torch.cat([l.bias.detach() if hb else torch.zeros(l.out_features, dtype=torch.bfloat16, device=self.weight.device)
                             for l, hb in zip(self.linears, has_bias)]) if any(has_bias) else None
      self.cols = self.weight.shape[0]
    if any(l.out_features % 8 for l in self.linears):
      raise ValueError("modulation widths must be multiples of 8")
    self.offsets = {}
    self.group_cols = []  # per group (block): [first column, last column + 1)
    start = 0
    for g in groups:
      width = sum(l.out_features for l in g)
      self.group_cols.append((start, start + width))
      start += width
    start = 0
    for i, l in enumerate(self.linears):
      self.offsets[id(l)] = (start, l.out_features)
      if not self.fp8:  # the members keep working on their own, on the shared storage
        l.weight = nn.Parameter(self.weight[start:start + l.out_features], requires_grad=False)
        if has_bias[i]:
          l.bias = nn.Parameter(self.bias[start:start + l.out_features], requires_grad=False)
      start += l.out_features
    self._out = None

  def still_valid(self) -> bool:
    """False once a member's weight no longer lives in the shared storage (the model was moved or reloaded)."""
    if self.fp8:
      return _members_share_storage(self.fused, self.linears)
    base = self.weight.data_ptr()
    k = self.weight.shape[1] * 2
    return all(l.weight.device == self.weight.device and l.weight.data_ptr() == base + self.offsets[id(l)][0] * k
               for l in self.linears)

  def begin_call(self, temb: torch.Tensor) -> None:
    """Remember this call's SiLU(temb) (quantized once for FP8 members); nothing is computed yet."""
    x = F.silu(temb)
    self._x = x if x.stride(1) == 1 else x.contiguous()
    if self.fp8:
      self._a_q, self._a_scale = self.linears[0].quantize_input(self._x)
    if self._out is None or self._out.shape[0] != x.shape[0]:
      self._out = torch.empty((x.shape[0], self.cols), dtype=torch.bfloat16, device=x.device)

  def prepare(self, first: int, last: int) -> None:
    """Compute the vectors of groups [first, last) (one group per block): this rank's share of their columns as
    one product, then one all-gather.  Called before the blocks run - with a cache runner once for the first
    blocks of a call and, only when the step is computed, once for the rest."""
    import torch.distributed as dist
    c0, c1 = self.group_cols[first][0], self.group_cols[last - 1][1]
    width = c1 - c0
    batch = self._x.shape[0]
    sharded = self.world > 1 and width % (self.world * 8) == 0
    per = width // self.world if sharded else width
    lo = c0 + (self.rank * per if sharded else 0)
    local = torch.empty((batch, per), dtype=torch.bfloat16, device=self._x.device)
    if self.fp8:
      f = self.fused
      _native.fp8_gemm_rowscaled(self._a_q, self._a_scale, f.weight_q[lo:lo + per], f.weight_scale[lo:lo + per],
                                 None if f.bias is None else f.bias[lo:lo + per], local)
    else:
      _native.bf16_gemv(self._x, self.weight[lo:lo + per], None if self.bias is None else self.bias[lo:lo + per], local)
    if sharded:
      gathered = torch.empty((self.world, batch, per), dtype=torch.bfloat16, device=local.device)
      dist.all_gather_into_tensor(gathered, local, group=self.group)
      self._out[:, c0:c1].unflatten(1, (self.world, per)).copy_(gathered.permute(1, 0, 2))
    else:
      self._out[:, c0:c1].copy_(local)

  def compute(self, temb: torch.Tensor) -> None:
    """All groups at once (a model that runs without a cache runner)."""
    self.begin_call(temb)
    self.prepare(0, len(self.group_cols))

  def outputs(self, linears: Sequence[nn.Module]) -> List[torch.Tensor]:
    """Views [batch, out_features] of the gathered vector for the given member linears."""
    return [self._out[:, o:o + n] for o, n in (self.offsets[id(l)] for l in linears)]


class RMSNorm(nn.Module):

  def __init__(self, dim: int, eps: float = 1e-6):
    super().__init__()
    self.eps = eps
    self.weight = nn.Parameter(torch.ones(dim))

  def forward(self, x):
    return F.rms_norm(x, (x.shape[-1], ), self.weight, self.eps)


def timestep_embedding(t: torch.Tensor, dim: int, max_period: float = 10000.0) -> torch.Tensor:
  half = dim // 2
  freqs = torch.exp(-math.log(max_period) * torch.arange(half, device=t.device, dtype=torch.float32) / half)
  args = t.float()[:, None] * freqs[None]
  return torch.cat([torch.cos(args), torch.sin(args)], dim=-1)


class TimestepMLP(nn.Module):

  def __init__(self, in_dim: int, dim: int):
    super().__init__()
    self.linear_1 = nn.Linear(in_dim, dim)
    self.linear_2 = nn.Linear(dim, dim)

  def forward(self, x):
    return self.linear_2(F.silu(self.linear_1(x)))


def rope_frequencies(ids: torch.Tensor, axes_dim: Sequence[int], theta: float = 10000.0):
  """ids [S, n_axes] -> (cos, sin) [S, sum(axes_dim)] with each frequency repeated for its pair."""
  cos, sin = [], []
  for i, d in enumerate(axes_dim):
    freqs = 1.0 / (theta**(torch.arange(0, d, 2, device=ids.device, dtype=torch.float32) / d))
    ang = ids[:, i].float()[:, None] * freqs[None]
    cos.append(torch.cos(ang).repeat_interleave(2, dim=-1))
    sin.append(torch.sin(ang).repeat_interleave(2, dim=-1))
  return torch.cat(cos, dim=-1), torch.cat(sin, dim=-1)


def apply_rope(x: torch.Tensor, rope: Tuple[torch.Tensor, torch.Tensor]) -> torch.Tensor:
  """x [B, S, H, D]; rotate consecutive pairs."""
  cos, sin = rope
  cos, sin = cos[None, :, None, :].to(x.dtype), sin[None, :, None, :].to(x.dtype)
  x1, x2 = x.unflatten(-1, (-1, 2)).unbind(-1)
  rot = torch.stack([-x2, x1], dim=-1).flatten(-2)
  return x * cos + rot * sin


def rope_tables(rope: Tuple[torch.Tensor, torch.Tensor], dtype) -> Tuple[torch.Tensor, torch.Tensor]:
  """The (cos, sin) tables in the activation dtype, contiguous: cast once per forward, not per block."""
  return rope[0].to(dtype).contiguous(), rope[1].to(dtype).contiguous()


class RopeCache:
  """(cos, sin) tables of the last position ids seen.  The ids of a generation do not change between
  denoising steps; recomputing the tables costs ~25 small launches per step."""

  def __init__(self):
    self._key = None
    self._value = None

  def get(self, id_tensors: Sequence[torch.Tensor], axes_dim: Sequence[int], dtype):
    key = tuple((t.data_ptr(), tuple(t.shape), t._version, t.device) for t in id_tensors) + (tuple(axes_dim), dtype)
    if key != self._key:
      ids = id_tensors[0] if len(id_tensors) == 1 else torch.cat(list(id_tensors), dim=0)
      self._value = rope_tables(rope_frequencies(ids, axes_dim), dtype)
      self._key = key
      self._ids = list(id_tensors)  # keep the tensors alive: the key holds their addresses
    return self._value


def _glue_kernels_apply(x: torch.Tensor) -> bool:
  return x.is_cuda and x.dtype == torch.bfloat16


def joint_qk_norm_rope(parts: Sequence[Tuple[torch.Tensor, "RMSNorm"]], rope, heads: int,
                       across_heads: bool = False) -> torch.Tensor:
  """RoPE(concat over tokens of RMSNorm(part)) -> [B, S_total, H, D].

  `parts` are the projections [B, T_i, H*D] in sequence order (text first), each with its norm: per
  head with weight [D], or (`across_heads`) over the whole row with weight [H*D].  On the GPU this is one
  kernel per part writing straight into the joint buffer; elsewhere the eager ops."""
  x0 = parts[0][0]
  d = x0.shape[-1] // heads
  total = sum(p.shape[1] for p, _ in parts)
  if _glue_kernels_apply(x0) and d in (64, 128, 256) and rope[0].dtype == x0.dtype and rope[0].is_contiguous():
    out = torch.empty(x0.shape[0], total, heads, d, device=x0.device, dtype=x0.dtype)
    off = 0
    for x, norm in parts:
      _native.scatter_heads(x, norm.weight, rope[0], rope[1], off, [out.data_ptr()], out.stride(0), off, heads,
                            norm.eps, across_heads)
      off += x.shape[1]
    return out
  if across_heads:
    normed = [norm(x).unflatten(-1, (heads, d)) for x, norm in parts]
  else:
    normed = [norm(x.unflatten(-1, (heads, d))) for x, norm in parts]
  return apply_rope(normed[0] if len(normed) == 1 else torch.cat(normed, dim=1), rope)


def split_tokens(x: torch.Tensor, n_first: int) -> Tuple[torch.Tensor, torch.Tensor]:
  """x[:, :n_first], x[:, n_first:] as views that remember the tensor they were cut from, so that
  `join_tokens` on the same pair returns it instead of copying (single-stream blocks hand the joint
  [text; image] sequence to each other as two views)."""
  a, b = x[:, :n_first], x[:, n_first:]
  a._joint_parent = x
  b._joint_parent = x
  return a, b


def join_tokens(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
  """cat([a, b], dim=1), without the copy when a and b are the two `split_tokens` views of one tensor."""
  parent = getattr(a, "_joint_parent", None)
  if parent is not None and parent is getattr(b, "_joint_parent", None) and a.shape[1] + b.shape[1] == parent.shape[1] \
      and a.data_ptr() == parent.data_ptr():
    return parent
  return torch.cat([a, b], dim=1)


def gated_add(x: torch.Tensor, gate: torch.Tensor, y: torch.Tensor) -> torch.Tensor:
  """x + gate[:, None] * y  (x, y [B, S, C]; gate [B, C])."""
  if _glue_kernels_apply(x) and x.is_contiguous() and x.shape[-1] % 8 == 0 and y.stride(-1) == 1 \
      and y.stride(1) % 8 == 0 and gate.stride(-1) == 1 and gate.stride(0) % 8 == 0:
    return _native.gated_residual(x, gate, y)
  return x + gate[:, None] * y


def gated_add_pair(xa, gate_a, ya, xb, gate_b, yb):
  """(xa + gate_a[:, None] * ya, xb + gate_b[:, None] * yb), one launch for both streams on the GPU."""
  ok = lambda x, g, y: (_glue_kernels_apply(x) and x.is_contiguous() and x.shape[-1] % 8 == 0 and y.stride(-1) == 1
                        and y.stride(1) % 8 == 0 and g.stride(-1) == 1 and g.stride(0) % 8 == 0)
  if ok(xa, gate_a, ya) and ok(xb, gate_b, yb) and xa.shape[-1] == xb.shape[-1]:
    return _native.gated_residual_pair(xa, gate_a, ya, xb, gate_b, yb)
  return gated_add(xa, gate_a, ya), gated_add(xb, gate_b, yb)


class UlyssesGroup:
  """What attention needs to know about context parallelism: the group, its size, and - when the
  ranks share one NVLink domain - the peer-memory exchange that replaces the all-to-all calls."""

  def __init__(self, group=None, exchange=None):
    import torch.distributed as dist
    self.group = group
    self.world = dist.get_world_size(group)
    self.rank = dist.get_rank(group)
    self.exchange = exchange


def _launch_scatter_jobs(jobs, heads: int, one_launch: bool):
  if one_launch:
    for i in range(0, len(jobs), 6):
      _native.scatter_heads_multi(jobs[i:i + 6], heads)
    return
  for j in jobs:
    _native.scatter_heads(j["x"], j.get("norm_weight"), j.get("cos"), j.get("sin"), j.get("table_row_offset", 0),
                          j["dst_ptrs"], j["dst_batch_stride"], j["dst_row_offset"], heads, j.get("eps", 0.0),
                          j.get("across_heads", False))


def joint_attention(q_parts, k_parts, v_parts, rope, heads: int, cp: Optional["UlyssesGroup"] = None,
                    across_heads: bool = False) -> torch.Tensor:
  """Attention over the concatenation (text first) of the given projections.

  q_parts / k_parts: sequences of (projection [B, T_i, H*D], RMSNorm module); v_parts: projections.
  Returns [B, sum T_i, H*D] for this rank's tokens.  Per-head norm, rotary embedding and the
  concatenation are one kernel per part; under Ulysses with a peer exchange the same kernel also does
  the head scatter to the other GPUs."""
  ex = cp.exchange if cp is not None and cp.world > 1 else None
  x0 = q_parts[0][0]
  d = x0.shape[-1] // heads
  local_total = sum(p.shape[1] for p, _ in q_parts)
  # Many tokens: one specialised launch per projection (fewer registers, ~40 % faster per byte).  Few
  # tokens (rank shards of a wide context-parallel run): all jobs in one launch, launch cost dominates.
  one_launch = x0.shape[0] * max(p.shape[1] for p, _ in q_parts) <= 1536
  if ex is None:
    if _glue_kernels_apply(x0) and d in (64, 128, 256) and rope[0].dtype == x0.dtype and rope[0].is_contiguous():
      q, k = (torch.empty(x0.shape[0], local_total, heads, d, device=x0.device, dtype=x0.dtype) for _ in range(2))
      # a single v projection is used where it lies (a strided view); several are gathered into one buffer
      v = v_parts[0].unflatten(-1, (heads, d)) if len(v_parts) == 1 else torch.empty_like(q)
      jobs, off = [], 0
      for (xq, nq), (xk, nk), xv in zip(q_parts, k_parts, v_parts):
        for x, norm, buf in ((xq, nq, q), (xk, nk, k)):
          jobs.append(dict(x=x, norm_weight=norm.weight, cos=rope[0], sin=rope[1], table_row_offset=off,
                           dst_ptrs=[buf.data_ptr()], dst_batch_stride=buf.stride(0), dst_row_offset=off,
                           eps=norm.eps, across_heads=across_heads))
        if len(v_parts) > 1:
          jobs.append(dict(x=xv, dst_ptrs=[v.data_ptr()], dst_batch_stride=v.stride(0), dst_row_offset=off))
        off += xq.shape[1]
      _launch_scatter_jobs(jobs, heads, one_launch)
      return attention(q, k, v, cp)
    q = joint_qk_norm_rope(q_parts, rope, heads, across_heads)
    k = joint_qk_norm_rope(k_parts, rope, heads, across_heads)
    vs = [part.unflatten(-1, (heads, d)) for part in v_parts]
    return attention(q, k, vs[0] if len(vs) == 1 else torch.cat(vs, dim=1), cp)
  ex.ensure(x0.shape[0], local_total, heads, d, x0.dtype)
  jobs, off = [], 0
  for (xq, nq), (xk, nk), xv in zip(q_parts, k_parts, v_parts):
    jobs.append(ex.scatter_job("q", xq, off, nq.weight, rope[0], rope[1], nq.eps, across_heads))
    jobs.append(ex.scatter_job("k", xk, off, nk.weight, rope[0], rope[1], nk.eps, across_heads))
    jobs.append(ex.scatter_job("v", xv, off))
    off += xq.shape[1]
  _launch_scatter_jobs(jobs, heads, one_launch or ex.fp8)
  ex.qkv_ready()
  b = ex.buffers
  o = F.scaled_dot_product_attention(b["q"].transpose(1, 2), b["k"].transpose(1, 2), b["v"].transpose(1, 2))
  o = o.transpose(1, 2).contiguous()  # [B, S_all, H/W, D]
  return ex.gather_output(o).flatten(2)


def _all_to_all(x: torch.Tensor, scatter_dim: int, gather_dim: int, cp: UlyssesGroup, counts=None) -> torch.Tensor:
  """Split `scatter_dim` over the ranks and concatenate what arrives along `gather_dim`.

  x is [B, tokens, heads, D].  `counts` = token counts of all ranks when they differ (None: equal):
  scattering heads (dim 2) then receives `counts[r]` tokens from rank r; scattering tokens (dim 1)
  splits them by `counts`."""
  import torch.distributed as dist
  w = cp.world

  def split(t):
    parts = t.split(list(counts), dim=1) if counts is not None and scatter_dim == 1 else t.chunk(w, dim=scatter_dim)
    return [c.contiguous() for c in parts]

  send = split(x)
  if dist.get_backend(cp.group) == "gloo":
    # gloo has no all-to-all: every rank publishes its tensor and keeps its slices (CPU tests only)
    everything = [None] * w
    dist.all_gather_object(everything, x.contiguous(), group=cp.group)
    recv = [split(e)[cp.rank] for e in everything]
  else:
    recv = []
    for r in range(w):
      shape = list(send[cp.rank].shape)
      if counts is not None and scatter_dim == 2:
        shape[1] = counts[r]
      recv.append(torch.empty(shape, dtype=x.dtype, device=x.device))
    dist.all_to_all(recv, send, group=cp.group)
  return torch.cat(recv, dim=gather_dim)


def _token_counts(local_tokens: int, cp: UlyssesGroup):
  """Token counts of all ranks, or None when they are equal (cached per local count)."""
  import torch.distributed as dist
  cache = cp.__dict__.setdefault("_token_counts", {})
  if local_tokens not in cache:
    counts = [None] * cp.world
    dist.all_gather_object(counts, int(local_tokens), group=cp.group)
    cache[local_tokens] = None if len(set(counts)) == 1 else counts
  return cache[local_tokens]


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cp: Optional[UlyssesGroup] = None) -> torch.Tensor:
  """q, k, v [B, S_local, H, D] -> [B, S_local, H*D].  Under Ulysses the heads are exchanged for the
  full sequence before the attention kernel and back after it (four all-to-alls)."""
  counts = None
  if cp is not None and cp.world > 1:
    counts = _token_counts(q.shape[1], cp)
    q, k, v = (_all_to_all(t, 2, 1, cp, counts) for t in (q, k, v))  # [B, S, H/W, D]
  o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2))
  o = o.transpose(1, 2)  # [B, S, H(/W), D]
  if cp is not None and cp.world > 1:
    o = _all_to_all(o.contiguous(), 1, 2, cp, counts)  # [B, S/W, H, D]
  return o.flatten(2)
