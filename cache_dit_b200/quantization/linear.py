"""`Float8RowwiseLinear`: an nn.Linear replacement backed by the sm_100a FP8 kernels.

Semantics follow the float8 per-row dynamic inference path the reference selects
(src/cache_dit/quantization/torchao/quantize_ao.py:540-558, 43-71 and .../_scaled_mm.py:62-91):
weights are quantized once to e4m3 with one scale per output row, activations are quantized per
token at every call, the product is scaled by both and returned in bf16.
"""
from __future__ import annotations

from typing import Optional

import torch

from .. import _native


class Float8RowwiseLinear(torch.nn.Module):
  """y = fp8_gemm(quant_rows(x), W_q) * a_scale * w_scale (+ bias); bf16 in, bf16 out."""

  def __init__(self, in_features: int, out_features: int, weight_q: torch.Tensor, weight_scale: torch.Tensor,
               bias: Optional[torch.Tensor]):
    super().__init__()
    self.in_features = in_features
    self.out_features = out_features
    self.register_buffer("weight_q", weight_q)          # [N, K] float8_e4m3fn
    self.register_buffer("weight_scale", weight_scale)  # [N] float32
    self.register_buffer("bias", bias)                  # [N] bf16 or None

  @classmethod
  def from_linear(cls, linear: torch.nn.Linear) -> "Float8RowwiseLinear":
    w = linear.weight.detach()
    if not w.is_cuda:
      raise RuntimeError("float8_per_row quantization runs on the GPU: move the module to CUDA first")
    if w.dtype != torch.bfloat16:
      raise RuntimeError(f"float8_per_row needs bf16 weights, got {w.dtype}")
    n, k = w.shape
    if k % 16 != 0 or n % 8 != 0:
      raise RuntimeError(f"float8_per_row needs in_features % 16 == 0 and out_features % 8 == 0, got {k}, {n}")
    w_q = torch.empty((n, k), dtype=torch.float8_e4m3fn, device=w.device)
    w_scale = torch.empty(n, dtype=torch.float32, device=w.device)
    _native.fp8_quant_rows(w.contiguous(), w_q, w_scale)
    bias = None if linear.bias is None else linear.bias.detach().to(torch.bfloat16).contiguous()
    return cls(k, n, w_q, w_scale, bias)

  @staticmethod
  def supports(linear: torch.nn.Linear) -> bool:
    n, k = linear.weight.shape
    return linear.weight.dtype == torch.bfloat16 and k % 16 == 0 and n % 8 == 0 and k <= 16384

  def quantize_input(self, x: torch.Tensor):
    x2 = x.reshape(-1, self.in_features)
    if x2.stride(-1) != 1:
      x2 = x2.contiguous()
    a_q = torch.empty(x2.shape, dtype=torch.float8_e4m3fn, device=x.device)
    a_scale = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
    _native.fp8_quant_rows(x2, a_q, a_scale)
    return a_q, a_scale

  def forward_quantized(self, a_q: torch.Tensor, a_scale: torch.Tensor, lead_shape, gelu: bool = False) -> torch.Tensor:
    """Product for activations that a fused producer kernel already quantized.  `gelu`: the output passes
    through tanh-GELU in the product's epilogue (bf16(gelu(bf16(y))), what an eager gelu(linear(x)) gives)."""
    out = torch.empty((a_q.shape[0], self.out_features), dtype=torch.bfloat16, device=a_q.device)
    if gelu:
      _native.fp8_gemm_rowscaled_grouped([(a_q, a_scale, self.weight_q, self.weight_scale, self.bias, out)], [0])
    else:
      _native.fp8_gemm_rowscaled(a_q, a_scale, self.weight_q, self.weight_scale, self.bias, out)
    return out.view(*lead_shape, self.out_features)

  def forward(self, x: torch.Tensor) -> torch.Tensor:
    if x.dtype != torch.bfloat16:
      x = x.to(torch.bfloat16)
    a_q, a_scale = self.quantize_input(x)
    return self.forward_quantized(a_q, a_scale, x.shape[:-1])

  def extra_repr(self) -> str:
    return f"in_features={self.in_features}, out_features={self.out_features}, bias={self.bias is not None}, fp8=e4m3 per-row"


def quantize_rows_fused(x: torch.Tensor, preop: int, mod_shift=None, mod_scale=None, eps: float = 1e-6):
  """Quantize `op(x)` without materialising it: op = adaLN-modulated LayerNorm or tanh-GELU.

  x [B, S, C] or [rows, C] bf16; for the LayerNorm variant mod_shift / mod_scale are [B, C]."""
  lead = x.shape[:-1]
  x2 = x.reshape(-1, x.shape[-1])
  if x2.stride(-1) != 1:
    x2 = x2.contiguous()
  a_q = torch.empty(x2.shape, dtype=torch.float8_e4m3fn, device=x.device)
  a_scale = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
  rows_per_batch = 0
  if preop == _native.PRE_LAYERNORM_MOD:
    batch = mod_shift.shape[0]
    rows_per_batch = x2.shape[0] // batch
  _native.fp8_quant_rows(x2, a_q, a_scale, preop, mod_shift, mod_scale, rows_per_batch, eps)
  return a_q, a_scale, lead


def quantize_rows_fused_pair(xa: torch.Tensor, xb: torch.Tensor, preop: int, mods_a=None, mods_b=None,
                             eps: float = 1e-6):
  """`quantize_rows_fused` on two tensors of the same width with ONE launch (image and text stream of a
  double-stream block).  mods_* = (shift, scale) for the LayerNorm variant.  Returns two
  (a_q, a_scale, lead_shape) triples."""
  jobs, results = [], []
  for x, mods in ((xa, mods_a), (xb, mods_b)):
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    if x2.stride(-1) != 1:
      x2 = x2.contiguous()
    a_q = torch.empty(x2.shape, dtype=torch.float8_e4m3fn, device=x.device)
    a_scale = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
    job = dict(x2d=x2, q=a_q, scale=a_scale)
    if preop == _native.PRE_LAYERNORM_MOD:
      job.update(mod_shift=mods[0], mod_scale=mods[1], rows_per_batch=x2.shape[0] // mods[0].shape[0])
    jobs.append(job)
    results.append((a_q, a_scale, lead))
  _native.fp8_quant_rows_pair(jobs, preop, eps)
  return results


class FusedFloat8Linears(torch.nn.Module):
  """Several FP8 linears that read the same activations, run as ONE GEMM over the concatenated
  output rows (q/k/v, or q/k/v + MLP-in).  Per-row weight scales make this exactly the same
  arithmetic as the separate products; the member layers keep working and share the storage
  (their `weight_q` / `weight_scale` / `bias` become views into the fused tensors)."""

  def __init__(self, linears):
    super().__init__()
    assert len({l.in_features for l in linears}) == 1
    self.in_features = linears[0].in_features
    self.splits = [l.out_features for l in linears]
    self.out_features = sum(self.splits)
    w = torch.cat([l.weight_q.view(torch.uint8) for l in linears], dim=0).view(torch.float8_e4m3fn)
    s = torch.cat([l.weight_scale for l in linears], dim=0)
    has_bias = [l.bias is not None for l in linears]
    b = None
    if any(has_bias):
      b = torch.cat([l.bias if l.bias is not None else
                     torch.zeros(l.out_features, dtype=torch.bfloat16, device=w.device) for l in linears])
    self.register_buffer("weight_q", w)
    self.register_buffer("weight_scale", s)
    self.register_buffer("bias", b)
    start = 0
    for l, n, hb in zip(linears, self.splits, has_bias):
      l.weight_q = w[start:start + n]
      l.weight_scale = s[start:start + n]
      if hb:
        l.bias = b[start:start + n]
      start += n

  def gelu_column(self, gelu_last: bool):
    """First output column of the last member (whose output is to be activated by the product's epilogue), or
    None: no activation wanted, or the member does not start on a multiple of 8 columns (the epilogue decides per
    16-byte chunk; the caller then activates the split itself)."""
    col = self.out_features - self.splits[-1]
    return col if gelu_last and col % 8 == 0 else None

  def finish(self, out: torch.Tensor, lead_shape, gelu_last: bool):
    """The members' outputs as views of the product; activates the last one here when the epilogue could not."""
    parts = list(out.view(*lead_shape, self.out_features).split(self.splits, dim=-1))
    if gelu_last and self.gelu_column(True) is None:
      parts[-1] = torch.nn.functional.gelu(parts[-1], approximate="tanh")
    return tuple(parts)

  def forward_quantized(self, a_q: torch.Tensor, a_scale: torch.Tensor, lead_shape, gelu_last: bool = False):
    """`gelu_last`: the last member's output passes through tanh-GELU, in the product's epilogue where possible
    (the MLP-in projection behind q/k/v)."""
    out = torch.empty((a_q.shape[0], self.out_features), dtype=torch.bfloat16, device=a_q.device)
    col = self.gelu_column(gelu_last)
    if col is not None:
      _native.fp8_gemm_rowscaled_grouped([(a_q, a_scale, self.weight_q, self.weight_scale, self.bias, out)], [col])
    else:
      _native.fp8_gemm_rowscaled(a_q, a_scale, self.weight_q, self.weight_scale, self.bias, out)
    return self.finish(out, lead_shape, gelu_last)


def _members_share_storage(fused: FusedFloat8Linears, linears) -> bool:
  """True while every member's weight still is the slice of the fused tensors it was made to be."""
  w = fused.weight_q
  row = 0
  for l, n in zip(linears, fused.splits):
    m = l.weight_q
    if m.device != w.device or m.data_ptr() != w.data_ptr() + row * fused.in_features or m.shape[0] != n:
      return False
    if l.weight_scale.data_ptr() != fused.weight_scale.data_ptr() + row * 4:
      return False
    row += n
  return True


def fused_group(linears) -> FusedFloat8Linears:
  """The fused module of a group of FP8 linears, built on first use and cached on the first member.

  The cache is not a registered submodule, so `model.to(...)` or anything else that replaces the members'
  buffers leaves it behind; the members are the truth then, and the group is rebuilt from them as soon
  as their storage is no longer the fused one (a pointer comparison per member and call)."""
  head = linears[0]
  key = tuple(id(l) for l in linears)
  cache = head.__dict__.setdefault("_fused_groups", {})
  fused = cache.get(key)
  if fused is None or not _members_share_storage(fused, linears):
    fused = FusedFloat8Linears(list(linears))
    cache[key] = fused
  return fused


def grouped_forward_quantized(items, gelu_last: bool = False):
  """Products of up to two FP8 linears (or fused groups) with already quantized activations as ONE
  launch: items = [(module, a_q, a_scale, lead_shape), ...].  Returns each module's usual result (a
  tensor, or the tuple of splits of a fused group).  The second product is typically the small text
  stream of a double-stream block, whose tiles fill the tail wave of the first.  `gelu_last`: every item's
  output (its last member's, for a fused group) passes through tanh-GELU in the epilogue."""
  outs = [torch.empty((a_q.shape[0], m.out_features), dtype=torch.bfloat16, device=a_q.device) for m, a_q, _, _ in items]
  problems = [(a_q, a_scale, m.weight_q, m.weight_scale, m.bias, out) for (m, a_q, a_scale, _), out in zip(items, outs)]
  act = None
  if gelu_last:
    act = [m.gelu_column(True) if isinstance(m, FusedFloat8Linears) else 0 for m, _, _, _ in items]
  for i in range(0, len(problems), 2):
    _native.fp8_gemm_rowscaled_grouped(problems[i:i + 2], None if act is None else act[i:i + 2])
  results = []
  for (m, _, _, lead), out in zip(items, outs):
    if isinstance(m, FusedFloat8Linears):
      results.append(m.finish(out, lead, gelu_last))
    else:
      results.append(out.view(*lead, m.out_features))
  return results
