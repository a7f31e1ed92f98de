"""CPU restatement of the FP8 (e4m3fn) w8a8 dynamic per-row linear (numpy only).

TEST INFRASTRUCTURE, NOT PRODUCT CODE: imported only by the tests, the smoke check and the
CPU-baseline leg of the benchmark.

PARITY: PINNED FOR THE E4M3 CAST AND THE PRODUCT, UNPINNED FOR TORCHAO'S SCALE RULE.  In the reference this
arithmetic lives in two third-party dependencies: torchao (pyproject lower bound `torchao>=0.17.0`, no lock
file; neither vendored nor installed here) for the dynamic activation / weight quantization, and
`torch._scaled_mm` for the product (which refuses row-wise scales on CPU).  The reference holds no golden
values for this path; its tests compare torchao with itself.  What is pinned: tests/golden/fp8_torch_cuda.npz
holds scales, e4m3 codes and row-wise `torch._scaled_mm` outputs that PyTorch's CUDA ops produced on a B200
for small seeded inputs (generator: tests/golden/make_fp8_torch_fixture.py); this file reproduces the scales
and codes bit for bit and the product to within one bf16 step.  What is not: that torchao computes the scale
as amax / 448 with 1 for an all-zero row is restated from its published algorithm and from the reference's
own call sites:
  * config: PerRow/PerRow, e4m3fn, dynamic activations .... src/cache_dit/quantization/torchao/quantize_ao.py:540-558
  * all-zero row -> scale 1 .............................. src/cache_dit/quantization/torchao/quantize_ao.py:43-71
  * operand / scale layout, bias, output dtype ........... src/cache_dit/quantization/torchao/_scaled_mm.py:62-91
  * which layers are quantized ........................... src/cache_dit/quantization/torchao/quantize_ao.py:666-775

Algorithm (torchao float8 dynamic quantization, row-wise granularity):
  scale_r = max_k |x[r,k]| / 448        (float32; 1 when the row is all zero).  On a GPU PyTorch divides a
            tensor by a Python scalar as a multiplication by the float32 reciprocal of the scalar (ATen's
            true-division kernel for a CPU-scalar divisor), so the value the reference gets there is
            amax * fl32(1/448), which can differ from amax / 448 in the last bit; that form is used here
  q[r,k]  = e4m3fn( clamp(x[r,k] / scale_r, -448, 448) )     round-to-nearest-even
  out     = bf16( (q_a @ q_w^T) * scale_a[:,None] * scale_w[None,:] + bias )   fp32 accumulate
"""
from __future__ import annotations

from typing import Optional, Tuple

import numpy as np

from .cache_oracle import round_bf16

E4M3_MAX = np.float32(448.0)


def e4m3_round(x: np.ndarray) -> np.ndarray:
  """Round float32 to the nearest e4m3fn value (ties to even), saturating at +-448."""
  a = np.clip(np.asarray(x, dtype=np.float32), -E4M3_MAX, E4M3_MAX)
  mag = np.abs(a)
  with np.errstate(divide="ignore"):
    e = np.floor(np.log2(np.where(mag > 0, mag, 1.0))).astype(np.int32)
  e = np.maximum(e, -6)  # below 2^-6 the grid is the subnormal one: step 2^-9
  quantum = np.exp2((e - 3).astype(np.float32)).astype(np.float32)
  r = np.rint(a / quantum).astype(np.float32) * quantum  # np.rint: ties to even
  return np.clip(r, -E4M3_MAX, E4M3_MAX).astype(np.float32)


def e4m3_encode(v: np.ndarray) -> np.ndarray:
  """Byte codes of values already on the e4m3fn grid."""
  v = np.asarray(v, dtype=np.float32)
  sign = (np.signbit(v)).astype(np.uint8) << 7
  mag = np.abs(v)
  with np.errstate(divide="ignore"):
    e = np.floor(np.log2(np.where(mag > 0, mag, 1.0))).astype(np.int32)
  normal = mag >= np.float32(2.0**-6)
  exp_field = np.where(normal, e + 7, 0).astype(np.int32)
  mant = np.where(normal, np.rint(mag / np.exp2(e.astype(np.float32)) * 8.0) - 8,
                  np.rint(mag * 512.0)).astype(np.int32)
  return (sign | (exp_field.astype(np.uint8) << 3) | mant.astype(np.uint8)).astype(np.uint8)


def e4m3_decode(codes: np.ndarray) -> np.ndarray:
  c = np.asarray(codes, dtype=np.uint8).astype(np.int32)
  sign = np.where(c & 0x80, -1.0, 1.0).astype(np.float32)
  exp_field = (c >> 3) & 0xF
  mant = (c & 7).astype(np.float32)
  normal = exp_field > 0
  val = np.where(normal, (1.0 + mant / 8.0) * np.exp2((exp_field - 7).astype(np.float32)),
                 mant * np.float32(2.0**-9))
  return (sign * val).astype(np.float32)


SCALE_RULES = ("fp32_reciprocal", "fp32_division", "bf16")


def row_scales(x: np.ndarray, rule: str = "fp32_reciprocal") -> np.ndarray:
  """Per-row scale under one of the ways `amax / 448` can be carried out.

  fp32_reciprocal  amax * fl32(1/448) in float32: what PyTorch's CUDA kernels give for `amax.float() / 448.0`
                   (the pinned rule, see the header)
  fp32_division    the correctly rounded float32 quotient amax / 448 (differs in the last bit at most)
  bf16             amax kept in the input dtype and divided there, i.e. the quotient rounded to bf16 and then
                   widened: what a quantizer that never leaves bf16 would produce (scales move by up to 2^-9)
  The alternatives exist to BOUND what the unpinned part of the rule (torchao cannot be run here) can cost; the
  product path and every parity test use the first."""
  x = np.asarray(x, dtype=np.float32)
  amax = np.max(np.abs(x), axis=1).astype(np.float32)
  if rule == "fp32_reciprocal":
    scale = (amax * (np.float32(1.0) / E4M3_MAX)).astype(np.float32)
  elif rule == "fp32_division":
    scale = (amax / E4M3_MAX).astype(np.float32)
  elif rule == "bf16":
    scale = round_bf16((amax * (np.float32(1.0) / E4M3_MAX)).astype(np.float32))
  else:
    raise ValueError(f"unknown scale rule {rule!r}")
  return np.where(scale == 0, np.float32(1.0), scale).astype(np.float32)


def quantize_rows(x: np.ndarray, rule: str = "fp32_reciprocal") -> Tuple[np.ndarray, np.ndarray]:
  """x [rows, cols] (float32 holding bf16 values) -> (e4m3 byte codes, float32 scales)."""
  x = np.asarray(x, dtype=np.float32)
  scale = row_scales(x, rule)
  q = e4m3_round((x / scale[:, None]).astype(np.float32))
  return e4m3_encode(q), scale


def layernorm_modulate(x: np.ndarray, shift: np.ndarray, scale: np.ndarray, eps: float) -> np.ndarray:
  """bf16 eager pipeline: LayerNorm (no affine, fp32 statistics, bf16 result), then
  round(round(norm * round(1 + scale)) + shift).  x [rows, cols]; shift/scale [cols]."""
  x = np.asarray(x, dtype=np.float32)
  mean = x.mean(axis=1, keepdims=True, dtype=np.float64)
  var = ((x - mean)**2).mean(axis=1, keepdims=True, dtype=np.float64)
  norm = round_bf16(((x - mean) / np.sqrt(var + eps)).astype(np.float32))
  one_plus = round_bf16(np.float32(1.0) + scale.astype(np.float32))
  return round_bf16(round_bf16(norm * one_plus) + shift.astype(np.float32))


def gelu_tanh(x: np.ndarray) -> np.ndarray:
  x = np.asarray(x, dtype=np.float64)
  y = 0.5 * x * (1.0 + np.tanh(0.7978845608028654 * (x + 0.044715 * x**3)))
  return round_bf16(y.astype(np.float32))


def scaled_mm(a_codes: np.ndarray, a_scale: np.ndarray, w_codes: np.ndarray, w_scale: np.ndarray,
              bias: Optional[np.ndarray] = None) -> np.ndarray:
  """(A_q @ W_q^T) * a_scale[:,None] * w_scale[None,:] (+ bias), rounded to bf16."""
  a = e4m3_decode(a_codes)
  w = e4m3_decode(w_codes)
  acc = a @ w.T  # float32 accumulate; every product of two e4m3 values is exact in float32
  out = acc * a_scale.astype(np.float32)[:, None] * w_scale.astype(np.float32)[None, :]
  if bias is not None:
    out = out + bias.astype(np.float32)[None, :]
  return round_bf16(out.astype(np.float32))


def fp8_linear(x: np.ndarray, w: np.ndarray, bias: Optional[np.ndarray] = None,
               rule: str = "fp32_reciprocal") -> np.ndarray:
  """Dynamic per-token activation quantization + per-output-row weight quantization + product."""
  a_codes, a_scale = quantize_rows(x, rule)
  w_codes, w_scale = quantize_rows(w, rule)
  return scaled_mm(a_codes, a_scale, w_codes, w_scale, bias)
