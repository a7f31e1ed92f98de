"""torch.library operators over the FP8 kernels.

`cache_dit_b200::float8_inference_scaled_mm` keeps the schema of the operator the reference
registers for its FP8 product (src/cache_dit/quantization/torchao/_scaled_mm.py:94-137):
    (Tensor a_data, Tensor a_scale, Tensor b_data, Tensor b_scale, Tensor? bias,
     int out_dtype_id, bool use_fast_accum) -> Tensor
with a_data [M, K] e4m3, a_scale [M, 1] f32, b_data [K, N] e4m3 given as the transposed view of the
[N, K] weight, b_scale [1, N] f32; dtype ids {fp16: 0, bf16: 1, fp32: 2}.  Only CUDA
implementations exist; the fake implementations carry shapes for tracing.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .. import _native

_DTYPE_TO_ID = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}
_ID_TO_DTYPE = {v: k for k, v in _DTYPE_TO_ID.items()}


def encode_output_dtype(dtype: torch.dtype) -> int:
  if dtype not in _DTYPE_TO_ID:
    raise ValueError(f"Unsupported float8 inference output dtype: {dtype}")
  return _DTYPE_TO_ID[dtype]


def decode_output_dtype(dtype_id: int) -> torch.dtype:
  if dtype_id not in _ID_TO_DTYPE:
    raise ValueError(f"Unsupported float8 inference output dtype id: {dtype_id}")
  return _ID_TO_DTYPE[dtype_id]


torch.library.define(
  "cache_dit_b200::float8_inference_scaled_mm",
  "(Tensor a_data, Tensor a_scale, Tensor b_data, Tensor b_scale, Tensor? bias, int out_dtype_id, "
  "bool use_fast_accum) -> Tensor")


@torch.library.impl("cache_dit_b200::float8_inference_scaled_mm", "CUDA")
def _scaled_mm_cuda(a_data, a_scale, b_data, b_scale, bias, out_dtype_id, use_fast_accum):
  out_dtype = decode_output_dtype(out_dtype_id)
  if out_dtype != torch.bfloat16:
    raise NotImplementedError("cache_dit_b200 FP8 GEMM writes bf16 (out_dtype_id 1)")
  lead = a_data.shape[:-1]
  a2 = a_data.reshape(-1, a_data.shape[-1])
  w = b_data.t()  # back to the [N, K] row-major weight
  if not w.is_contiguous():
    w = w.contiguous()
  if not a2.is_contiguous():
    a2 = a2.contiguous()
  out = torch.empty((a2.shape[0], w.shape[0]), dtype=torch.bfloat16, device=a_data.device)
  _native.fp8_gemm_rowscaled(a2, a_scale.reshape(-1).contiguous(), w, b_scale.reshape(-1).contiguous(),
                             None if bias is None else bias.to(torch.bfloat16).contiguous(), out)
  return out.view(*lead, w.shape[0])


@torch.library.register_fake("cache_dit_b200::float8_inference_scaled_mm")
def _scaled_mm_fake(a_data, a_scale, b_data, b_scale, bias, out_dtype_id, use_fast_accum):
  return a_data.new_empty((*a_data.shape[:-1], b_data.shape[-1]), dtype=decode_output_dtype(out_dtype_id))


torch.library.define("cache_dit_b200::float8_quantize_rows", "(Tensor x) -> (Tensor, Tensor)")


@torch.library.impl("cache_dit_b200::float8_quantize_rows", "CUDA")
def _quantize_rows_cuda(x):
  x2 = x.reshape(-1, x.shape[-1])
  if x2.stride(-1) != 1:
    x2 = x2.contiguous()
  q = torch.empty(x2.shape, dtype=torch.float8_e4m3fn, device=x.device)
  scale = torch.empty(x2.shape[0], dtype=torch.float32, device=x.device)
  _native.fp8_quant_rows(x2, q, scale)
  return q.view(x.shape), scale.view(*x.shape[:-1], 1)


@torch.library.register_fake("cache_dit_b200::float8_quantize_rows")
def _quantize_rows_fake(x):
  return (x.new_empty(x.shape, dtype=torch.float8_e4m3fn),
          x.new_empty((*x.shape[:-1], 1), dtype=torch.float32))


def float8_inference_scaled_mm(a_data, a_scale, b_data, b_scale, bias: Optional[torch.Tensor] = None,
                               output_dtype: torch.dtype = torch.bfloat16, use_fast_accum: bool = True):
  return torch.ops.cache_dit_b200.float8_inference_scaled_mm(a_data, a_scale, b_data, b_scale, bias,
                                                             encode_output_dtype(output_dtype), use_fast_accum)


def float8_quantize_rows(x: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
  return torch.ops.cache_dit_b200.float8_quantize_rows(x)
