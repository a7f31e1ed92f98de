"""`quantize(module, QuantizeConfig)`: swap eligible nn.Linear layers for FP8 row-wise linears.

Layer selection follows the reference's filter (src/cache_dit/quantization/torchao/quantize_ao.py:74-163,
666-775): inside the repeated transformer block classes only (regional quantization), names not
matching `exclude_layers`, bf16 weights only; a custom `filter_fn` replaces the name filter.
"""
from __future__ import annotations

import logging
from typing import List

import torch

from .config import QuantizeConfig
from .linear import Float8RowwiseLinear

logger = logging.getLogger("cache_dit_b200")


def _eligible(name: str, m: torch.nn.Module, cfg: QuantizeConfig, skipped: List[str]) -> bool:
  if not isinstance(m, torch.nn.Linear) or isinstance(m, Float8RowwiseLinear):
    return False
  if cfg.filter_fn is not None:
    return bool(cfg.filter_fn(m, name))
  for pattern in (cfg.exclude_layers or []):
    if pattern in name:
      skipped.append(f"skip: {name} -> pattern<{pattern}>")
      return False
  if m.weight.dtype != torch.bfloat16:
    skipped.append(f"skip: {name} -> pattern<dtype({m.weight.dtype})!=bfloat16>")
    return False
  if not Float8RowwiseLinear.supports(m):
    skipped.append(f"skip: {name} -> pattern<shape{tuple(m.weight.shape)}>")
    return False
  return True


def _swap_linears(root: torch.nn.Module, prefix: str, cfg: QuantizeConfig, skipped: List[str]) -> int:
  count = 0
  for child_name, child in list(root.named_children()):
    full = f"{prefix}.{child_name}" if prefix else child_name
    if _eligible(full, child, cfg, skipped):
      setattr(root, child_name, Float8RowwiseLinear.from_linear(child))
      count += 1
    else:
      count += _swap_linears(child, full, cfg, skipped)
  return count


def quantize(module: torch.nn.Module, quantize_config: QuantizeConfig = None, **kwargs) -> torch.nn.Module:
  if quantize_config is None:
    quantize_config = QuantizeConfig(**kwargs)
  if getattr(module, "_is_quantized", False):
    logger.warning(f"Module {module.__class__.__name__} is already quantized, skipping.")
    return module
  repeated = list(getattr(module, "_repeated_blocks", None) or quantize_config.repeated_blocks or [])
  regional = quantize_config.regional_quantize and bool(repeated)
  skipped: List[str] = []
  total = sum(1 for m in module.modules() if isinstance(m, torch.nn.Linear))
  quantized = 0
  if regional:
    hit = False
    for name, sub in list(module.named_modules()):
      if sub.__class__.__name__ in repeated:
        hit = True
        # names are relative to the repeated block ("attn.to_q", not "transformer_blocks.1.attn.to_q"): the
        # reference quantizes block by block, so `exclude_layers` patterns and a custom `filter_fn(m, name)`
        # see block-relative names there (quantize_ao.py:128-131, 666-720) and must see the same here
        quantized += _swap_linears(sub, "", quantize_config, skipped)
    if not hit:
      raise ValueError(f"Regional quantization failed because {repeated} classes are not found in the module.")
  else:
    quantized = _swap_linears(module, "", quantize_config, skipped)
  if torch.cuda.is_available():
    torch.cuda.empty_cache()
  fused_blocks = 0
  if quantized:
    # blocks with the attribute layout of the public FLUX blocks get forwards that fuse the producers (adaLN
    # LayerNorm, GELU, concatenation, QK norm + rotary embedding) into the quantization and glue kernels
    from .fused_blocks import install_fused_block_forwards
    fused_blocks = install_fused_block_forwards(module)
  module._is_quantized = True
  module._quantize_config = quantize_config
  module._quantize_type = quantize_config.quant_type
  module._exclude_layers = quantize_config.exclude_layers
  module._quantize_stats = dict(linear_layers=total, quantized=quantized, skipped=skipped, fused_blocks=fused_blocks)
  if quantize_config.verbose:
    for line in skipped:
      logger.info(line)
  logger.info(f"Quantized {quantized}/{total} linear layers of {module.__class__.__name__} to "
              f"{quantize_config.quant_type}")
  return module


def remove_quantization_stats(module) -> None:
  if module is not None and getattr(module, "_quantize_stats", {}).get("fused_blocks"):
    from .fused_blocks import remove_fused_block_forwards
    remove_fused_block_forwards(module)
  for attr in ("_is_quantized", "_quantize_config", "_quantize_type", "_exclude_layers", "_quantize_stats"):
    if module is not None and attr in vars(module):
      delattr(module, attr)
