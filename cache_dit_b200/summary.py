"""`summary()`: read the statistics the cache engine leaves on modules after a run.

Mirrors the reference's read-out (src/cache_dit/summary.py:22-166, 330-568): one `CacheStats` per
cached block list followed by one per transformer; `cached_steps` is the hit mask and
`residual_diffs` maps str(step) -> relative-L1 diff.
"""
from __future__ import annotations

import dataclasses
import logging
from typing import Any, Dict, List

import numpy as np
import torch

from .caching.block_adapters import BlockAdapter, FakeDiffusionPipeline, flatten
from .caching.cache_types import CacheType

logger = logging.getLogger("cache_dit_b200")


@dataclasses.dataclass
class CacheStats:
  cache_options: dict = dataclasses.field(default_factory=dict)
  cached_steps: List[int] = dataclasses.field(default_factory=list)
  residual_diffs: Dict[str, float] = dataclasses.field(default_factory=dict)
  cfg_cached_steps: List[int] = dataclasses.field(default_factory=list)
  cfg_residual_diffs: Dict[str, float] = dataclasses.field(default_factory=dict)
  accumulated_cached_steps: int = 0
  cfg_accumulated_cached_steps: int = 0
  accumulated_executed_steps: int = 0
  accumulated_transformer_executed_steps: int = 0
  # block-pruning fields exist for layout compatibility; pruning is not part of this package
  pruned_steps: List[int] = dataclasses.field(default_factory=list)
  pruned_blocks: List[int] = dataclasses.field(default_factory=list)
  actual_blocks: List[int] = dataclasses.field(default_factory=list)
  pruned_ratio: float = None
  cfg_pruned_steps: List[int] = dataclasses.field(default_factory=list)
  cfg_pruned_blocks: List[int] = dataclasses.field(default_factory=list)
  cfg_actual_blocks: List[int] = dataclasses.field(default_factory=list)
  cfg_pruned_ratio: float = None
  parallelism_config: Any = None
  quantize_config: Any = None


def _quantiles_line(tag: str, steps: List[int], diffs: Dict[str, float]) -> str:
  vals = [v for v in diffs.values() if isinstance(v, (int, float))]
  if not vals:
    return f"{tag}: cached steps {len(steps)}, no diffs recorded"
  q = np.percentile(vals, [0, 25, 50, 75, 95])
  return (f"{tag}: cached steps {len(steps)} | diffs P00 {q[0]:.3f} P25 {q[1]:.3f} P50 {q[2]:.3f} "
          f"P75 {q[3]:.3f} P95 {q[4]:.3f} min {min(vals):.3f} max {max(vals):.3f}")


def _summary(module, details: bool = False, logging: bool = True) -> CacheStats:
  stats = CacheStats()
  if not isinstance(module, torch.nn.Module):
    module = module.transformer
  name = module[0].__class__.__name__ if isinstance(module, torch.nn.ModuleList) and len(module) else \
      module.__class__.__name__
  if hasattr(module, "_context_kwargs"):
    stats.cache_options = module._context_kwargs
  if hasattr(module, "_parallelism_config"):
    stats.parallelism_config = module._parallelism_config
  if hasattr(module, "_quantize_config"):
    stats.quantize_config = module._quantize_config
  if hasattr(module, "_cached_steps"):
    stats.cached_steps = list(module._cached_steps)
    stats.residual_diffs = dict(module._residual_diffs)
    stats.accumulated_cached_steps = module._accumulated_cached_steps
    stats.accumulated_executed_steps = getattr(module, "_accumulated_executed_steps", 0)
    stats.accumulated_transformer_executed_steps = getattr(module, "_accumulated_transformer_executed_steps", 0)
    if logging and (stats.residual_diffs or stats.cached_steps):
      logger.info(_quantiles_line(f"cache stats {name}", stats.cached_steps, stats.residual_diffs))
      if details:
        logger.info(f"cached steps: {stats.cached_steps}\nresidual diffs: {stats.residual_diffs}")
  if hasattr(module, "_cfg_cached_steps"):
    stats.cfg_cached_steps = list(module._cfg_cached_steps)
    stats.cfg_residual_diffs = dict(module._cfg_residual_diffs)
    stats.cfg_accumulated_cached_steps = module._cfg_accumulated_cached_steps
    if logging and (stats.cfg_residual_diffs or stats.cfg_cached_steps):
      logger.info(_quantiles_line(f"CFG cache stats {name}", stats.cfg_cached_steps, stats.cfg_residual_diffs))
  return stats


def summary(adapter_or_others, details: bool = False, logging: bool = True, **kwargs) -> List[CacheStats]:
  if adapter_or_others is None:
    return [CacheStats()]
  if isinstance(adapter_or_others, FakeDiffusionPipeline):
    raise ValueError("Please pass DiffusionPipeline, BlockAdapter or transfomer, not FakeDiffusionPipeline.")
  collected: List[CacheStats] = []
  if isinstance(adapter_or_others, BlockAdapter):
    if not BlockAdapter.check_block_adapter(adapter_or_others):
      return [CacheStats()]
    for blocks in flatten(adapter_or_others.blocks):
      if getattr(blocks, "_context_kwargs", None) is not None:
        collected.append(_summary(blocks, details, logging))
    for transformer in flatten(adapter_or_others.transformer):
      collected.append(_summary(transformer, details, logging))
  else:
    if isinstance(adapter_or_others, torch.nn.Module):
      transformers = [adapter_or_others]
    else:
      transformers = [t for t in (getattr(adapter_or_others, "transformer", None),
                                  getattr(adapter_or_others, "transformer_2", None)) if t is not None]
    for t in transformers:
      if getattr(t, "_is_cached", False):
        for blocks in BlockAdapter.find_blocks(t):
          collected.append(_summary(blocks, details, logging))
    for t in transformers:
      collected.append(_summary(t, details, logging))
  collected = [s for s in collected if s.cache_options or s.parallelism_config or s.quantize_config]
  return collected if collected else [CacheStats()]


def strify(adapter_or_others) -> str:
  """One-line tag of the active optimisations, e.g. `DBCache_F8B0_W8I1M0MC0_R0.08_T1O1_S14`."""
  if isinstance(adapter_or_others, CacheStats):
    stats = adapter_or_others
  elif isinstance(adapter_or_others, list):
    stats = adapter_or_others[0]
  else:
    stats = summary(adapter_or_others, logging=False)[-1]
  options = stats.cache_options or {}
  tag = ""
  cache_config = options.get("cache_config")
  if cache_config is not None and cache_config.cache_type != CacheType.NONE:
    calibrator_config = options.get("calibrator_config")
    tag = cache_config.strify() + "_" + (calibrator_config.strify() if calibrator_config is not None else "T0O0")
  if stats.parallelism_config is not None:
    tag += f"_{stats.parallelism_config.strify()}"
  if stats.quantize_config is not None:
    tag += f"_{stats.quantize_config.strify()}"
  if stats.accumulated_cached_steps and cache_config is not None:
    tag += f"_S{stats.accumulated_cached_steps}"
  return tag.strip("_")
