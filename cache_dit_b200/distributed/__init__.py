"""Context parallelism (Ulysses) for the DiT hot path: config and the enable / disable switches."""
from __future__ import annotations

import logging

import torch

from .config import ParallelismBackend, ParallelismConfig

logger = logging.getLogger("cache_dit_b200")


def enable_parallelism(transformer: torch.nn.Module, parallelism_config: ParallelismConfig) -> torch.nn.Module:
  """Shard the transformer's sequence over the ranks of the process group.

  The model supplies the plan (what to split, what to gather, where attention exchanges heads for
  tokens) through `enable_context_parallel(config)`, the counterpart of the reference's per-model
  plans (src/cache_dit/distributed/transformers/flux.py:49-61, qwen_image.py:63-79, wan.py:52-65)."""
  if getattr(transformer, "_is_parallelized", False):
    logger.warning(f"{transformer.__class__.__name__} is already parallelized, skipping.")
    return transformer
  if not parallelism_config.enabled():
    return transformer
  if not hasattr(transformer, "enable_context_parallel"):
    raise ValueError(f"{transformer.__class__.__name__} does not define a context-parallel plan "
                     "(method `enable_context_parallel(config)`).")
  transformer.enable_context_parallel(parallelism_config)
  transformer._is_parallelized = True
  transformer._parallelism_config = parallelism_config
  return transformer


def remove_parallelism_stats(module) -> None:
  if module is None:
    return
  if getattr(module, "_is_parallelized", False) and hasattr(module, "disable_context_parallel"):
    module.disable_context_parallel()
  for attr in ("_is_parallelized", "_parallelism_config"):
    if attr in vars(module):
      delattr(module, attr)
