"""Public entry points: `enable_cache`, `refresh_context`, `disable_cache`, `steps_mask`.

Signatures and the order cache -> parallelism -> quantization follow the reference
(src/cache_dit/caching/cache_interface.py:26-537, 576-831).
"""
from __future__ import annotations

import logging
from typing import List, Optional, Union

import torch

from .block_adapters import BlockAdapter, BlockAdapterRegister, ParamsModifier, flatten
from .cache_adapter import CachedAdapter, _is_pipeline
from .cache_config import DBCacheConfig
from .cache_types import CacheType
from .calibrators import CalibratorConfig, TaylorSeerCalibratorConfig

logger = logging.getLogger("cache_dit_b200")

_LEGACY_CACHE_KEYS = ParamsModifier._LEGACY_CACHE_KEYS


def enable_cache(pipe_or_adapter, cache_config: Optional[DBCacheConfig] = None,
                 calibrator_config: Optional[CalibratorConfig] = None,
                 params_modifiers: Optional[Union[ParamsModifier, List[ParamsModifier],
                                                  List[List[ParamsModifier]]]] = None,
                 parallelism_config=None, attention_backend: Optional[str] = None, quantize_config=None,
                 **kwargs):
  """Install DBCache (+ optional calibrator) on a pipeline, `BlockAdapter` or transformer, then
  optionally shard it for context parallelism and swap its linear layers to FP8.

  Returns the object it was given.  With every config left at None a default `DBCacheConfig` is used.
  """
  if cache_config is None and parallelism_config is None and attention_backend is None \
      and quantize_config is None:
    cache_config = DBCacheConfig()
  legacy = {k: kwargs[k] for k in _LEGACY_CACHE_KEYS if kwargs.get(k) is not None}
  if legacy:
    logger.warning("Passing cache options as loose keyword arguments is deprecated; use cache_config.")
    cache_config = cache_config.update(**legacy) if cache_config is not None else DBCacheConfig(**legacy)
  if cache_config is not None and (kwargs.get("enable_taylorseer") is not None
                                   or kwargs.get("enable_encoder_taylorseer") is not None):
    calibrator_config = TaylorSeerCalibratorConfig(
      enable_calibrator=kwargs.get("enable_taylorseer"),
      enable_encoder_calibrator=kwargs.get("enable_encoder_taylorseer"),
      calibrator_cache_type=kwargs.get("taylorseer_cache_type", "residual"),
      taylorseer_order=kwargs.get("taylorseer_order", 1))

  if cache_config is not None and cache_config.cache_type == CacheType.NONE:
    cache_config = None
  if cache_config is not None:
    if not (isinstance(pipe_or_adapter, (BlockAdapter, torch.nn.Module)) or _is_pipeline(pipe_or_adapter)):
      raise ValueError(f"type: {type(pipe_or_adapter)} is not valid, Please pass DiffusionPipeline or "
                       "BlockAdapter for the 1's position param: pipe_or_adapter")
    context_kwargs = {"cache_config": cache_config}
    if calibrator_config is not None:
      context_kwargs["calibrator_config"] = calibrator_config
    if params_modifiers is not None:
      context_kwargs["params_modifiers"] = params_modifiers
    pipe_or_adapter = CachedAdapter.apply(pipe_or_adapter, **context_kwargs)
  else:
    logger.warning(f"cache_config is None, skip cache acceleration for {pipe_or_adapter.__class__.__name__}.")

  if attention_backend is not None and parallelism_config is not None \
      and getattr(parallelism_config, "attention_backend", None) is None:
    parallelism_config.attention_backend = attention_backend

  if parallelism_config is None and quantize_config is None:
    return pipe_or_adapter
  transformers = _transformers_of(pipe_or_adapter, cache_config is None)
  if not transformers:
    logger.warning("No transformer is detected, skip enabling parallelism or quantization.")
    return pipe_or_adapter
  if parallelism_config is not None:
    from ..distributed import ParallelismConfig, enable_parallelism
    assert isinstance(parallelism_config, ParallelismConfig), (
      "parallelism_config should be of type ParallelismConfig.")
    for t in transformers:
      enable_parallelism(t, parallelism_config)
  if quantize_config is not None:
    from ..quantization import QuantizeConfig, quantize
    assert isinstance(quantize_config, QuantizeConfig), "quantize_config should be of type QuantizeConfig."
    for t in transformers:
      quantize(t, quantize_config=quantize_config)
  return pipe_or_adapter


def _transformers_of(pipe_or_adapter, skip_post_init: bool) -> List[torch.nn.Module]:
  if isinstance(pipe_or_adapter, torch.nn.Module):
    return [pipe_or_adapter]
  if isinstance(pipe_or_adapter, BlockAdapter):
    return [t for t in flatten(pipe_or_adapter.transformer) if t is not None]
  adapter = BlockAdapterRegister.get_adapter(pipe_or_adapter) if BlockAdapterRegister.is_supported(
    pipe_or_adapter) else None
  if adapter is not None:
    return [t for t in flatten(adapter.transformer) if t is not None]
  assert hasattr(pipe_or_adapter, "transformer"), ("The given pipeline does not have a 'transformer' "
                                                   "attribute, cannot enable parallelism.")
  return [pipe_or_adapter.transformer]


def refresh_context(transformer: torch.nn.Module, **force_refresh_kwargs):
  """Restart the persistent cache contexts of a transformer, optionally with new settings
  (`num_inference_steps=...`, `cache_config=...`, `calibrator_config=...`).  Call it before every
  generation when the transformer is driven without a pipeline."""
  if force_refresh_kwargs:
    if "cache_config" not in force_refresh_kwargs:
      # loose fields (`num_inference_steps=50`, `enable_taylorseer=True`, ...): only what is named overrides
      # the context's current configuration (src/cache_dit/caching/cache_interface.py:514-525)
      from .load_configs import load_cache_config
      cache_config, calibrator_config = load_cache_config(force_refresh_kwargs, reset=True)
      force_refresh_kwargs["cache_config"] = cache_config
      if calibrator_config is not None:
        force_refresh_kwargs["calibrator_config"] = calibrator_config
    else:
      extra = set(force_refresh_kwargs) - {"cache_config", "calibrator_config", "verbose"}
      if extra:
        logger.warning(f"force_refresh_kwargs contains cache_config, please put the extra kwargs: {extra} "
                       "into cache_config directly. Otherwise, these kwargs will be ignored.")
  CachedAdapter.maybe_refresh_context(transformer, **force_refresh_kwargs)


def disable_cache(pipe_or_adapter):
  """Remove the cache hooks, contexts and statistics that `enable_cache` installed."""
  CachedAdapter.maybe_release_hooks(pipe_or_adapter)
  from ..distributed import remove_parallelism_stats
  from ..quantization import remove_quantization_stats
  for t in ([pipe_or_adapter] if isinstance(pipe_or_adapter, torch.nn.Module) else
            _transformers_of(pipe_or_adapter, True)):
    remove_parallelism_stats(t)
    remove_quantization_stats(t)
  logger.warning(f"Acceleration hooks is disabled for: {pipe_or_adapter.__class__.__name__}.")


def supported_pipelines(**kwargs):
  return BlockAdapterRegister.supported_pipelines()


def get_adapter(pipe_or_module=None):
  return BlockAdapterRegister.get_adapter(pipe_or_module)


# ---------------------------------------------------------------------------- step masks
def _steps_mask(compute_bins: List[int], cache_bins: List[int], total_steps: Optional[int] = None) -> List[int]:
  """Interleave runs of 1s (compute) and 0s (may cache): compute_bins[0], cache_bins[0], ..."""
  if total_steps is not None:
    assert sum(compute_bins) + sum(cache_bins) >= total_steps, (
      "The sum of compute and cache intervals must be at least total_steps.")
  else:
    total_steps = sum(compute_bins) + sum(cache_bins)
  mask: List[int] = []
  i = 0
  while len(mask) < total_steps and (i < len(compute_bins) or i < len(cache_bins)):
    if i < len(compute_bins):
      mask.extend([1] * compute_bins[i])
    if i < len(cache_bins):
      mask.extend([0] * cache_bins[i])
    i += 1
  return mask[:total_steps]


# compute / cache run lengths for a 28-step schedule; other lengths are derived from these
_POLICIES_28 = {
  "slow": ([8, 3, 3, 2, 1, 1], [1, 2, 2, 2, 3]),
  "medium": ([6, 2, 2, 2, 2, 1], [1, 3, 3, 3, 3]),
  "fast": ([6, 1, 1, 1, 1, 1], [1, 3, 4, 5, 4]),
  "ultra": ([4, 1, 1, 1, 1], [2, 5, 6, 7]),
}
_POLICIES_9_15 = {
  "slow": ([4, 2, 2, 2, 1], [1, 1, 1, 1]),
  "medium": ([4, 2, 1, 1, 1], [1, 1, 2, 2]),
  "fast": ([3, 1, 1, 1, 1], [1, 2, 2, 3]),
  "ultra": ([2, 1, 1, 1, 1], [1, 2, 3, 3]),
}
_POLICIES_9 = {
  "slow": ([5, 2, 1], [1]),
  "medium": ([5, 1, 1], [1, 1]),
  "fast": ([4, 1, 1], [1, 2]),
  "ultra": ([3, 1, 1], [2, 2]),
}
_POLICIES_8 = {
  "slow": ([5, 1, 1], [1]),
  "medium": ([4, 1, 1], [1, 1]),
  "fast": ([3, 1, 1], [1, 2]),
  "ultra": ([2, 1, 1], [2, 2]),
}


def _truncate(compute: List[int], cache: List[int], target: int):
  """Shorten from the back, alternating cache / compute runs, until the lengths sum to `target`."""
  while sum(compute) + sum(cache) > target:
    if cache:
      cache[-1] -= 1
      if cache[-1] == 0:
        cache.pop()
    if sum(compute) + sum(cache) <= target:
      break
    if compute:
      compute[-1] -= 1
      if compute[-1] == 0:
        compute.pop()
  return compute, cache


def _expand(compute: List[int], cache: List[int], total_steps: int):
  """Grow every run in proportion to total_steps / 28 until the schedule is long enough."""
  base_compute, base_cache = list(compute), list(cache)
  pairs = min(len(compute), len(cache))
  grow = (total_steps / 28) * 0.5
  while sum(compute) + sum(cache) < total_steps:
    done = False
    for i in range(pairs):
      compute[i] += max(int(base_compute[i] * grow), 1)
      if sum(compute) + sum(cache) >= total_steps:
        done = True
        break
      cache[i] += max(int(base_cache[i] * grow), 1)
      if sum(compute) + sum(cache) >= total_steps:
        done = True
        break
    if done:
      break
    compute[-1] += 1
  return compute, cache


def steps_mask(compute_bins: Optional[List[int]] = None, cache_bins: Optional[List[int]] = None,
               total_steps: Optional[int] = None, mask_policy: Optional[str] = "medium") -> List[int]:
  """Per-step plan for `steps_computation_mask`: 1 = compute, 0 = cache allowed.

  Either give explicit run lengths (`compute_bins`, `cache_bins`) or a named policy
  ("slow" | "medium" | "fast" | "ultra") with `total_steps`; the last step always computes when a
  policy is used."""
  if compute_bins is not None and cache_bins is not None:
    return _steps_mask(compute_bins, cache_bins, total_steps)
  assert total_steps is not None, "total_steps must be provided when using predefined mask_policy."
  if total_steps >= 16:
    table = {k: (list(c), list(h)) for k, (c, h) in _POLICIES_28.items()}
    if total_steps > 28:
      table = {k: _expand(c, h, total_steps) for k, (c, h) in table.items()}
    if total_steps != 28:
      table = {k: _truncate(c, h, total_steps) for k, (c, h) in table.items()}
  elif total_steps >= 8:
    src = _POLICIES_8 if total_steps == 8 else (_POLICIES_9 if total_steps == 9 else _POLICIES_9_15)
    table = {k: _truncate(list(c), list(h), total_steps) for k, (c, h) in src.items()}
  else:
    assert total_steps in (4, 6), ("Only total_steps=4 or 6 is supported for predefined masks "
                                   f"while total_steps < 8. Got total_steps={total_steps}.")
    constant = ([2, 1], [1]) if total_steps == 4 else ([3, 1], [2])
    table = {k: (list(constant[0]), list(constant[1])) for k in _POLICIES_28}
  if mask_policy not in table:
    raise ValueError(f"mask_policy {mask_policy} is not valid, choose from {list(table)}")
  compute, cache = table[mask_policy]
  mask = _steps_mask(compute, cache, total_steps)
  mask[-1] = 1
  return mask
