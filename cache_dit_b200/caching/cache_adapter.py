"""Installs / refreshes / removes the cached block runner on a pipeline or transformer.

Behaviour follows the reference's `CachedAdapter`
(src/cache_dit/caching/cache_adapters/cache_adapter.py:32-723):
  * one cache context per block list, named after the list; per-list overrides by `ParamsModifier`;
  * a real pipeline gets its `__call__` wrapped so that every generation starts from fresh
    contexts and publishes statistics at the end; a bare transformer gets persistent contexts
    that restart after `num_inference_steps` calls or on `refresh_context`;
  * while the transformer's own forward runs, its block list attribute holds a one-element list
    with the cached runner (and extra lists, e.g. FLUX's single-stream list, are empty), so the
    model's forward code needs no change.
The swap is done directly in the module's `_modules` table (two dict writes per forward).
"""
from __future__ import annotations

import copy
import functools
import logging
from typing import Any, Dict, List, Tuple

import torch

from .block_adapters import (BlockAdapter, BlockAdapterRegister, FakeDiffusionPipeline, ParamsModifier,
                             flatten)
from .cache_blocks import UnifiedBlocks, apply_stats, remove_stats
from .cache_config import BasicCacheConfig
from .cache_manager import CachedContextManager
from .cache_types import CacheType
from .calibrators import CalibratorConfig

logger = logging.getLogger("cache_dit_b200")


def _is_pipeline(obj) -> bool:
  return not isinstance(obj, (torch.nn.Module, BlockAdapter, FakeDiffusionPipeline)) and hasattr(
    obj, "transformer")


class CachedAdapter:

  def __call__(self, *args, **kwargs):
    return self.apply(*args, **kwargs)

  # ---------------------------------------------------------------- entry
  @classmethod
  def apply(cls, pipe_or_adapter, **context_kwargs):
    assert pipe_or_adapter is not None, "pipe or block_adapter can not both None!"
    if isinstance(pipe_or_adapter, BlockAdapter):
      if pipe_or_adapter.params_modifiers is None:
        modifiers = context_kwargs.pop("params_modifiers", None)
        if modifiers:
          pipe_or_adapter.params_modifiers = modifiers
      else:
        context_kwargs.pop("params_modifiers", None)
      return cls.cachify(pipe_or_adapter, **context_kwargs)
    if not BlockAdapterRegister.is_supported(pipe_or_adapter):
      raise ValueError(f"{pipe_or_adapter.__class__.__name__} is not officially supported "
                       "by cache-dit, please set BlockAdapter instead!")
    adapter = BlockAdapterRegister.get_adapter(pipe_or_adapter)
    modifiers = context_kwargs.pop("params_modifiers", None)
    if modifiers:
      adapter.params_modifiers = modifiers
    adapter = cls.cachify(adapter, **context_kwargs)
    return adapter.pipe if _is_pipeline(pipe_or_adapter) else adapter.transformer[0]

  @classmethod
  def cachify(cls, block_adapter: BlockAdapter, **context_kwargs) -> BlockAdapter:
    if block_adapter.auto:
      block_adapter = BlockAdapter.auto_block_adapter(block_adapter)
    if BlockAdapter.check_block_adapter(block_adapter):
      block_adapter = BlockAdapter.normalize(block_adapter)
      if BlockAdapter.is_cached(block_adapter):
        return block_adapter
      _, contexts_kwargs = cls.create_context(block_adapter, **context_kwargs)
      cls.mock_blocks(block_adapter, contexts_kwargs)
    return block_adapter

  # ---------------------------------------------------------------- contexts
  @classmethod
  def check_context_kwargs(cls, block_adapter: BlockAdapter, **context_kwargs):
    cache_config: BasicCacheConfig = context_kwargs["cache_config"]
    assert cache_config is not None, "cache_config can not be None."
    if cache_config.enable_separate_cfg is None:
      cache_config.enable_separate_cfg = BlockAdapterRegister.has_separate_cfg(block_adapter)
    cache_type = context_kwargs.pop("cache_type", None)
    if cache_type is not None:
      assert isinstance(cache_type, CacheType), f"cache_type must be CacheType Enum, but got {type(cache_type)}."
      assert cache_type == cache_config.cache_type, (
        f"cache_type from context_kwargs ({cache_type}) must be the same "
        f"as that from cache_config ({cache_config.cache_type}).")
    return context_kwargs

  @classmethod
  def create_context(cls, block_adapter: BlockAdapter, **context_kwargs) -> Tuple[List[str], List[Dict[str, Any]]]:
    BlockAdapter.assert_normalized(block_adapter)
    context_kwargs = cls.check_context_kwargs(block_adapter, **context_kwargs)
    pipe = block_adapter.pipe
    persistent = isinstance(pipe, FakeDiffusionPipeline)
    manager = CachedContextManager(name=f"{pipe.__class__.__name__}_{id(pipe)}", persistent_context=persistent)
    names, contexts_kwargs = cls.modify_context_params(block_adapter, **context_kwargs)
    pipe._context_manager = manager
    if persistent:
      for name, kw in zip(names, contexts_kwargs):
        manager.reset_context(name, **kw)
      pipe._is_cached = True
    else:
      original_call = pipe.__class__.__call__

      @functools.wraps(original_call)
      def new_call(self, *args, **kwargs):
        mgr = getattr(self, "_context_manager", None)
        if mgr is None:  # another instance of the class that was never cache-enabled
          return original_call(self, *args, **kwargs)
        for name, kw in zip(self._context_names, self._contexts_kwargs):
          mgr.reset_context(name, **kw)  # every generation starts from fresh contexts
        outputs = original_call(self, *args, **kwargs)
        cls.apply_stats_hooks(self._block_adapter)
        return outputs

      pipe._context_names, pipe._contexts_kwargs, pipe._block_adapter = names, contexts_kwargs, block_adapter
      pipe.__class__.__call__ = new_call
      pipe.__class__._original_call = original_call
      pipe.__class__._is_cached = True
    cls.apply_params_hooks(block_adapter, contexts_kwargs)
    return names, contexts_kwargs

  @classmethod
  def modify_context_params(cls, block_adapter: BlockAdapter, **context_kwargs):
    names = flatten(block_adapter.unique_blocks_name)
    contexts_kwargs = [copy.deepcopy(context_kwargs) for _ in names]
    for kw, name in zip(contexts_kwargs, names):
      kw["name"] = name
    if block_adapter.params_modifiers is not None:
      modifiers: List[ParamsModifier] = flatten(block_adapter.params_modifiers)
      for i in range(min(len(contexts_kwargs), len(modifiers))):
        contexts_kwargs[i] = cls._modify_context_params(modifiers[i]._context_kwargs, contexts_kwargs[i])
    for kw in contexts_kwargs:
      cls._config_messages(**kw)
    return names, contexts_kwargs

  @classmethod
  def _modify_context_params(cls, new_kwargs: Dict[str, Any], old_kwargs: Dict[str, Any]) -> Dict[str, Any]:
    merged = copy.deepcopy(old_kwargs)
    if "cache_config" not in new_kwargs:
      return merged
    for key, kind in (("cache_config", BasicCacheConfig), ("calibrator_config", CalibratorConfig)):
      new = new_kwargs.get(key)
      if new is None:
        continue
      assert isinstance(new, kind), f"{key} must be {kind.__name__}, but got {type(new)}."
      if merged.get(key) is None:
        merged[key] = new
      else:
        merged[key].update(**new.as_dict())
    return merged

  @classmethod
  def _config_messages(cls, logging: bool = True, **contexts_kwargs) -> str:
    cache_config = contexts_kwargs.get("cache_config")
    calibrator_config = contexts_kwargs.get("calibrator_config")
    message = ""
    if cache_config is not None:
      message = f"Collected Context Config: {cache_config.strify()}, Calibrator Config: "
      message += calibrator_config.strify(details=True) if calibrator_config is not None else "None"
    if logging:
      logger.info(message)
    return message

  # ---------------------------------------------------------------- runner installation
  @classmethod
  def collect_unified_blocks(cls, block_adapter: BlockAdapter, contexts_kwargs: List[Dict]):
    manager = block_adapter.pipe._context_manager
    total, shift = [], 0
    for i, transformer in enumerate(block_adapter.transformer):
      bound = {}
      for j, blocks in enumerate(block_adapter.blocks[i]):
        cache_config: BasicCacheConfig = contexts_kwargs[shift + j]["cache_config"]
        bound[block_adapter.unique_blocks_name[i][j]] = torch.nn.ModuleList([
          UnifiedBlocks(blocks, transformer=transformer, forward_pattern=block_adapter.forward_pattern[i][j],
                        check_forward_pattern=block_adapter.check_forward_pattern,
                        check_num_outputs=block_adapter.check_num_outputs,
                        cache_prefix=block_adapter.blocks_name[i][j],
                        cache_context=block_adapter.unique_blocks_name[i][j], context_manager=manager,
                        cache_type=cache_config.cache_type)
        ])
      shift += len(block_adapter.blocks[i])
      total.append(bound)
    return total

  @classmethod
  def mock_blocks(cls, block_adapter: BlockAdapter, contexts_kwargs: List[Dict]):
    BlockAdapter.assert_normalized(block_adapter)
    if getattr(block_adapter.transformer[0], "_is_cached", False):
      return block_adapter.transformer
    unified = cls.collect_unified_blocks(block_adapter, contexts_kwargs)
    for i, transformer in enumerate(block_adapter.transformer):
      cls.mock_transformer(unified[i], transformer, block_adapter.blocks_name[i],
                           block_adapter.unique_blocks_name[i],
                           block_adapter.dummy_blocks_names[i] if block_adapter.dummy_blocks_names else [],
                           block_adapter)
    return block_adapter.transformer

  @classmethod
  def mock_transformer(cls, unified_blocks, transformer, blocks_name, unique_blocks_name, dummy_blocks_names,
                       block_adapter: BlockAdapter):
    manager: CachedContextManager = block_adapter.pipe._context_manager
    original_forward = transformer.forward
    empty = torch.nn.ModuleList()
    swaps = [(name, unified_blocks[ctx]) for name, ctx in zip(blocks_name, unique_blocks_name)]
    swaps += [(name, empty) for name in dummy_blocks_names]
    transformer._context_manager = manager
    transformer._context_names = list(unique_blocks_name)
    # kept reachable so that tools working on the runners (CUDA-graph capture) can find them
    transformer.__dict__["_unified_blocks"] = unified_blocks

    def new_forward(*args, **kwargs):
      modules = transformer._modules
      saved = [(name, modules[name]) for name, _ in swaps]
      for name, runner in swaps:
        modules[name] = runner
      try:
        outputs = original_forward(*args, **kwargs)
      finally:
        for name, original in saved:
          modules[name] = original
      if manager.persistent_context and manager.is_pre_refreshed():
        cls.apply_stats_hooks(block_adapter)
      return outputs

    transformer.forward = functools.update_wrapper(new_forward, original_forward)
    transformer._original_forward = original_forward
    transformer._is_cached = True
    return transformer

  @classmethod
  def apply_params_hooks(cls, block_adapter: BlockAdapter, contexts_kwargs: List[Dict]):
    block_adapter.pipe._context_kwargs = contexts_kwargs[0]
    shift = 0
    for i, transformer in enumerate(block_adapter.transformer):
      transformer._forward_pattern = block_adapter.forward_pattern
      transformer._has_separate_cfg = block_adapter.has_separate_cfg
      transformer._context_kwargs = contexts_kwargs[shift]
      for j, blocks in enumerate(block_adapter.blocks[i]):
        blocks._forward_pattern = block_adapter.forward_pattern[i][j]
        blocks._context_kwargs = contexts_kwargs[shift + j]
      shift += len(block_adapter.blocks[i])

  @classmethod
  def apply_stats_hooks(cls, block_adapter: BlockAdapter):
    manager = block_adapter.pipe._context_manager
    for i, transformer in enumerate(block_adapter.transformer):
      apply_stats(transformer, cache_context=block_adapter.unique_blocks_name[i][-1], context_manager=manager)
      for blocks, name in zip(block_adapter.blocks[i], block_adapter.unique_blocks_name[i]):
        apply_stats(blocks, cache_context=name, context_manager=manager)

  # ---------------------------------------------------------------- refresh / release
  @classmethod
  def maybe_refresh_context(cls, transformer: torch.nn.Module, **force_refresh_kwargs):
    verbose = force_refresh_kwargs.pop("verbose", False)
    manager = getattr(transformer, "_context_manager", None)
    if manager is None:
      logger.warning("Transformer has no attribute '_context_manager', skip refreshing cache context.")
      return
    if not manager.persistent_context:
      logger.warning("Transformer's context manager is not persistent, skip refreshing cache context.")
      return
    for name in getattr(transformer, "_context_names", []):
      current = manager.get_context(name)
      new_kwargs = copy.deepcopy(getattr(current, "_init_kwargs", {}))
      manager.remove_context(name)
      new_kwargs = cls._modify_context_params(force_refresh_kwargs, new_kwargs)
      manager.reset_context(name, **new_kwargs)
      if verbose:
        logger.info(f"Refreshed cache context: {name}, {cls._config_messages(logging=False, **new_kwargs)}")
      if hasattr(transformer, "_context_kwargs"):
        transformer._context_kwargs = new_kwargs

  @classmethod
  def maybe_release_hooks(cls, pipe_or_adapter):
    """Undo everything `apply` did: forwards, contexts, attributes, statistics."""
    if isinstance(pipe_or_adapter, BlockAdapter):
      BlockAdapter.assert_normalized(pipe_or_adapter)
      pipe = pipe_or_adapter.pipe
      transformers = flatten(pipe_or_adapter.transformer)
    elif isinstance(pipe_or_adapter, torch.nn.Module):
      pipe, transformers = None, [pipe_or_adapter]
    else:
      pipe = pipe_or_adapter
      transformers = [t for t in (getattr(pipe, "transformer", None), getattr(pipe, "transformer_2", None))
                      if t is not None]
    if pipe is not None:
      if hasattr(pipe.__class__, "_original_call"):
        pipe.__class__.__call__ = pipe.__class__._original_call
        del pipe.__class__._original_call
      manager = getattr(pipe, "_context_manager", None)
      if isinstance(manager, CachedContextManager):
        manager.clear_contexts()
      for attr in ("_context_manager", "_context_kwargs", "_context_names", "_contexts_kwargs",
                   "_block_adapter"):
        if attr in vars(pipe):
          delattr(pipe, attr)
      if "_is_cached" in vars(pipe):
        del pipe._is_cached
      elif "_is_cached" in vars(pipe.__class__):
        del pipe.__class__._is_cached
      remove_stats(pipe)
    for transformer in transformers:
      if hasattr(transformer, "_original_forward"):
        vars(transformer).pop("forward", None)  # the class's own forward is visible again
        del transformer._original_forward
      manager = getattr(transformer, "_context_manager", None)
      if isinstance(manager, CachedContextManager):
        manager.clear_contexts()
      for attr in ("_is_cached", "_context_manager", "_context_names", "_forward_pattern", "_has_separate_cfg",
                   "_context_kwargs", "_unified_blocks"):
        if attr in vars(transformer):
          delattr(transformer, attr)
      remove_stats(transformer)
      for blocks in BlockAdapter.find_blocks(transformer):
        for attr in ("_forward_pattern", "_context_kwargs"):
          if attr in vars(blocks):
            delattr(blocks, attr)
        remove_stats(blocks)
