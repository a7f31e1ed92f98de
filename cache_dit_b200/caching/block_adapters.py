"""Where the cached runner is installed: `BlockAdapter`, `ParamsModifier`, adapter registry.

`BlockAdapter` names a transformer (or several), its block lists, how each block is called
(`ForwardPattern`) and which attribute names hold the lists; field names follow the reference
(src/cache_dit/caching/block_adapters/block_adapters.py:28-117) so adapters written for it can be
passed here.  Internally everything is normalised to "one list of block-lists per transformer".
Model families are looked up by class-name prefix in `BlockAdapterRegister`
(src/cache_dit/caching/block_adapters/block_registers.py:15-121); only the three DiT shapes the
hot path is measured on are pre-registered (see cache_dit_b200.synthetic).
"""
from __future__ import annotations

import dataclasses
import logging
from collections.abc import Iterable
from typing import Any, Callable, Dict, List, Optional, Union

import torch

from .cache_config import BasicCacheConfig
from .calibrators import CalibratorConfig, TaylorSeerCalibratorConfig
from .forward_pattern import ForwardPattern

logger = logging.getLogger("cache_dit_b200")

_ATOMS = (str, bytes, torch.nn.ModuleList, torch.nn.Module, torch.Tensor)


class FakeDiffusionPipeline:
  """Stands in for a pipeline when only a transformer is given (contexts then persist)."""

  def __init__(self, transformer: Optional[torch.nn.Module] = None):
    self.transformer = transformer


class ParamsModifier:
  """Per-block-list overrides of the cache / calibrator config
  (src/cache_dit/caching/params_modifier.py:10-81)."""

  _LEGACY_CACHE_KEYS = ("Fn_compute_blocks", "Bn_compute_blocks", "max_warmup_steps", "max_cached_steps",
                        "max_continuous_cached_steps", "residual_diff_threshold", "enable_separate_cfg",
                        "cfg_compute_first", "cfg_diff_compute_separate")

  def __init__(self, cache_config: BasicCacheConfig = None,
               calibrator_config: Optional[CalibratorConfig] = None, **kwargs):
    self._context_kwargs: Dict[str, Any] = {}
    legacy = {k: kwargs[k] for k in self._LEGACY_CACHE_KEYS if kwargs.get(k) is not None}
    if legacy:
      cache_config = cache_config.update(**legacy) if cache_config is not None else BasicCacheConfig(**legacy)
    if cache_config is not None:
      self._context_kwargs["cache_config"] = cache_config
    if kwargs.get("enable_taylorseer") is not None or kwargs.get("enable_encoder_taylorseer") is not None:
      calibrator_config = TaylorSeerCalibratorConfig(
        enable_calibrator=kwargs.get("enable_taylorseer"),
        enable_encoder_calibrator=kwargs.get("enable_encoder_taylorseer"),
        calibrator_cache_type=kwargs.get("taylorseer_cache_type", "residual"),
        taylorseer_order=kwargs.get("taylorseer_order", 1))
    if calibrator_config is not None:
      self._context_kwargs["calibrator_config"] = calibrator_config


def nested_depth(obj: Any) -> int:
  """str / module: 0, list of those: 1, list of lists: 2."""
  if isinstance(obj, _ATOMS) or not isinstance(obj, Iterable):
    return 0
  items = obj.values() if isinstance(obj, dict) else obj
  return 1 + max((nested_depth(i) for i in items), default=0)


def flatten(attr) -> List[Any]:
  if isinstance(attr, _ATOMS) or not isinstance(attr, Iterable):
    return [attr]
  out: List[Any] = []
  for a in attr:
    out.extend(flatten(a))
  return out


@dataclasses.dataclass
class BlockAdapter:
  pipe: Any = None
  transformer: Union[torch.nn.Module, List[torch.nn.Module]] = None
  blocks: Union[torch.nn.ModuleList, List[torch.nn.ModuleList], List[List[torch.nn.ModuleList]]] = None
  blocks_name: Union[str, List[str], List[List[str]]] = None
  unique_blocks_name: Union[str, List[str], List[List[str]]] = dataclasses.field(default_factory=list)
  dummy_blocks_names: Union[List[str], List[List[str]]] = dataclasses.field(default_factory=list)
  forward_pattern: Union[ForwardPattern, List[ForwardPattern], List[List[ForwardPattern]]] = None
  params_modifiers: Optional[Union[ParamsModifier, List[ParamsModifier], List[List[ParamsModifier]]]] = None
  check_forward_pattern: Optional[bool] = None
  check_num_outputs: bool = False
  patch_functor: Optional[Any] = None  # object with .apply(transformer) run before caching
  has_separate_cfg: bool = False
  auto: bool = False
  allow_prefixes: List[str] = dataclasses.field(default_factory=lambda: [
    "transformer", "single_transformer", "blocks", "layers", "single_stream_blocks", "double_stream_blocks"])
  check_prefixes: bool = True
  allow_suffixes: List[str] = dataclasses.field(default_factory=lambda: ["TransformerBlock"])
  check_suffixes: bool = False
  blocks_policy: str = "max"
  skip_post_init: bool = False

  def __post_init__(self):
    if self.skip_post_init:
      return
    if self.pipe is None:
      self.pipe = FakeDiffusionPipeline()
    if self.transformer is None and getattr(self.pipe, "transformer", None) is not None:
      self.transformer = self.pipe.transformer
    if isinstance(self.pipe, FakeDiffusionPipeline) and self.pipe.transformer is None:
      self.pipe.transformer = self.transformer
    if self.transformer is None:
      return
    if self.blocks is not None and self.blocks_name is None:
      self.blocks_name = self._find_names(self.transformer, self.blocks)
    if self.patch_functor is not None and nested_depth(self.transformer) == 0:
      self.transformer = self.patch_functor.apply(self.transformer) or self.transformer
    if self.check_forward_pattern is None:
      # blocks of models that do not come from diffusers cannot be assumed to follow its naming
      first = flatten(self.transformer)[0]
      self.check_forward_pattern = first.__module__.startswith("diffusers")

  @staticmethod
  def _find_names(transformer, blocks):
    """Attribute name(s) under which the given block list(s) live on the transformer."""

    def find(tr, bl):
      for attr, value in vars(tr).get("_modules", {}).items():
        if value is bl:
          return attr
      # a concatenation of several lists (e.g. double + single stream) is patched in under the
      # name of the list its first block belongs to
      first = bl[0] if len(bl) else None
      for attr, value in vars(tr).get("_modules", {}).items():
        if isinstance(value, torch.nn.ModuleList) and len(value) and value[0] is first:
          return attr
      raise ValueError("blocks_name is required: the block list is not an attribute of the transformer")

    if nested_depth(blocks) == 0:
      return find(flatten(transformer)[0], blocks)
    trs = flatten(transformer)
    if nested_depth(blocks) == 1:
      if len(trs) == len(blocks) and len(trs) > 1:
        return [find(t, b) for t, b in zip(trs, blocks)]
      return [find(trs[0], b) for b in blocks]
    return [[find(t, b) for b in bs] for t, bs in zip(trs, blocks)]

  # ---- normalisation: transformer -> [T], every other attribute -> [[...] per transformer]
  @staticmethod
  def normalize(adapter: "BlockAdapter", unique: bool = True) -> "BlockAdapter":
    if getattr(adapter, "_is_normalized", False):
      return adapter
    if nested_depth(adapter.transformer) == 0:
      adapter.transformer = [adapter.transformer]
    n = len(adapter.transformer)

    def norm(attr):
      if attr is None:
        return None
      depth = nested_depth(attr)
      if depth == 0:
        attr = [[attr]]
      elif depth == 1:
        if not attr:
          attr = [[] for _ in range(n)]
        elif len(attr) == n:
          attr = [[a] for a in attr]
        else:
          attr = [list(attr)]
      assert len(attr) == n
      return attr

    adapter.blocks = norm(adapter.blocks)
    adapter.blocks_name = norm(adapter.blocks_name)
    adapter.forward_pattern = norm(adapter.forward_pattern)
    adapter.dummy_blocks_names = norm(adapter.dummy_blocks_names)
    adapter.params_modifiers = norm(adapter.params_modifiers)
    if unique:
      for i in range(n):
        assert len(adapter.blocks[i]) == len(adapter.blocks_name[i]) == len(adapter.forward_pattern[i])
      if not adapter.unique_blocks_name:
        adapter.unique_blocks_name = [[f"{name}_{id(blocks)}" for blocks, name in zip(bl, nm)]
                                      for bl, nm in zip(adapter.blocks, adapter.blocks_name)]
      else:
        adapter.unique_blocks_name = norm(adapter.unique_blocks_name)
    adapter._is_normalized = True
    return adapter

  @staticmethod
  def assert_normalized(adapter: "BlockAdapter"):
    if not getattr(adapter, "_is_normalized", False):
      raise RuntimeError("block_adapter must be normailzed.")

  @staticmethod
  def is_normalized(adapter: "BlockAdapter") -> bool:
    return getattr(adapter, "_is_normalized", False)

  @classmethod
  def is_cached(cls, adapter: Any) -> bool:
    if isinstance(adapter, cls):
      cls.assert_normalized(adapter)
      return bool(getattr(adapter.pipe, "_is_cached", False)
                  and getattr(adapter.transformer[0], "_is_cached", False))
    if isinstance(adapter, list):
      return getattr(adapter[0], "_is_cached", False)
    return getattr(adapter, "_is_cached", False)

  @classmethod
  def is_parallelized(cls, adapter: Any) -> bool:
    return cls._flag(adapter, "_is_parallelized")

  @classmethod
  def is_quantized(cls, adapter: Any) -> bool:
    return cls._flag(adapter, "_is_quantized")

  @classmethod
  def _flag(cls, adapter: Any, name: str) -> bool:
    if isinstance(adapter, cls):
      cls.assert_normalized(adapter)
      return getattr(adapter.transformer[0], name, False)
    if isinstance(adapter, list):
      return getattr(adapter[0], name, False)
    if not isinstance(adapter, torch.nn.Module) and hasattr(adapter, "transformer"):
      return getattr(adapter.transformer, name, False)
    return getattr(adapter, name, False)

  nested_depth = staticmethod(nested_depth)
  flatten = staticmethod(flatten)

  @staticmethod
  def check_block_adapter(adapter: "BlockAdapter") -> bool:
    for attr in ("pipe", "transformer", "blocks", "blocks_name", "forward_pattern"):
      if getattr(adapter, attr, None) is None:
        logger.warning(f"{attr} is None!")
        return False
    first = flatten(adapter.forward_pattern)[0]
    return isinstance(first, ForwardPattern)

  @staticmethod
  def find_blocks(transformer: torch.nn.Module) -> List[torch.nn.ModuleList]:
    return [m for m in vars(transformer).get("_modules", {}).values() if isinstance(m, torch.nn.ModuleList)]

  @staticmethod
  def auto_block_adapter(adapter: "BlockAdapter") -> "BlockAdapter":
    """Pick the block list by name prefix (largest or smallest list, `blocks_policy`)."""
    assert adapter.auto, "Please manually set `auto` to True!"
    transformer = flatten(adapter.transformer)[0]
    candidates = []
    for attr, value in vars(transformer).get("_modules", {}).items():
      if not isinstance(value, torch.nn.ModuleList) or len(value) == 0:
        continue
      if adapter.check_prefixes and not any(attr.startswith(p) for p in adapter.allow_prefixes):
        continue
      if adapter.check_suffixes and not any(
          value[0].__class__.__name__.endswith(s) for s in adapter.allow_suffixes):
        continue
      candidates.append((len(value), attr, value))
    if not candidates:
      raise ValueError("auto block adapter: no block list found")
    candidates.sort(key=lambda c: c[0], reverse=adapter.blocks_policy == "max")
    _, adapter.blocks_name, adapter.blocks = candidates[0]
    return adapter


class BlockAdapterRegister:
  """Class-name-prefix -> adapter factory.  `register("Flux")(fn)`; `fn(pipe_or_transformer)`."""

  _adapters: Dict[str, Callable[..., BlockAdapter]] = {}
  _separate_cfg_prefixes: List[str] = []

  @classmethod
  def register(cls, name: str, supported: bool = True, separate_cfg: bool = False):

    def decorator(fn):
      if supported:
        cls._adapters[name] = fn
        if separate_cfg and name not in cls._separate_cfg_prefixes:
          cls._separate_cfg_prefixes.append(name)
      return fn

    return decorator

  @classmethod
  def _match(cls, obj) -> Optional[str]:
    cls_name = obj if isinstance(obj, str) else obj.__class__.__name__
    for name in cls._adapters:
      if cls_name.startswith(name):
        return name
    return None

  @classmethod
  def get_adapter(cls, pipe_or_module, **kwargs) -> Optional[BlockAdapter]:
    name = cls._match(pipe_or_module)
    return cls._adapters[name](pipe_or_module, **kwargs) if name else None

  @classmethod
  def is_supported(cls, pipe_or_module) -> bool:
    return cls._match(pipe_or_module) is not None

  @classmethod
  def has_separate_cfg(cls, pipe_or_adapter) -> bool:
    if isinstance(pipe_or_adapter, BlockAdapter):
      if pipe_or_adapter.has_separate_cfg:
        return True
      target = flatten(pipe_or_adapter.transformer)[0] if isinstance(
        pipe_or_adapter.pipe, FakeDiffusionPipeline) else pipe_or_adapter.pipe
    else:
      target = pipe_or_adapter
    cls_name = target.__class__.__name__
    return any(cls_name.startswith(p) for p in cls._separate_cfg_prefixes)

  @classmethod
  def supported_pipelines(cls):
    names = [f"{n}*" for n in cls._adapters]
    return len(names), names
