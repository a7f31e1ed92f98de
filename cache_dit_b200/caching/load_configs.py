"""Configuration from a YAML file or a dictionary.

Same entry points and file layout as the reference (src/cache_dit/caching/load_configs.py:22-470), so that a
configuration written for it drives this package unchanged:

    cache_config:            # DBCacheConfig fields, plus the calibrator switches
      Fn_compute_blocks: 8
      residual_diff_threshold: 0.08
      steps_computation_mask: fast        # a policy name is expanded with num_inference_steps
      num_inference_steps: 28
      enable_taylorseer: true
      taylorseer_order: 1
    parallelism_config:      # ParallelismConfig fields; `ulysses: 8` is short for `ulysses_size: 8`, "auto" = world size
      ulysses_size: auto
    attention_backend: native
    quantize_config:         # QuantizeConfig fields
      quant_type: float8_per_row

A file without a `cache_config` section is read as the older flat layout (the cache fields at top level),
unless it holds one of the other sections, in which case there is no cache configuration in it.
Calibrators and cache types outside this package (DMD, FoCa, DBPrune) are refused by name.
"""
from __future__ import annotations

import copy
import logging
from typing import Any, Dict, Optional, Tuple, Union

from .cache_config import DBCacheConfig
from .calibrators import CalibratorConfig, TaylorSeerCalibratorConfig
from ..distributed.config import ParallelismBackend, ParallelismConfig
from ..quantization.config import QuantizeConfig

logger = logging.getLogger("cache_dit_b200")

_SECTIONS = ("parallelism_config", "attention_backend", "quantize_config")
_SIZE_KEYS = ("ulysses_size", "ring_size", "tp_size")


def _read(path_or_dict: Union[str, dict]) -> dict:
  """The configuration as a private dictionary (a deep copy, or the parsed file)."""
  if isinstance(path_or_dict, dict):
    return copy.deepcopy(path_or_dict)
  if not isinstance(path_or_dict, str):
    raise ValueError("Input must be a file path (str) or a configuration dictionary (dict).")
  import yaml
  try:
    with open(path_or_dict, "r") as f:
      data = yaml.safe_load(f)
  except FileNotFoundError:
    raise FileNotFoundError(f"Configuration file not found: {path_or_dict}")
  except yaml.YAMLError as e:
    raise yaml.YAMLError(f"YAML file parsing error: {str(e)}")
  return data if data is not None else {}


def _calibrator_from(fields: dict, reset: bool) -> Optional[CalibratorConfig]:
  chosen = [name for name in ("enable_taylorseer", "enable_dmd", "enable_foca") if fields.get(name, False)]
  if len(chosen) > 1:
    raise ValueError("`enable_taylorseer`, `enable_dmd`, and `enable_foca` are mutually exclusive. "
                     "Please set only one of them to true.")
  if not chosen:
    return None
  if chosen[0] != "enable_taylorseer":
    raise NotImplementedError(f"`{chosen[0]}`: only the TaylorSeer calibrator is built in cache_dit_b200")
  values = dict(enable_calibrator=fields.get("enable_taylorseer"),
                enable_encoder_calibrator=fields.get("enable_encoder_taylorseer", False),
                calibrator_cache_type=fields.get("taylorseer_cache_type", "residual"),
                taylorseer_order=fields.get("taylorseer_order", 1))
  return TaylorSeerCalibratorConfig().reset(**values) if reset else TaylorSeerCalibratorConfig(**values)


def _cache_options(fields: dict, reset: bool) -> Dict[str, Any]:
  """{"cache_config": ..., ["calibrator_config": ...]} from the flat field layout.  With `reset` every field
  that the input does not name is None, so that the result only overrides what was named."""
  try:
    fields = copy.deepcopy(fields)
    out: Dict[str, Any] = {}
    calibrator = _calibrator_from(fields, reset)
    if calibrator is not None:
      out["calibrator_config"] = calibrator
    kind = str(fields["cache_type"]) if "cache_type" in fields else "DBCache"
    if kind == "DBPrune":
      raise NotImplementedError("cache_type DBPrune is not built in cache_dit_b200 (DBCache only)")
    if kind != "DBCache":
      raise ValueError(f"Unsupported cache_type: {kind}.")
    fields.pop("cache_type", None)  # the dataclass keeps the enum, not its name
    config = DBCacheConfig().reset() if reset else DBCacheConfig()
    out["cache_config"] = config.update(**fields)
    return out
  except NotImplementedError:
    raise
  except Exception as e:
    raise ValueError(f"Error parsing cache configuration. {str(e)}")


def load_options(path_or_dict: Union[str, dict], reset: bool = False) -> dict:
  """Deprecated flat layout: returns the keyword arguments for `enable_cache`."""
  logger.warning("`load_options` is deprecated and will be removed in future versions. "
                 "Please use `load_configs` instead.")
  return _cache_options(_read(path_or_dict), reset)


def load_cache_config(path_or_dict: Union[str, dict], **kwargs) -> Tuple[Optional[DBCacheConfig], Optional[CalibratorConfig]]:
  """(cache config, calibrator config or None); (None, None) when the input only holds other sections."""
  data = _read(path_or_dict)
  reset = kwargs.get("reset", False)
  if "cache_config" in data:
    fields = data["cache_config"]
    policy = fields.get("steps_computation_mask")
    if isinstance(policy, str):
      assert "num_inference_steps" in fields, (
        "To parse steps_mask from str, 'num_inference_steps' must be provided in cache_config.")
      from .cache_interface import steps_mask
      fields["steps_computation_mask"] = steps_mask(total_steps=fields["num_inference_steps"], mask_policy=policy)
  elif any(section in data for section in _SECTIONS):
    return None, None
  else:
    fields = data
  options = _cache_options(fields, reset)
  if options.get("cache_config") is None:
    raise ValueError("Failed to load 'cache_config'. Got None.")
  return options["cache_config"], options.get("calibrator_config")


def _resolve_auto_sizes(fields: dict) -> None:
  """Replace the one size given as "auto" by (number of ranks) / (product of the other sizes)."""

  def is_auto(v) -> bool:
    return isinstance(v, str) and v.lower() == "auto"

  autos = [k for k in _SIZE_KEYS if is_auto(fields.get(k))]
  if len(autos) > 1:
    raise ValueError("Only one of 'ulysses_size', 'ring_size', or 'tp_size' can be set to 'auto'.")
  for key in _SIZE_KEYS:
    v = fields.get(key)
    if v is not None and not isinstance(v, int) and not is_auto(v):
      raise ValueError(f"Invalid parallel size value: {v}. Must be int or 'auto'.")
  if not autos:
    return
  import torch.distributed as dist
  others = 1
  for key in _SIZE_KEYS:
    if key != autos[0]:
      others *= fields.get(key) or 1
  size = dist.get_world_size() // others if dist.is_available() and dist.is_initialized() else 1
  if size == 1:
    logger.warning("Auto parallel size selected as 1. Make sure to run with torch.distributed "
                   "to utilize multiple devices for parallelism.")
  fields[autos[0]] = size


def load_parallelism_config(path_or_dict: Union[str, dict], **kwargs) -> Union[Optional[ParallelismConfig], bool]:
  """The `parallelism_config` section (None if absent); `check_only=True` only says whether it is there."""
  data = _read(path_or_dict)
  if kwargs.get("check_only", False):
    return "parallelism_config" in data
  if "parallelism_config" not in data:
    return None
  fields = data["parallelism_config"]
  for short, full in (("ulysses", "ulysses_size"), ("ring", "ring_size"), ("tp", "tp_size")):
    if short not in fields:
      continue
    if full in fields and fields[full] != fields[short]:
      raise ValueError(f"Both {short} and {full} are set with different values: {fields[short]} vs {fields[full]}.")
    fields[full] = fields.pop(short)
  if "backend" in fields:
    fields["backend"] = ParallelismBackend.from_str(fields["backend"])
  if kwargs.get("auto_parallel_size", True):
    _resolve_auto_sizes(fields)
  return ParallelismConfig(**fields)


def load_attn_backend_config(path_or_dict: Union[str, dict], **kwargs) -> Optional[str]:
  return _read(path_or_dict).get("attention_backend")


def load_quantize_config(path_or_dict: Union[str, dict], **kwargs) -> Optional[QuantizeConfig]:
  """The `quantize_config` section; unknown keys and None values are dropped."""
  data = _read(path_or_dict)
  if "quantize_config" not in data:
    return None
  known = QuantizeConfig.__dataclass_fields__
  return QuantizeConfig(**{k: v for k, v in data["quantize_config"].items() if k in known and v is not None})


def load_configs(path_or_dict: Union[str, dict], return_dict: bool = True, **kwargs):
  """Everything `enable_cache` takes, from one file or dictionary: a dictionary keyed by argument name, or
  the tuple (cache, calibrator, parallelism, attention backend, quantize)."""
  cache_config, calibrator_config = load_cache_config(path_or_dict, **kwargs)
  parallelism_config = load_parallelism_config(path_or_dict, **kwargs)
  if isinstance(parallelism_config, bool):  # check_only was passed through
    parallelism_config = None
  loaded = dict(cache_config=cache_config, calibrator_config=calibrator_config, parallelism_config=parallelism_config,
                attention_backend=load_attn_backend_config(path_or_dict, **kwargs),
                quantize_config=load_quantize_config(path_or_dict, **kwargs))
  return loaded if return_dict else tuple(loaded.values())
