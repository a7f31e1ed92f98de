"""Quantization config with the reference's field names
(src/cache_dit/quantization/config.py:329-705).

Only the path this package accelerates is implemented: `quant_type="float8_per_row"` (dynamic
per-token e4m3 activations x per-output-row e4m3 weights).  Unlike the reference, constructing the
config does not require torchao: the kernels are this package's own.
"""
from __future__ import annotations

import dataclasses
from enum import Enum
from typing import Any, Callable, Dict, List, Optional, Union

SUPPORTED_QUANT_TYPES = ("float8_per_row", )
KNOWN_QUANT_TYPES = ("float8_per_tensor", "float8_per_row", "float8_per_block", "float8_weight_only", "nvfp4",
                     "nvfp4_weight_only", "int8_per_tensor", "int8_per_row", "int8_weight_only",
                     "int4_weight_only")


class QuantizeBackend(Enum):
  AUTO = "auto"
  NATIVE = "native"  # the sm_100a kernels of this package

  @classmethod
  def from_str(cls, name: str) -> "QuantizeBackend":
    name = name.lower()
    # backend names of the reference all resolve to the one backend that exists here
    return cls.AUTO if name == "auto" else cls.NATIVE


@dataclasses.dataclass
class QuantizeConfig:
  backend: Union[str, QuantizeBackend] = QuantizeBackend.AUTO
  quant_type: str = "float8_per_row"
  # a linear layer whose qualified name contains one of these strings stays in bf16
  exclude_layers: Optional[list] = dataclasses.field(
    default_factory=lambda: ["embedder", "embed", "modulation", "mod"])
  # quantize only inside the repeated transformer block classes (named here or by the model's
  # `_repeated_blocks` attribute); False: every eligible linear of the module
  regional_quantize: bool = True
  repeated_blocks: List[str] = dataclasses.field(default_factory=list)
  # filter_fn(module, qualified_name) -> bool overrides exclude_layers
  filter_fn: Optional[Callable[..., bool]] = None
  components_to_quantize: Optional[Union[List[str], Dict[str, Dict[str, str]]]] = None
  per_tensor_fallback: bool = True
  precision_plan: Optional[Dict[str, str]] = None
  calibrate_fn: Optional[Callable[..., Any]] = None
  serialize_to: Optional[str] = None
  svdq_kwargs: Optional[Dict[str, Any]] = None
  verbose: bool = False

  def __post_init__(self):
    if isinstance(self.quant_type, str):
      self.quant_type = self.quant_type.lower()
    if isinstance(self.backend, str):
      self.backend = QuantizeBackend.from_str(self.backend)
    if self.backend == QuantizeBackend.AUTO:
      self.backend = QuantizeBackend.NATIVE
    if self.quant_type not in SUPPORTED_QUANT_TYPES:
      known = self.quant_type in KNOWN_QUANT_TYPES or self.quant_type.startswith("svdq")
      raise NotImplementedError(
        f"quant_type {self.quant_type!r} is {'not built' if known else 'unknown'} in cache_dit_b200; "
        f"supported: {SUPPORTED_QUANT_TYPES}")
    if self.svdq_kwargs is not None:
      raise ValueError("svdq_kwargs is only valid when quant_type starts with 'svdq'.")
    if self.precision_plan:
      for layer, qt in self.precision_plan.items():
        if qt.lower() not in SUPPORTED_QUANT_TYPES:
          raise NotImplementedError(f"precision_plan[{layer!r}] = {qt!r} is not built in cache_dit_b200")

  def as_dict(self) -> Dict[str, Any]:
    return dataclasses.asdict(self)

  def update(self, **kwargs) -> "QuantizeConfig":
    for key, value in kwargs.items():
      if hasattr(self, key) and value is not None:
        setattr(self, key, value)
    if "backend" not in kwargs:
      self.backend = QuantizeBackend.AUTO
    self.__post_init__()
    return self

  def strify(self) -> str:
    if self.components_to_quantize is None or isinstance(self.components_to_quantize, list):
      return self.quant_type
    return "".join(f"<{c}:{d.get('quant_type', self.quant_type)}>" for c, d in self.components_to_quantize.items())

  def is_svdq(self) -> bool:
    return False

  def component_quant_types(self) -> Dict[str, str]:
    if self.components_to_quantize is None:
      return {"transformer": self.quant_type}
    if isinstance(self.components_to_quantize, list):
      return {c: self.quant_type for c in self.components_to_quantize}
    return {c: d.get("quant_type", self.quant_type) for c, d in self.components_to_quantize.items()}

  @classmethod
  def expand_configs(cls, config: "QuantizeConfig") -> List["QuantizeConfig"]:
    if config.components_to_quantize is None:
      return [config]
    if isinstance(config.components_to_quantize, list):
      return [dataclasses.replace(config, components_to_quantize=[c]) for c in config.components_to_quantize]
    return [
      dataclasses.replace(config, components_to_quantize=[c], quant_type=d.get("quant_type", config.quant_type),
                          exclude_layers=d.get("exclude_layers", config.exclude_layers),
                          regional_quantize=d.get("regional_quantize", config.regional_quantize),
                          repeated_blocks=d.get("repeated_blocks", config.repeated_blocks))
      for c, d in config.components_to_quantize.items()
    ]
