"""Parallelism config with the reference's field names (src/cache_dit/distributed/config.py:11-163).

Only Ulysses context parallelism on one node is built here (`ulysses_size`); ring and tensor
parallel sizes are accepted for schema compatibility and must be left at None / 1.
"""
from __future__ import annotations

import dataclasses
import enum
from typing import Any, Dict, List, Optional, Union

import torch
import torch.distributed as dist


class ParallelismBackend(enum.Enum):
  """Backend names of the reference (src/cache_dit/distributed/backend.py:28-93).  One backend exists here
  (context parallelism of this package); the names are kept so that configuration files load unchanged."""
  AUTO = "Auto"
  CACHE_DIT = "CACHE_DIT"
  NATIVE_DIFFUSER = "Native_Diffuser"
  NATIVE_PYTORCH = "Native_PyTorch"
  NATIVE_HYBRID = "Native_Hybrid"
  NONE = "None"

  @classmethod
  def from_str(cls, name: str) -> "ParallelismBackend":
    key = str(name).lower()
    for member in cls:
      if key in (member.value.lower(), member.name.lower()):
        return cls.canonicalize(member)
    raise ValueError(f"Unsupported parallelism backend: {name}.")

  @classmethod
  def canonicalize(cls, backend: "ParallelismBackend") -> "ParallelismBackend":
    return cls.CACHE_DIT if backend == cls.NATIVE_DIFFUSER else backend

  @classmethod
  def is_supported(cls, backend: "ParallelismBackend") -> bool:
    backend = cls.canonicalize(backend)
    if backend == cls.NONE:
      raise ValueError("ParallelismBackend.NONE is not a valid backend")
    return backend in (cls.AUTO, cls.CACHE_DIT)  # tensor parallel / hybrid are not built

  def __str__(self) -> str:
    return self.value


@dataclasses.dataclass
class ParallelismConfig:
  backend: Union[str, ParallelismBackend] = ParallelismBackend.AUTO
  ulysses_size: Optional[int] = None
  ring_size: Optional[int] = None
  tp_size: Optional[int] = None
  cp_plan: Optional[Any] = None
  attention_backend: Optional[str] = None
  # allow token counts (and head counts) that do not divide by the number of ranks
  ulysses_anything: Optional[bool] = False
  ulysses_float8: Optional[bool] = False
  ulysses_async: Optional[bool] = False
  extra_parallel_modules: Optional[List[Any]] = dataclasses.field(default_factory=list)
  parallel_kwargs: Dict[str, Any] = dataclasses.field(default_factory=dict)
  _has_controlnet: bool = False
  _group: Optional[Any] = None  # process group of the context-parallel ranks (None: default group)

  def __post_init__(self):
    if isinstance(self.backend, str):
      self.backend = ParallelismBackend.from_str(self.backend)
    if not ParallelismBackend.is_supported(self.backend):
      raise NotImplementedError(f"parallelism backend {self.backend} is not built in cache_dit_b200 "
                                "(context parallelism only)")
    # legacy location of the switches (also under their older `experimental_` names)
    for key in ("attention_backend", "ulysses_anything", "ulysses_float8", "ulysses_async"):
      for legacy in (key, "experimental_" + key):
        if legacy in self.parallel_kwargs and not getattr(self, key):
          setattr(self, key, self.parallel_kwargs[legacy])
    if not any((size or 1) > 1 for size in (self.ulysses_size, self.ring_size, self.tp_size)):
      # same refusal as the reference (src/cache_dit/distributed/config.py:212-214): a config object means "parallel"
      raise ValueError("No parallelism is enabled. Please set ulysses_size, ring_size, or tp_size "
                       "to enable parallelism.")
    if (self.ring_size or 1) > 1:
      raise NotImplementedError("ring attention is not built in cache_dit_b200 (Ulysses only)")
    if (self.tp_size or 1) > 1:
      raise NotImplementedError("tensor parallelism is not built in cache_dit_b200 (context parallel only)")
    if self.ulysses_async:
      raise NotImplementedError("async Ulysses is not built in cache_dit_b200 yet")
    if self.backend == ParallelismBackend.AUTO:
      self.backend = ParallelismBackend.CACHE_DIT
    if self.cp_enabled() and dist.is_available() and dist.is_initialized():
      world = dist.get_world_size(self._group)
      assert self.ulysses_size == world, (
        f"ulysses_size {self.ulysses_size} must equal the number of ranks in the group ({world})")

  def cp_enabled(self) -> bool:
    return (self.ulysses_size or 1) > 1

  def exchange_mode(self) -> str:
    """How attention trades heads for tokens: "peer" = stores into the other GPUs' memory fused with
    the producing kernels (single node, NCCL process group, at most 8 ranks), "nccl" = all-to-all
    collectives.  `parallel_kwargs["exchange"]` or CACHE_DIT_B200_ULYSSES_EXCHANGE picks one; the
    default takes "peer" whenever it applies."""
    import os
    want = self.parallel_kwargs.get("exchange") or os.environ.get("CACHE_DIT_B200_ULYSSES_EXCHANGE") or "auto"
    if want not in ("auto", "peer", "nccl"):
      raise ValueError(f"unknown Ulysses exchange {want!r} (auto | peer | nccl)")
    if want != "auto":
      return want
    if not (dist.is_available() and dist.is_initialized() and torch.cuda.is_available()):
      return "nccl"
    one_node = os.environ.get("LOCAL_WORLD_SIZE", os.environ.get("WORLD_SIZE", "1")) == os.environ.get("WORLD_SIZE", "1")
    world = dist.get_world_size(self._group)
    return "peer" if dist.get_backend(self._group) == "nccl" and one_node and 1 < world <= 8 else "nccl"

  def enabled(self) -> bool:
    return self.cp_enabled()

  def strify(self, details: bool = False) -> str:
    if details:
      return f"ParallelismConfig(ulysses_size={self.ulysses_size}, ulysses_anything={self.ulysses_anything})"
    tag = f"Ulysses{self.ulysses_size}" if self.cp_enabled() else "NoParallel"
    return tag + ("_anything" if self.ulysses_anything else "")
