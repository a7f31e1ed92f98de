"""Parallelism config with the reference's field names (src/cache_dit/distributed/config.py:11-163).

Only Ulysses context parallelism on one node is built here (`ulysses_size`); ring and tensor
parallel sizes are accepted for schema compatibility and must be left at None / 1.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional

import torch
import torch.distributed as dist


@dataclasses.dataclass
class ParallelismConfig:
  backend: str = "auto"
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
    # legacy location of the switches
    for key in ("attention_backend", "ulysses_anything", "ulysses_float8", "ulysses_async"):
      if key in self.parallel_kwargs and not getattr(self, key):
        setattr(self, key, self.parallel_kwargs[key])
    if (self.ring_size or 1) > 1:
      raise NotImplementedError("ring attention is not built in cache_dit_b200 (Ulysses only)")
    if (self.tp_size or 1) > 1:
      raise NotImplementedError("tensor parallelism is not built in cache_dit_b200 (context parallel only)")
    if self.ulysses_async:
      raise NotImplementedError("async Ulysses is not built in cache_dit_b200 yet")
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
