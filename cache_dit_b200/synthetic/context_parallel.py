"""Root-level Ulysses plan shared by the stand-ins: shard token tensors on entry, gather on exit.

The reference declares the same plan per model as split / gather hooks on module inputs and outputs
(src/cache_dit/distributed/transformers/flux.py:49-61, qwen_image.py:63-79, wan.py:52-65).  Token
counts that do not divide by the number of ranks are split like `torch.tensor_split` (the first
ranks hold one token more): the reference's `ulysses_anything` mode.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .layers import UlyssesGroup


class ContextParallelMixin:
  _cp: Optional[UlyssesGroup] = None

  def _cp_blocks(self) -> List[torch.nn.Module]:
    raise NotImplementedError

  def enable_context_parallel(self, config):
    group = getattr(config, "_group", None)
    exchange = None
    if config.exchange_mode() == "peer":
      from ..distributed.peer_exchange import PeerExchange
      exchange = PeerExchange(group, fp8=bool(config.ulysses_float8))
    elif config.ulysses_float8:
      raise NotImplementedError("FP8 head/token exchange is built for the peer-memory exchange only "
                                "(parallel_kwargs={'exchange': 'peer'})")
    self._cp = UlyssesGroup(group, exchange)
    for block in self._cp_blocks():
      block.cp = self._cp

  def disable_context_parallel(self):
    if self._cp is not None and self._cp.exchange is not None:
      self._cp.exchange.close()
    self._cp = None
    for block in self._cp_blocks():
      block.cp = None

  def cp_active(self) -> bool:
    return self._cp is not None and self._cp.world > 1

  def cp_shard(self, t: torch.Tensor, dim: int) -> torch.Tensor:
    """This rank's piece of `t` along `dim` (sizes differ by at most one)."""
    if not self.cp_active():
      return t
    return torch.tensor_split(t, self._cp.world, dim=dim)[self._cp.rank]

  def cp_gather(self, t: torch.Tensor, dim: int, total: int) -> torch.Tensor:
    """Concatenate every rank's piece along `dim`; `total` is the unsharded extent."""
    if not self.cp_active():
      return t
    import torch.distributed as dist
    cp = self._cp
    sizes = [len(c) for c in torch.tensor_split(torch.empty(total, device="meta"), cp.world)]
    cap = max(sizes)
    local = t.contiguous()
    if local.shape[dim] < cap:  # pad to the common size so that one equal-sized all-gather does it
      pad_shape = list(local.shape)
      pad_shape[dim] = cap - local.shape[dim]
      local = torch.cat([local, local.new_zeros(pad_shape)], dim=dim)
    parts = [torch.empty_like(local) for _ in range(cp.world)]
    dist.all_gather(parts, local, group=cp.group)
    return torch.cat([p.narrow(dim, 0, n) for p, n in zip(parts, sizes)], dim=dim)
