"""Root-level Ulysses plan shared by the stand-ins: shard token tensors on entry, gather on exit.

The reference declares the same plan per model as split / gather hooks on module inputs and outputs
(src/cache_dit/distributed/transformers/flux.py:49-61, qwen_image.py:63-79, wan.py:52-65).  Token
counts that do not divide by the number of ranks are split like `torch.tensor_split` (the first
ranks hold one token more): the reference's `ulysses_anything` mode.
"""
from __future__ import annotations

import os
from typing import List, Optional

import torch

from .layers import ModulationBank, UlyssesGroup


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
    self._cp_block_list = self._cp_blocks()  # inside `forward` of a cache-enabled model the list holds the cache runner
    for block in self._cp_block_list:
      block.cp = self._cp
    self._mod_bank = None
    self._mod_bank_wanted = self._cp.world > 1 and os.environ.get("CACHE_DIT_B200_MODULATION_BANK", "1") != "0"

  def disable_context_parallel(self):
    if self._cp is not None and self._cp.exchange is not None:
      self._cp.exchange.close()
    self._cp = None
    self._mod_bank = None
    self._mod_bank_wanted = False
    for block in self._cp_blocks():
      block.cp = None
      block.mod_bank = None

  def _modulation_groups(self, blocks):
    """Per block, the linears that read only SiLU(temb) (none: the model has no per-block modulation projections)."""
    return []

  def modulation_for_call(self, temb: torch.Tensor) -> None:
    """Under context parallelism: all blocks' modulation vectors as one column-sharded product + all-gather per call
    (`ModulationBank`) instead of one replicated weight-streaming product per block and rank."""
    if not getattr(self, "_mod_bank_wanted", False) or not temb.is_cuda:
      return
    bank = self._mod_bank
    if bank is None or not bank.still_valid():
      groups = self._modulation_groups(self._cp_block_list)
      try:
        bank = ModulationBank(groups, self._cp.group) if groups else None
      except ValueError:
        bank = None
      if bank is None:
        self._mod_bank_wanted = False
        return
      self._mod_bank = bank
      self._mod_bank_index = {id(b): i for i, b in enumerate(self._cp_block_list)}
      for b in self._cp_block_list:
        b.mod_bank = bank
    bank.begin_call(temb)
    if self._runs_blocks_itself():
      bank.prepare(0, len(self._cp_block_list))

  def _runs_blocks_itself(self) -> bool:
    """False while a cache runner stands in for the block list (it announces the blocks it runs)."""
    return True

  @staticmethod
  def is_cache_runner_list(block_list) -> bool:
    """During `forward` of a cache-enabled model a block list attribute holds a one-element list with the runner."""
    return len(block_list) == 1 and hasattr(block_list[0], "context_manager") and hasattr(block_list[0], "transformer_blocks")

  def prepare_blocks(self, blocks) -> None:
    """Called by the cache runner before it runs `blocks` (a contiguous slice of the block list)."""
    bank = getattr(self, "_mod_bank", None)
    if bank is None or not getattr(self, "_mod_bank_wanted", False):
      return
    index = self._mod_bank_index
    if id(blocks[0]) in index:
      bank.prepare(index[id(blocks[0])], index[id(blocks[-1])] + 1)

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
