"""Ulysses exchange around attention over peer memory (NVLink stores) instead of NCCL all-to-all.

Each rank owns four buffers that every rank of the group maps through CUDA IPC:

    q, k, v   [batch, tokens_all, heads / W, head_dim]   written by ALL ranks (each its token rows)
    o         [batch, tokens_all / W, heads, head_dim]   written by ALL ranks (each its heads)

and `W` 32-bit flag words.  Per attention call a rank (1) scatters its q, k (normalised and rotated
in the same kernel) and v into the owners' q/k/v buffers, (2) signals and waits, (3) runs attention
on its own heads over all tokens, (4) scatters the output rows to the token owners' `o` buffers,
(5) signals and waits, (6) reads its `o`.  One buffer set serves every block: a rank can reach step
(1) of the next block only after all ranks passed the second wait of this one, and step (4) only
after all ranks passed the first wait, so nothing is overwritten while it is still being read.

All launches have fixed addresses, so block segments including the exchange are CUDA-graph
capturable; the reference's plan for the same step is four all-to-all collectives per block
(src/cache_dit/distributed/transformers/flux.py:49-61).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from .. import _native


class _DeviceBuffer:
  """A raw device allocation exposed to torch through the CUDA array interface."""

  def __init__(self, ptr: int, shape: Tuple[int, ...], typestr: str):
    self.__cuda_array_interface__ = {"shape": tuple(shape), "typestr": typestr, "data": (ptr, False), "version": 3,
                                     "strides": None}


def _as_tensor(ptr: int, shape, dtype: torch.dtype, device) -> torch.Tensor:
  carrier = {2: ("<i2", torch.int16), 4: ("<i4", torch.int32)}[torch.empty((), dtype=dtype).element_size()]
  t = torch.as_tensor(_DeviceBuffer(ptr, tuple(shape), carrier[0]), device=device)
  return t.view(dtype)


class PeerExchange:
  """Buffers, flags and launch helpers of one rank.  Construction and `ensure` are collective."""

  def __init__(self, group=None, device: Optional[torch.device] = None, timeout_s: float = 10.0, fp8: bool = False):
    # fp8: e4m3 bytes + one scale per (token, head) cross NVLink instead of bf16 (the reference's
    # `ulysses_float8`, src/cache_dit/distributed/core/_distributed_primitives.py:741-813); the receiver unpacks
    self.fp8 = bool(fp8)
    self.group = group
    self.world = dist.get_world_size(group)
    self.rank = dist.get_rank(group)
    if self.world > 8:
      raise NotImplementedError("peer-memory Ulysses exchange supports up to 8 ranks (one NVSwitch domain)")
    self.device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    self.timeout_ns = int(timeout_s * 1e9)
    self._owned: List[int] = []
    self._imported: List[int] = []
    self._shape_key = None
    self.buffers: Dict[str, torch.Tensor] = {}
    self.ptrs: Dict[str, List[int]] = {}
    flags_ptr, self.flag_ptrs = self._alloc_shared(256)
    self.flags = _as_tensor(flags_ptr, (64, ), torch.int32, self.device)
    # {epoch, status}: the first exchange of a device keeps them in the device's mailbox, so that the status
    # a run-out wait latches reaches the host with the per-step copy of the cache decision
    # (`DeviceStepOps.rel_l1_means` raises on it); further exchanges on one device keep words of their own
    assert _native.lib().cdb_peer_sync_bytes() == 8
    self._mailbox_sync = True
    self.sync = _native.claim_peer_sync(self.device)
    if self.sync is None:
      self._mailbox_sync = False
      self.sync = torch.zeros(2, dtype=torch.int32, device=self.device)

  # ---- collective allocation
  def _alloc_shared(self, nbytes: int) -> Tuple[int, List[int]]:
    with torch.cuda.device(self.device):
      own = _native.peer_alloc(nbytes)
      self._owned.append(own)
      handles = [None] * self.world
      dist.all_gather_object(handles, _native.peer_export(own), group=self.group)
      ptrs = []
      for r, h in enumerate(handles):
        if r == self.rank:
          ptrs.append(own)
        else:
          p = _native.peer_import(h)
          self._imported.append(p)
          ptrs.append(p)
    return own, ptrs

  def ensure(self, batch: int, tokens_local: int, heads: int, head_dim: int, dtype: torch.dtype):
    """Allocate (first call, collective) the exchange buffers for this attention shape.  Ranks may hold
    different numbers of tokens; everyone learns all counts here."""
    key = (batch, tokens_local, heads, head_dim, dtype)
    if key == self._shape_key:
      return
    if self._shape_key is not None:
      raise RuntimeError("peer-memory Ulysses exchange: one attention shape per model "
                         f"(have {self._shape_key}, asked for {key})")
    if heads % self.world:
      raise ValueError(f"heads ({heads}) must divide by the Ulysses degree ({self.world})")
    counts = [None] * self.world
    dist.all_gather_object(counts, int(tokens_local), group=self.group)
    self.row_starts = [0]
    for c in counts:
      self.row_starts.append(self.row_starts[-1] + c)
    self.tokens_local = tokens_local
    self.capacity = max(counts)
    self.uneven = len(set(counts)) > 1
    esz = torch.empty((), dtype=dtype).element_size()
    hpr, all_tokens = heads // self.world, self.row_starts[-1]
    self.head_dim = head_dim
    if not self.fp8:
      for name in ("q", "k", "v"):
        shape = (batch, all_tokens, hpr, head_dim)
        own, self.ptrs[name] = self._alloc_shared(batch * all_tokens * hpr * head_dim * esz)
        self.buffers[name] = _as_tensor(own, shape, dtype, self.device)
      shape = (batch, self.capacity, heads, head_dim)
      own, self.ptrs["o"] = self._alloc_shared(batch * self.capacity * heads * head_dim * esz)
      self.buffers["o"] = _as_tensor(own, shape, dtype, self.device)
    else:
      if dtype != torch.bfloat16:
        raise NotImplementedError("FP8 exchange packs bf16 activations")
      for name in ("q", "k", "v"):
        n = batch * all_tokens * hpr
        own, self.ptrs[name] = self._alloc_shared(n * head_dim)
        self.buffers[name + "8"] = _as_tensor(own, (n * head_dim // 4, ), torch.int32, self.device)
        own, self.ptrs[name + "_scale"] = self._alloc_shared(n * 4)
        self.buffers[name + "_scale"] = _as_tensor(own, (n, ), torch.float32, self.device)
        self.buffers[name] = torch.empty(batch, all_tokens, hpr, head_dim, dtype=dtype, device=self.device)
      n = batch * self.capacity * heads
      own, self.ptrs["o"] = self._alloc_shared(n * head_dim)
      self.buffers["o8"] = _as_tensor(own, (n * head_dim // 4, ), torch.int32, self.device)
      own, self.ptrs["o_scale"] = self._alloc_shared(n * 2)
      self.buffers["o_scale"] = _as_tensor(own, (n, ), torch.bfloat16, self.device)
      self.buffers["o"] = torch.empty(batch, self.capacity, heads, head_dim, dtype=dtype, device=self.device)
    self._shape_key = key
    dist.barrier(group=self.group)

  # ---- launches
  def scatter(self, name: str, x: torch.Tensor, heads: int, row_offset_local: int, norm_weight=None, cos=None,
              sin=None, eps: float = 0.0, across_heads: bool = False):
    """x [batch, t, heads*head_dim]: this rank's rows [row_offset_local, +t) of its token shard."""
    if self.fp8:
      return self.scatter_jobs([self.scatter_job(name, x, row_offset_local, norm_weight, cos, sin, eps, across_heads)],
                               heads)
    buf = self.buffers[name]
    _native.scatter_heads(x, norm_weight, cos, sin, row_offset_local, self.ptrs[name], buf.stride(0),
                          self.row_starts[self.rank] + row_offset_local, heads, eps, across_heads)

  def scatter_job(self, name: str, x: torch.Tensor, row_offset_local: int, norm_weight=None, cos=None, sin=None,
                  eps: float = 0.0, across_heads: bool = False) -> dict:
    """The same scatter as a job description for `scatter_jobs` (several in one launch)."""
    return dict(x=x, norm_weight=norm_weight, cos=cos, sin=sin, table_row_offset=row_offset_local,
                dst_ptrs=self.ptrs[name], dst_batch_stride=self.buffers[name].stride(0),
                dst_row_offset=self.row_starts[self.rank] + row_offset_local, eps=eps, across_heads=across_heads,
                dst_scale_ptrs=self.ptrs[name + "_scale"] if self.fp8 else None)

  def scatter_jobs(self, jobs, heads: int):
    for i in range(0, len(jobs), 6):
      _native.scatter_heads_multi(jobs[i:i + 6], heads)

  def barrier(self):
    _native.peer_barrier(self.flag_ptrs, self.flags, self.rank, self.sync, self.timeout_ns)

  def qkv_ready(self):
    """After the scatters of all ranks: wait for them, and unpack the FP8 wire format if it is in use."""
    self.barrier()
    if self.fp8:
      b = self.buffers
      _native.fp8_dequant_heads([b["q8"], b["k8"], b["v8"]], [b["q_scale"], b["k_scale"], b["v_scale"]],
                                [b["q"], b["k"], b["v"]], self.head_dim)

  def gather_output(self, o_local: torch.Tensor) -> torch.Tensor:
    """o_local [batch, tokens_all, heads / W, head_dim] -> this rank's `o` buffer after the exchange."""
    if self.fp8:
      _native.gather_tokens_fp8(o_local, self.ptrs["o"], self.ptrs["o_scale"], self.rank, self.row_starts, self.capacity)
      self.barrier()
      b = self.buffers
      _native.fp8_dequant_heads([b["o8"]], [b["o_scale"]], [b["o"]], self.head_dim)
    else:
      _native.gather_tokens(o_local, self.ptrs["o"], self.rank, self.row_starts, self.capacity)
      self.barrier()
    out = self.buffers["o"]
    return out if self.tokens_local == self.capacity else out[:, :self.tokens_local]

  def status(self) -> int:
    """0, or 1 + the index of a peer whose signal did not arrive within the timeout (synchronises)."""
    return int(self.sync[1].item())

  def close(self):
    for p in self._imported:
      _native.peer_release(p)
    self._imported.clear()
    if dist.is_initialized():
      dist.barrier(group=self.group)
    for p in self._owned:
      _native.peer_free(p)
    self._owned.clear()
    self.buffers.clear()
    if self._mailbox_sync:
      self.sync.zero_()  # a latched status belongs to this exchange, not to whatever runs on the device next
      _native.release_peer_sync(self.device)
      self._mailbox_sync = False
