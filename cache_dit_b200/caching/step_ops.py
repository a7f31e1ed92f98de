"""Device operations of one cache step, as the host-side state machine sees them.

`DeviceStepOps` is the only implementation shipped: it launches the sm_100a kernels through the
C ABI and refuses anything that is not a CUDA tensor.  The indirection (`get_ops` / `set_ops`)
exists so that CPU-only tests of the host logic can plug in a checker-backed double; the package
itself never installs anything else.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch

from .. import _native

_BF16 = torch.bfloat16
_F16 = torch.float16


def round_to_dtype(value: float, dtype: torch.dtype) -> float:
  """Round a host float to the nearest value of `dtype` (ties to even), as a Python float."""
  import numpy as np
  v = np.float32(value)
  if dtype == torch.float32:
    return float(v)
  if dtype == _F16:
    with np.errstate(over="ignore"):
      return float(np.float32(np.float16(v)))
  if dtype == _BF16:
    if np.isnan(v):
      return float("nan")
    u = np.array([v], dtype=np.float32).view(np.uint32)
    bias = ((u >> np.uint32(16)) & np.uint32(1)) + np.uint32(0x7FFF)
    return float(((u + bias) & np.uint32(0xFFFF0000)).view(np.float32)[0])
  raise ValueError(f"unsupported dtype {dtype}")


def ratio_in_dtype(mean_diff: float, mean_prev: float, dtype: torch.dtype) -> float:
  """`(mean_diff / mean_t1).item()` for 0-dim tensors of `dtype`
  (src/cache_dit/caching/cache_contexts/cache_manager.py:619)."""
  import numpy as np
  with np.errstate(divide="ignore", invalid="ignore"):
    q = np.float32(mean_diff) / np.float32(mean_prev)
  return round_to_dtype(float(q), dtype)


class DeviceStepOps:
  """Launches the hot-path kernels. One instance per process."""

  name = "sm_100a"

  def __init__(self):
    self._pinned = {}  # device index -> int32[8] pinned host image of the device's mailbox

  # ---- buffers ---------------------------------------------------------------------------
  def _means_buffer(self, device: torch.device) -> torch.Tensor:
    """The two float32 means live in the device's mailbox (`_native.device_mailbox`), next to the latched
    status words of the bounded device-side waits, so that one copy brings all of them to the host."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    if idx not in self._pinned:
      self._pinned[idx] = torch.zeros(_native.MAILBOX_WORDS, dtype=torch.int32).pin_memory()
    return _native.mailbox_means(device)

  def empty_like(self, t: torch.Tensor) -> torch.Tensor:
    return torch.empty(t.shape, dtype=t.dtype, device=t.device)

  # ---- relative L1 -------------------------------------------------------------------------
  def residual(self, after: torch.Tensor, before: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """out = round(after - before) (src/cache_dit/caching/cache_blocks/pattern_base.py:195)."""
    _native.rel_l1(after, before, None, out, None)
    return out

  def rel_l1_means(self, cur: torch.Tensor, base: Optional[torch.Tensor], prev: torch.Tensor,
                   residual_out: Optional[torch.Tensor], group=None) -> Tuple[float, float, int]:
    """One fused pass, then the single host synchronisation of the step.

    Raises `_native.DeviceTimeoutError` if a bounded wait of an earlier kernel (FP8 GEMM pipeline, peer
    exchange) ran out.  Returns (mean|prev - r|, mean|prev|, world) where r = cur - base (or cur); with a process
    group the two local means are summed over the ranks by ONE all-reduce of two float32 and
    `world` is the number of ranks (the caller divides and rounds like ReduceOp.AVG would,
    src/cache_dit/caching/cache_contexts/cache_manager.py:612-614)."""
    means = self._means_buffer(cur.device)
    _native.rel_l1(cur, base, prev, residual_out, means)
    world = 1
    if group is not None:
      import torch.distributed as dist
      world = dist.get_world_size(group if group is not True else None)
      if world > 1:
        dist.all_reduce(means, op=dist.ReduceOp.SUM, group=group if group is not True else None)
    idx = cur.device.index if cur.device.index is not None else torch.cuda.current_device()
    host = self._pinned[idx]
    host.copy_(_native.device_mailbox(cur.device), non_blocking=True)
    torch.cuda.current_stream(cur.device).synchronize()
    # the same 32 bytes carry the status words: a wait that ran out since the last step invalidates what
    # was computed after it, so the step fails here instead of producing silently wrong latents
    _native.raise_on_device_status(int(host[_native.MAILBOX_GEMM_STATUS]), int(host[_native.MAILBOX_PEER_STATUS]))
    m = host[0:2].view(torch.float32)
    return float(m[0]), float(m[1]), world

  # ---- Taylor ------------------------------------------------------------------------------
  def taylor_apply(self, hidden: Optional[torch.Tensor], derivs: Sequence[torch.Tensor],
                   elapsed: int, add_hidden: bool, out: torch.Tensor) -> torch.Tensor:
    k = len(derivs)
    coef = [1.0 / math.factorial(i) for i in range(k)]
    power = [float(elapsed**i) for i in range(k)]
    _native.taylor_apply(hidden, list(derivs), coef, power, add_hidden, out)
    return out

  def taylor_update(self, after: torch.Tensor, before: Optional[torch.Tensor],
                    prev: Sequence[torch.Tensor], cur: List[torch.Tensor], n_new: int,
                    window: int) -> None:
    _native.taylor_update(after, before, list(prev), list(cur), n_new, float(window))


_ops = None


def get_ops():
  global _ops
  if _ops is None:
    _native.lib()  # raises if the CUDA library has not been built
    _ops = DeviceStepOps()
  return _ops


def set_ops(ops) -> None:
  """Install another implementation (used by CPU-only tests of the host logic)."""
  global _ops
  _ops = ops
