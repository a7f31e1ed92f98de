"""A stand-in for the device step-ops, backed by the numpy oracle, for CPU-only tests of the host
logic (state machine, adapters, block runner).  It is installed with
`cache_dit_b200.caching.step_ops.set_ops` by a fixture and never ships."""
from __future__ import annotations


import numpy as np
import torch

from oracle import cache_oracle as O

NAME = {torch.float32: "fp32", torch.bfloat16: "bf16", torch.float16: "fp16"}


def _np(t):
  return t.detach().float().cpu().numpy()


def _put(out: torch.Tensor, values: np.ndarray):
  out.copy_(torch.from_numpy(np.ascontiguousarray(values)).to(out.dtype).view(out.shape))
  return out


class OracleStepOps:
  name = "oracle-double"

  def __init__(self):
    self.calls = []

  def empty_like(self, t):
    return torch.empty(t.shape, dtype=t.dtype, device=t.device)

  def residual(self, after, before, out):
    self.calls.append("residual")
    return _put(out, O.residual(_np(after), _np(before), NAME[after.dtype]))

  def rel_l1_means(self, cur, base, prev, residual_out, group=None):
    self.calls.append("rel_l1_fused" if base is not None else "rel_l1")
    dt = NAME[cur.dtype]
    r = _np(cur) if base is None else O.residual(_np(cur), _np(base), dt)
    if residual_out is not None:
      _put(residual_out, r)
    md, mp = O.local_means(_np(prev), r, dt)
    world = 1
    if group is not None:
      import torch.distributed as dist
      world = dist.get_world_size()
      if world > 1:
        buf = torch.tensor([float(md), float(mp)], dtype=torch.float32)
        dist.all_reduce(buf, op=dist.ReduceOp.SUM)
        md, mp = float(buf[0]), float(buf[1])
    return float(md), float(mp), world

  def taylor_apply(self, hidden, derivs, elapsed, add_hidden, out):
    self.calls.append(f"apply{len(derivs)}")
    dt = NAME[out.dtype]
    approx = O.taylor_series([_np(d) for d in derivs], elapsed, dt)
    return _put(out, O.apply_add(approx, _np(hidden), dt) if add_hidden else approx)

  def taylor_update(self, after, before, prev, cur, n_new, window):
    self.calls.append(f"update{n_new}" + ("_fused" if before is not None else ""))
    dt = NAME[after.dtype]
    y = _np(after) if before is None else O.residual(_np(after), _np(before), dt)
    ladder = O.taylor_derivatives(y, [_np(p) for p in prev[:n_new]] + [None], window, True, dt)
    if before is not None or cur[0] is not after:
      _put(cur[0], ladder[0])
    for k in range(n_new):
      _put(cur[k + 1], ladder[k + 1])
