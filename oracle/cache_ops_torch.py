"""The four tensor operations of the cache step as the reference itself runs them: eager PyTorch ops, here on CPU
tensors and all host threads.

TEST INFRASTRUCTURE, NOT PRODUCT CODE: imported only by the tests and by the CPU-baseline leg of the benchmark.
PARITY: PINNED - tests/test_oracle_golden.py holds these functions against the numpy restatement
(oracle/cache_oracle.py), which is itself held bit for bit against fixtures generated from the unmodified
reference (tests/golden/make_golden.py).

The reference has no kernels for this path: what it executes is the op sequence below, so on a CPU the closest
thing to "the reference's own implementation" is the same sequence of torch ops on CPU tensors.  Each function
cites the lines it restates.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch


def residual(after: torch.Tensor, before: torch.Tensor) -> torch.Tensor:
  """Fn / Mn residual (src/cache_dit/caching/cache_blocks/pattern_base.py:195, :414)."""
  return after - before


def local_means(prev: torch.Tensor, cur: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
  """mean|t1 - t2| and mean|t1| as 0-dim tensors of the tensor dtype
  (src/cache_dit/caching/cache_contexts/cache_manager.py:609-610)."""
  return (prev - cur).abs().mean(), prev.abs().mean()


def rel_l1(prev: torch.Tensor, cur: torch.Tensor) -> float:
  """(mean_diff / mean_t1).item() (src/cache_dit/caching/cache_contexts/cache_manager.py:619)."""
  mean_diff, mean_t1 = local_means(prev, cur)
  return (mean_diff / mean_t1).item()


def taylor_derivatives(y: torch.Tensor, prev: Sequence[Optional[torch.Tensor]], window: int,
                       past_first_step: bool) -> List[Optional[torch.Tensor]]:
  """dY[0] = Y; dY[i + 1] = (dY[i] - dY_prev[i]) / window while dY_prev[i] exists
  (src/cache_dit/caching/cache_contexts/calibrators/taylorseer.py:68-89)."""
  out: List[Optional[torch.Tensor]] = [None] * len(prev)
  out[0] = y
  for i in range(len(prev) - 1):
    if prev[i] is not None and past_first_step:
      out[i + 1] = (out[i] - prev[i]) / window
    else:
      break
  return out


def taylor_series(derivs: Sequence[Optional[torch.Tensor]], elapsed: int):
  """sum_i (1 / i!) * dY[i] * elapsed**i, stopping at the first missing term
  (src/cache_dit/caching/cache_contexts/calibrators/taylorseer.py:91-104)."""
  output = 0
  for i, d in enumerate(derivs):
    if d is None:
      break
    output = output + (1 / math.factorial(i)) * d * (elapsed**i)
  return output


def apply_add(approx: torch.Tensor, hidden: torch.Tensor) -> torch.Tensor:
  """hidden_states = approximation + hidden_states (src/cache_dit/caching/cache_contexts/cache_manager.py:831)."""
  return approx + hidden
