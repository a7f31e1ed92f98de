"""CUDA-graph replay of block-list segments.

The reference recommends `torch.compile` for the transformer blocks it caches
(src/cache_dit/compile/utils.py; docs "torch.compile" section).  A tracing compiler is not part of
this package; what it buys on this path is mostly the removal of per-kernel launch cost, and a CUDA
graph does that directly: the first-n, middle and last-n segments that `CachedBlocks` runs are
static launch sequences between the host-side cache decisions, so each is captured once and
replayed as ONE launch.  A FLUX-shape step has ~1150 kernel launches; eager Python issues them at
about the rate the GPU retires them, so every host synchronisation of the cache decision leaves
the GPU idle while the queue refills.

Rules of the runner
  * a segment is keyed by (tag, input shapes / dtypes / strides, constant arguments); the first
    `warmup_calls` calls of a key run eagerly (lazy initialisation happens there), the next call is
    captured, later calls replay;
  * inputs are copied into the capture's static input tensors, outputs are cloned out of its static
    outputs, so callers may keep references across steps (the cache context does);
  * anything the runner cannot capture (CPU tensors, autograd, an exception during capture) runs
    eagerly, and a key whose capture failed is not tried again.
"""
from __future__ import annotations

import logging
from typing import Any, Callable, Dict, List, Tuple

import torch

logger = logging.getLogger("cache_dit_b200")


def _flatten(obj: Any, tensors: List[torch.Tensor]):
  """Replace every tensor in a nest of tuples / lists / dicts by its index in `tensors`; return a
  hashable description of the nest with constants in place."""
  if isinstance(obj, torch.Tensor):
    tensors.append(obj)
    return ("T", len(tensors) - 1)
  if isinstance(obj, (tuple, list)):
    return ("L" if isinstance(obj, list) else "U", tuple(_flatten(o, tensors) for o in obj))
  if isinstance(obj, dict):
    return ("D", tuple((k, _flatten(v, tensors)) for k, v in obj.items()))
  hash(obj)  # constants must be hashable: they are part of the key
  return ("C", obj)


def _rebuild(spec: Any, tensors: List[torch.Tensor]):
  kind, payload = spec
  if kind == "T":
    return tensors[payload]
  if kind == "U":
    return tuple(_rebuild(s, tensors) for s in payload)
  if kind == "L":
    return [_rebuild(s, tensors) for s in payload]
  if kind == "D":
    return {k: _rebuild(s, tensors) for k, s in payload}
  return payload


class _Segment:
  __slots__ = ("calls", "graph", "static_in", "static_out", "out_spec", "failed", "native_launches")

  def __init__(self):
    self.calls = 0
    self.graph = None
    self.static_in: List[torch.Tensor] = []
    self.static_out: List[torch.Tensor] = []
    self.out_spec = None
    self.failed = False
    self.native_launches = 0


class BlockGraphRunner:
  """Captures and replays `fn(*inputs)` per key.  One runner per `CachedBlocks` instance."""

  def __init__(self, warmup_calls: int = 2):
    self.warmup_calls = max(1, int(warmup_calls))
    self.enabled = True
    self.segments: Dict[Tuple, _Segment] = {}
    self.replays = 0
    self.captures = 0

  def reset(self):
    self.segments.clear()

  @staticmethod
  def _capturable(tensors: List[torch.Tensor]) -> bool:
    if not tensors or torch.is_grad_enabled() and any(t.requires_grad for t in tensors):
      return False
    dev = tensors[0].device
    return dev.type == "cuda" and all(t.device == dev for t in tensors)

  def run(self, tag: Tuple, fn: Callable, inputs: Tuple):
    """fn(*inputs) -> nest of tensors.  `inputs` is a nest of tensors and hashable constants."""
    if not self.enabled:
      return fn(*inputs)
    flat: List[torch.Tensor] = []
    try:
      spec = _flatten(tuple(inputs), flat)
    except TypeError:  # an unhashable constant: nothing to key on
      return fn(*inputs)
    if not self._capturable(flat):
      return fn(*inputs)
    key = (tag, spec, tuple((tuple(t.shape), t.dtype, tuple(t.stride())) for t in flat))
    seg = self.segments.get(key)
    if seg is None:
      seg = self.segments[key] = _Segment()
    if seg.failed:
      return fn(*inputs)
    if seg.graph is None:
      seg.calls += 1
      if seg.calls <= self.warmup_calls:
        return fn(*inputs)
      if not self._capture(seg, fn, spec, flat):
        return fn(*inputs)
    else:
      for s, t in zip(seg.static_in, flat):
        if s.data_ptr() != t.data_ptr():
          s.copy_(t)
    seg.graph.replay()
    self.replays += 1
    from .. import _native
    _native.launch_count += seg.native_launches
    return _rebuild(seg.out_spec, [o.clone() for o in seg.static_out])

  def _capture(self, seg: _Segment, fn: Callable, spec, flat: List[torch.Tensor]) -> bool:
    from .. import _native
    try:
      seg.static_in = [t.clone() for t in flat]
      torch.cuda.synchronize()
      graph = torch.cuda.CUDAGraph()
      before = _native.launch_count
      with torch.cuda.graph(graph):
        out = fn(*_rebuild(spec, seg.static_in))
      seg.native_launches = _native.launch_count - before
      _native.launch_count = before  # nothing ran during capture; the replay below counts
      outs: List[torch.Tensor] = []
      seg.out_spec = _flatten(out, outs)
      seg.static_out = outs
      seg.graph = graph
      self.captures += 1
      return True
    except Exception as e:  # leave the eager path in charge of this key
      logger.warning(f"CUDA-graph capture of segment {seg!r} failed ({type(e).__name__}: {e}); running it eagerly.")
      seg.failed = True
      seg.graph = None
      seg.static_in, seg.static_out = [], []
      return False


def enable_cuda_graphs(module_or_pipe, warmup_calls: int = 2) -> int:
  """Give every `CachedBlocks` runner under a module (or a pipeline's transformer(s)) a graph runner.
  Call after `enable_cache`.  Returns the number of runners switched on."""
  from .cache_blocks import CachedBlocks
  n = 0
  for root in _roots(module_or_pipe):
    cp = getattr(root, "_cp", None)
    if cp is not None and getattr(cp, "world", 1) > 1 and getattr(cp, "exchange", None) is None:
      # NCCL all-to-all inside a captured segment hung on two GPUs; only the peer-memory exchange
      # (fixed addresses, plain kernels) is replayed from graphs
      logger.warning(f"{root.__class__.__name__}: context parallelism over NCCL all-to-all is not captured in CUDA "
                     "graphs; use the peer exchange (ParallelismConfig(parallel_kwargs={'exchange': 'peer'})).")
      continue
    for m in _cached_blocks_of(root):
      if isinstance(m, CachedBlocks):
        m.graph_runner = BlockGraphRunner(warmup_calls)
        n += 1
  return n


def disable_cuda_graphs(module_or_pipe) -> None:
  from .cache_blocks import CachedBlocks
  for root in _roots(module_or_pipe):
    for m in _cached_blocks_of(root):
      if isinstance(m, CachedBlocks):
        m.graph_runner = None


def graph_runners(module_or_pipe) -> List[BlockGraphRunner]:
  from .cache_blocks import CachedBlocks
  return [m.graph_runner for root in _roots(module_or_pipe) for m in _cached_blocks_of(root)
          if isinstance(m, CachedBlocks) and m.graph_runner is not None]


def _roots(obj) -> List[torch.nn.Module]:
  if isinstance(obj, torch.nn.Module):
    return [obj]
  roots = []
  for name in ("transformer", "transformer_2"):
    t = getattr(obj, name, None)
    for m in (t if isinstance(t, (list, tuple)) else [t]):
      if isinstance(m, torch.nn.Module) and all(m is not r for r in roots):
        roots.append(m)
  pipe = getattr(obj, "pipe", None)  # a BlockAdapter
  if not roots and pipe is not None and pipe is not obj:
    return _roots(pipe)
  return roots


def _cached_blocks_of(root: torch.nn.Module):
  """The cached runners of a transformer: those installed in the module tree and those the cache
  adapter keeps aside and swaps in during forward."""
  from .cache_blocks import CachedBlocks as CachedBlocks_
  seen = set()
  for m in root.modules():
    if id(m) not in seen:
      seen.add(id(m))
      yield m
  holder = getattr(root, "_unified_blocks", None)  # {context name: ModuleList([CachedBlocks])}
  for runners in (holder.values() if isinstance(holder, dict) else ()):
    for m in runners.modules():
      if isinstance(m, CachedBlocks_) and id(m) not in seen:
        seen.add(id(m))
        yield m
