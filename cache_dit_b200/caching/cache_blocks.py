"""The cached block runner: first-n / middle / last-n execution of a transformer block list.

One class covers all six block contracts (`ForwardPattern`).  It follows the step protocol of the
reference's runners (src/cache_dit/caching/cache_blocks/pattern_base.py:198-321 for patterns 0-2,
.../pattern_3_4_5.py:80-205 for patterns 3-5):

    run first Fn blocks -> indicator = hidden - input -> mark_step_begin -> can_cache?
      hit : add_cached_step, hidden <- forecast + hidden, run last Bn blocks
      miss: store indicator, run middle blocks, store (hidden - hidden_before_middle) for the
            forecast, run last Bn blocks

but never materialises the two residuals itself: it hands `LazyResidual` objects to the context
manager, which fuses the subtraction into the relative-L1 kernel (hit/miss check) and into the
TaylorSeer update kernel.
"""
from __future__ import annotations

import inspect
import logging
from typing import Optional

import torch
import torch.distributed as dist

from .cache_manager import CachedContextManager, ContextNotExistError, LazyResidual
from .cache_types import CacheType
from .forward_pattern import ForwardPattern

logger = logging.getLogger("cache_dit_b200")


class CachedBlocks(torch.nn.Module):
  _supported_patterns = ForwardPattern.supported_patterns()

  def __init__(self, transformer_blocks: torch.nn.ModuleList, transformer: torch.nn.Module = None,
               forward_pattern: ForwardPattern = ForwardPattern.Pattern_0,
               check_forward_pattern: bool = True, check_num_outputs: bool = True,
               cache_prefix: str = None, cache_context=None,
               context_manager: CachedContextManager = None, cache_type: CacheType = CacheType.DBCache,
               **kwargs):
    super().__init__()
    assert transformer is not None, "transformer can't be None."
    assert forward_pattern is not None, "forward_pattern can't be None."
    assert cache_context is not None, "cache_context can't be None."
    assert context_manager is not None, "context_manager can't be None."
    assert cache_type == CacheType.DBCache, f"Cache type {cache_type} is not supported for CachedBlocks."
    # the transformer is referenced, not registered as a sub-module (it owns this runner)
    object.__setattr__(self, "transformer", transformer)
    self.transformer_blocks = transformer_blocks
    self.forward_pattern = forward_pattern
    self.check_forward_pattern = check_forward_pattern
    self.check_num_outputs = check_num_outputs
    self.cache_prefix = cache_prefix
    self.cache_context = cache_context
    self.context_manager = context_manager
    self.cache_type = cache_type
    # optional CUDA-graph replay of the block segments (block_graphs.enable_cuda_graphs)
    self.graph_runner = None
    self._check_forward_pattern()

  # ---------------------------------------------------------------- checks
  def _check_forward_pattern(self):
    if not self.check_forward_pattern:
      return
    assert self.forward_pattern.Supported and self.forward_pattern in self._supported_patterns, (
      f"Pattern {self.forward_pattern} is not supported now!")
    for block in self.transformer_blocks:
      inner = getattr(block, "block", None)
      if isinstance(inner, torch.nn.Module):
        block = inner
      sig = inspect.signature(block.forward)
      if self.check_num_outputs:
        num_outputs = str(sig.return_annotation).count("torch.Tensor")
        if num_outputs > 0:
          assert len(self.forward_pattern.Out) == num_outputs, (
            f"The number of block's outputs is {num_outputs} don't not match the number of the "
            f"pattern: {self.forward_pattern}, Out: {len(self.forward_pattern.Out)}.")
      for required in self.forward_pattern.In:
        assert required in sig.parameters, f"The input parameters must contains: {required}."

  def _check_cache_params(self):
    n = len(self.transformer_blocks)
    assert self.context_manager.Fn_compute_blocks() <= n, (
      f"Fn_compute_blocks {self.context_manager.Fn_compute_blocks()} must be less than "
      f"the number of transformer blocks {n}")
    assert self.context_manager.Bn_compute_blocks() <= n, (
      f"Bn_compute_blocks {self.context_manager.Bn_compute_blocks()} must be less than "
      f"the number of transformer blocks {n}")

  def _is_parallelized(self) -> bool:
    if getattr(self.transformer, "_is_parallelized", False):
      return True
    return dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1

  # ---------------------------------------------------------------- block calls
  def _unpack(self, out, encoder):
    """Normalise one block's return value to (hidden, encoder)."""
    if isinstance(out, torch.Tensor):
      return out, (None if self.forward_pattern.Forward_H_only else encoder)
    if self.forward_pattern.Forward_H_only:
      if len(out) == 1:
        return out[0], None
      assert len(out) == 2, f"Unexpected output length: {len(out)}"
      if isinstance(out[1], torch.Tensor):
        a, b = out
        return (a, b) if self.forward_pattern.Return_H_First else (b, a)
      if isinstance(out[0], torch.Tensor):
        return out[0], None
      raise ValueError("Unexpected hidden_states format.")
    a, b = out
    return (a, b) if self.forward_pattern.Return_H_First else (b, a)

  def _run(self, blocks, hidden, encoder, args, kwargs):
    # A model may want to get per-call work for exactly the blocks that are about to run out of the way first
    # (e.g. their adaLN modulation vectors as one product): it is told here, outside any captured graph.
    prepare = getattr(self.transformer, "prepare_blocks", None)
    if prepare is not None and len(blocks) > 0:
      prepare(blocks)
    runner = self.graph_runner
    if runner is None or len(blocks) == 0:
      return self._run_eager(blocks, hidden, encoder, args, kwargs)
    tag = (id(blocks[0]), len(blocks))
    return runner.run(tag, lambda h, e, a, k: self._run_eager(blocks, h, e, a, k),
                      (hidden, encoder, tuple(args), dict(kwargs)))

  def _run_eager(self, blocks, hidden, encoder, args, kwargs):
    h_only = self.forward_pattern.Forward_H_only
    if h_only:
      encoder = None
    for block in blocks:
      out = block(hidden, *args, **kwargs) if h_only else block(hidden, encoder, *args, **kwargs)
      hidden, encoder = self._unpack(out, encoder)
    return hidden, encoder

  def _pack(self, hidden, encoder):
    p = self.forward_pattern
    if p.Return_H_Only:
      return hidden
    return (hidden, encoder) if p.Return_H_First else (encoder, hidden)

  def _split(self):
    fn = self.context_manager.Fn_compute_blocks()
    bn = self.context_manager.Bn_compute_blocks()
    blocks = self.transformer_blocks
    n = len(blocks)
    return blocks[:fn], blocks[fn:n - bn if bn > 0 else n], (blocks[n - bn:] if bn > 0 else [])

  def call_blocks(self, hidden_states, encoder_hidden_states=None, *args, **kwargs):
    """All blocks, no caching."""
    return self._run(self.transformer_blocks, hidden_states, encoder_hidden_states, args, kwargs)

  # ---------------------------------------------------------------- forward
  def forward(self, hidden_states: torch.Tensor, *args, **kwargs):
    h_only = self.forward_pattern.Forward_H_only
    encoder = None
    if not h_only:
      if args:
        encoder, args = args[0], args[1:]
      else:
        encoder = kwargs.pop("encoder_hidden_states", None)
    cm = self.context_manager
    try:
      cm.set_context(self.cache_context)
      self._check_cache_params()
    except ContextNotExistError as e:
      logger.warning(f"Cache context not exist: {e}, skip cache.")
      return self._pack(*self._run(self.transformer_blocks, hidden_states, encoder, args, kwargs))

    name = self.cache_prefix
    fn_blocks, mn_blocks, bn_blocks = self._split()
    original = hidden_states
    hidden, encoder = self._run(fn_blocks, hidden_states, encoder, args, kwargs)
    # Indicator of the step: the change the first blocks made.  When the sequence was sharded
    # inside the first block (context parallelism applied at block level) input and output have
    # different shapes and the post-Fn hidden states stand in for the residual.
    if original.shape == hidden.shape:
      indicator = LazyResidual(hidden, original.to(hidden.device))
    else:
      indicator = hidden
    del original

    cm.mark_step_begin()
    l1 = cm.is_l1_diff_enabled()
    hit = cm.can_cache(hidden if l1 else indicator, parallelized=self._is_parallelized(),
                       prefix=f"{name}_Fn_hidden_states" if l1 else f"{name}_Fn_residual")
    bn_prefix = f"{name}_Bn_residual" if cm.is_cache_residual() else f"{name}_Bn_hidden_states"
    bn_encoder_prefix = (f"{name}_Bn_residual" if cm.is_encoder_cache_residual() else
                         f"{name}_Bn_hidden_states")
    if hit:
      cm.add_cached_step()
      del indicator
      hidden, encoder = cm.apply_cache(hidden, encoder, prefix=bn_prefix, encoder_prefix=bn_encoder_prefix)
    else:
      cm.set_Fn_buffer(indicator, prefix=f"{name}_Fn_residual")
      if l1:
        cm.set_Fn_buffer(hidden, f"{name}_Fn_hidden_states")
      del indicator
      before, encoder_before = hidden, encoder
      hidden, encoder = self._run(mn_blocks, hidden, encoder, args, kwargs)
      hidden = hidden.contiguous()
      if cm.is_cache_residual():
        cm.set_Bn_buffer(LazyResidual(hidden, before), prefix=bn_prefix)
      else:
        cm.set_Bn_buffer(hidden, prefix=bn_prefix)
      if encoder is not None and encoder_before is not None:
        encoder = encoder.contiguous()
        # blocks that take hidden states only always cache the encoder *residual*
        if h_only or cm.is_encoder_cache_residual():
          cm.set_Bn_encoder_buffer(LazyResidual(encoder, encoder_before), prefix=bn_encoder_prefix)
        else:
          cm.set_Bn_encoder_buffer(encoder, prefix=bn_encoder_prefix)
    if bn_blocks:
      hidden, encoder = self._run(bn_blocks, hidden, encoder, args, kwargs)
    return self._pack(hidden, encoder)


class UnifiedBlocks:
  """Factory kept for API compatibility: returns the runner for a cache type."""

  def __new__(cls, transformer_blocks, transformer=None, forward_pattern=None, check_forward_pattern=True,
              check_num_outputs=True, cache_prefix=None, cache_context=None, context_manager=None,
              cache_type: CacheType = CacheType.DBCache, **kwargs):
    if cache_type != CacheType.DBCache:
      raise ValueError(f"Cache type {cache_type} is not supported now!")
    return CachedBlocks(transformer_blocks, transformer=transformer, forward_pattern=forward_pattern,
                        check_forward_pattern=check_forward_pattern, check_num_outputs=check_num_outputs,
                        cache_prefix=cache_prefix, cache_context=cache_context,
                        context_manager=context_manager, cache_type=cache_type, **kwargs)


# ---------------------------------------------------------------- statistics on modules
_STATS = ("_cached_steps", "_residual_diffs", "_cfg_cached_steps", "_cfg_residual_diffs",
          "_accumulated_cached_steps", "_cfg_accumulated_cached_steps", "_accumulated_executed_steps",
          "_accumulated_transformer_executed_steps")


def apply_stats(module, cache_context=None, context_manager: Optional[CachedContextManager] = None):
  """Publish the run's statistics as attributes of `module`
  (src/cache_dit/caching/cache_blocks/pattern_utils.py:9-31)."""
  if module is None or context_manager is None:
    return
  if cache_context is not None:
    context_manager.set_context(cache_context)
  cm = context_manager
  module._cached_steps = cm.get_cached_steps()
  module._residual_diffs = cm.get_residual_diffs()
  module._cfg_cached_steps = cm.get_cfg_cached_steps()
  module._cfg_residual_diffs = cm.get_cfg_residual_diffs()
  module._accumulated_cached_steps = cm.get_accumulated_cached_steps()
  module._cfg_accumulated_cached_steps = cm.get_cfg_accumulated_cached_steps()
  module._accumulated_executed_steps = cm.get_accumulated_executed_steps()
  module._accumulated_transformer_executed_steps = cm.get_accumulated_transformer_executed_steps()


def remove_stats(module):
  if module is None:
    return
  for attr in _STATS:
    if hasattr(module, attr):
      delattr(module, attr)
