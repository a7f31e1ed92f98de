from .block_adapters import (BlockAdapter, BlockAdapterRegister, FakeDiffusionPipeline, ParamsModifier)
from .block_graphs import BlockGraphRunner, disable_cuda_graphs, enable_cuda_graphs, graph_runners
from .cache_adapter import CachedAdapter
from .cache_blocks import CachedBlocks, UnifiedBlocks, apply_stats, remove_stats
from .cache_config import BasicCacheConfig, DBCacheConfig, ExtraCacheConfig
from .cache_context import CachedContext
from .cache_interface import (disable_cache, enable_cache, get_adapter, refresh_context, steps_mask,
                              supported_pipelines)
from .cache_manager import CachedContextManager, ContextNotExistError, LazyResidual
from .cache_types import CacheType, block_range, cache_type
from .calibrators import (Calibrator, CalibratorBase, CalibratorConfig, TaylorSeerCalibrator,
                          TaylorSeerCalibratorConfig, TaylorSeerState)
from .forward_pattern import ForwardPattern
from .load_configs import (load_attn_backend_config, load_cache_config, load_configs, load_options,
                           load_parallelism_config, load_quantize_config)
