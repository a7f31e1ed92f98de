"""B200-native (sm_100a) hot path behind cache-dit's public API.

    import cache_dit_b200 as cache_dit
    cache_dit.enable_cache(pipe_or_adapter_or_transformer,
                           cache_config=cache_dit.DBCacheConfig(...),
                           calibrator_config=cache_dit.TaylorSeerCalibratorConfig(...),
                           parallelism_config=cache_dit.ParallelismConfig(ulysses_size=8),
                           quantize_config=cache_dit.QuantizeConfig(quant_type="float8_per_row"))

The names exported here are those of the reference package (src/cache_dit/__init__.py:19-82) that
belong to the DBCache / TaylorSeer / FP8-linear / Ulysses path.
"""
from .caching import (BasicCacheConfig, BlockAdapter, BlockGraphRunner, disable_cuda_graphs, enable_cuda_graphs,
                      graph_runners, BlockAdapterRegister, CachedAdapter, CachedBlocks,
                      CachedContext, CachedContextManager, CacheType, Calibrator, CalibratorBase,
                      CalibratorConfig, ContextNotExistError, DBCacheConfig, ExtraCacheConfig,
                      FakeDiffusionPipeline, ForwardPattern, LazyResidual, ParamsModifier, TaylorSeerCalibrator,
                      TaylorSeerCalibratorConfig, UnifiedBlocks, block_range, cache_type, disable_cache,
                      enable_cache, get_adapter, load_attn_backend_config, load_cache_config, load_configs,
                      load_options, load_parallelism_config, load_quantize_config, refresh_context, steps_mask,
                      supported_pipelines)
from .distributed import ParallelismBackend, ParallelismConfig, enable_parallelism
from .quantization import Float8RowwiseLinear, QuantizeBackend, QuantizeConfig, quantize
from .summary import CacheStats, strify, summary
from . import synthetic  # registers the block adapters of the DiT stand-ins

NONE = CacheType.NONE
DBCache = CacheType.DBCache

Pattern_0 = ForwardPattern.Pattern_0
Pattern_1 = ForwardPattern.Pattern_1
Pattern_2 = ForwardPattern.Pattern_2
Pattern_3 = ForwardPattern.Pattern_3
Pattern_4 = ForwardPattern.Pattern_4
Pattern_5 = ForwardPattern.Pattern_5

__version__ = "0.1.0"
