"""Random-init DiT stand-ins (FLUX-, Qwen-Image-, Wan-shape) and a minimal denoising loop.

No weights, prompts or datasets are involved: the modules only reproduce layer shapes and data
flow so that the cache engine, the FP8 linears and the context-parallel plan can be run and timed.
Importing this package registers their block adapters.
"""
from .flux import FluxSingleTransformerBlock, FluxTransformer2DModel, FluxTransformerBlock
from .qwen_image import QwenImageTransformer2DModel, QwenImageTransformerBlock
from .wan import WanTransformer3DModel, WanTransformerBlock
from .pipeline import DenoisePipeline, FluxDenoisePipeline, QwenImageDenoisePipeline, WanDenoisePipeline
