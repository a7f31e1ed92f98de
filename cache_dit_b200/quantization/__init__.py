from .config import QuantizeBackend, QuantizeConfig
from .linear import (Float8RowwiseLinear, FusedFloat8Linears, fused_group, grouped_forward_quantized,
                     quantize_rows_fused)
from .quantize import quantize, remove_quantization_stats
from . import ops
