from .config import QuantizeBackend, QuantizeConfig
from .linear import (Float8RowwiseLinear, FusedFloat8Linears, fused_group, grouped_forward_quantized,
                     quantize_rows_fused, quantize_rows_fused_pair)
from .quantize import quantize, remove_quantization_stats
from . import ops
