"""B200-native weight-only quantized matmul (drop-in for the reference's
examples/quantization/matmul_a16wx.py operator surface)."""
from .dtypes import *  # noqa: F401,F403
from .linear import QuantizedLinear  # noqa: E402,F401
from .ops import dequantize, quantized_matmul  # noqa: E402,F401
