"""xn_b200: a B200-native (sm_100a) GGUF block-quantized matmul path behind xn-core's quantized-linear API."""
from .dtypes import GgmlDType  # noqa: F401
