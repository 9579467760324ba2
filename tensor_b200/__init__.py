"""B200-native (sm_100a) GGUF dequant-fused GEMV / GEMM behind the Tensor runtime's contract.

The arithmetic lives in ``tensor_b200/csrc`` (CUDA) behind the C ABI of
``include/tensor_b200_gguf.h``; this package is the thin Python host layer over it.  Importing the
package does not load the library; the first operation does, and fails loudly if it is absent.
"""

from ._native import AbiError, LIB_PATH, TensorRuntimeError
from .formats import Q4_0, Q4_K, Q6_K, Q8_0, BlockFormat, get_format
from .kernel import GgufKernel, gguf
from .ops import (GemvList, dequantize, device_status, gemm, gemv, gemv_plan, gemv_scratch_bytes,
                  set_peer_wait_limit, weight_bytes)

__all__ = [
    "AbiError", "BlockFormat", "GemvList", "GgufKernel", "LIB_PATH", "Q4_0", "Q4_K", "Q6_K", "Q8_0",
    "TensorRuntimeError", "dequantize", "device_status", "gemm", "gemv", "gemv_scratch_bytes",
    "gemv_plan", "get_format", "gguf", "set_peer_wait_limit", "weight_bytes",
]
