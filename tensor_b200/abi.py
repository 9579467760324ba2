"""ctypes mirrors of the runtime ABI 1.3 structs the C library consumes.

Layouts are the reference's frozen ones (src/tensor/include/tensor/abi.h:37-85; Python mirrors in
src/tensor/runtime/abi.py:50-119): 48 / 64 / 16 / 72 / 512 bytes.
"""

from __future__ import annotations

import ctypes

ABI_VERSION = 1
DEVICE_CUDA = 2
ARG_BUFFER = 1
ARG_SCALAR = 2
OK, ERROR_ABI, ERROR_ARGUMENT, ERROR_PROVIDER = 0, 1, 2, 3

DTYPE_IDS = {"uint8": 3, "int32": 6, "int64": 8, "float16": 10, "float32": 11, "bfloat16": 13}
DTYPE_BYTES = {3: 1, 6: 4, 8: 8, 10: 2, 11: 4, 13: 2}


class TensorBufferV1(ctypes.Structure):
    _fields_ = [("address", ctypes.c_uint64), ("byte_size", ctypes.c_uint64),
                ("shape", ctypes.POINTER(ctypes.c_int64)), ("strides", ctypes.POINTER(ctypes.c_int64)),
                ("rank", ctypes.c_uint32), ("dtype", ctypes.c_uint32),
                ("device_type", ctypes.c_uint32), ("device_ordinal", ctypes.c_int32)]


class TensorArgumentV1(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_uint32), ("dtype", ctypes.c_uint32),
                ("buffer", TensorBufferV1), ("scalar", ctypes.c_uint64)]


class TensorStreamV1(ctypes.Structure):
    _fields_ = [("device_type", ctypes.c_uint32), ("device_ordinal", ctypes.c_int32),
                ("handle", ctypes.c_uint64)]


class TensorCallV1(ctypes.Structure):
    _fields_ = [("abi_version", ctypes.c_uint32), ("struct_size", ctypes.c_uint32),
                ("arguments", ctypes.POINTER(TensorArgumentV1)), ("argument_count", ctypes.c_uint32),
                ("flags", ctypes.c_uint32), ("grid", ctypes.c_uint32 * 3), ("block", ctypes.c_uint32 * 3),
                ("shared_memory_bytes", ctypes.c_uint64), ("stream", TensorStreamV1)]


class TensorErrorV1(ctypes.Structure):
    _fields_ = [("code", ctypes.c_int32), ("message", ctypes.c_char * 508)]


class TB200GemvItem(ctypes.Structure):
    """One projection of ``tb200_gguf_gemv_list`` (include/tensor_b200_gguf.h)."""
    _fields_ = [("format", ctypes.c_int32), ("x_dtype", ctypes.c_int32), ("x", ctypes.c_void_p),
                ("w", ctypes.c_void_p), ("outs", ctypes.c_void_p * 8), ("out_count", ctypes.c_int32),
                ("reserved", ctypes.c_int32), ("out_ld", ctypes.c_int64), ("m", ctypes.c_int64),
                ("n", ctypes.c_int64), ("k", ctypes.c_int64)]


class TB200Schedule(ctypes.Structure):
    """Pinned launch choices (include/tensor_b200_gguf.h); zero fields are derived by the library."""
    _fields_ = [("k_splits", ctypes.c_int32), ("ctas_per_sm", ctypes.c_int32), ("convert_ahead", ctypes.c_int32),
                ("overlap", ctypes.c_int32), ("gemm_shape", ctypes.c_int32), ("reserved", ctypes.c_int32 * 3)]


assert ctypes.sizeof(TensorBufferV1) == 48
assert ctypes.sizeof(TensorArgumentV1) == 64
assert ctypes.sizeof(TensorStreamV1) == 16
assert ctypes.sizeof(TensorCallV1) == 72
assert ctypes.sizeof(TensorErrorV1) == 512
assert ctypes.sizeof(TB200GemvItem) == 128


def buffer_argument(address: int, byte_size: int, dtype: int, ordinal: int, shape=None) -> TensorArgumentV1:
    """A kind-1 argument for device memory at ``address`` (borrowed, never owned)."""
    arg = TensorArgumentV1()
    arg.kind = ARG_BUFFER
    arg.dtype = dtype
    arg.buffer.address = address
    arg.buffer.byte_size = byte_size
    if shape is not None:
        dims = (ctypes.c_int64 * len(shape))(*shape)
        arg._keep = dims  # keep the array alive with the argument
        arg.buffer.shape = dims
        arg.buffer.rank = len(shape)
    arg.buffer.dtype = dtype
    arg.buffer.device_type = DEVICE_CUDA
    arg.buffer.device_ordinal = ordinal
    return arg


def scalar_argument(value: int, dtype: int = DTYPE_IDS["int64"]) -> TensorArgumentV1:
    arg = TensorArgumentV1()
    arg.kind = ARG_SCALAR
    arg.dtype = dtype
    if dtype == DTYPE_IDS["int32"]:
        arg.scalar = ctypes.c_uint32(value & 0xFFFFFFFF).value
    else:
        arg.scalar = ctypes.c_uint64(value & 0xFFFFFFFFFFFFFFFF).value
    return arg


def make_call(arguments, ordinal: int, stream_handle: int):
    """TensorCallV1 over ``arguments``; returns (call, keepalive)."""
    array = (TensorArgumentV1 * len(arguments))(*arguments)
    call = TensorCallV1()
    call.abi_version = ABI_VERSION
    call.struct_size = ctypes.sizeof(TensorCallV1)
    call.arguments = array
    call.argument_count = len(arguments)
    call.stream.device_type = DEVICE_CUDA
    call.stream.device_ordinal = ordinal
    call.stream.handle = stream_handle
    return call, (array, arguments)
