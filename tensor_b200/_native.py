"""Loader of the in-tree CUDA library.  There is no fallback: if ``libtensor_b200_gguf.so`` is
missing or does not load, every operation of this package raises."""

from __future__ import annotations

import ctypes
import os

from . import abi

LIB_PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "lib", "libtensor_b200_gguf.so")

#: every symbol include/tensor_b200_gguf.h declares
EXPORTS = (
    "tb200_gguf_version", "tb200_gguf_weight_bytes", "tb200_gguf_gemv_scratch_bytes",
    "tb200_gguf_device_status", "tb200_gguf_gemv_plan", "tb200_gguf_gemv_launch_config",
    "tb200_gguf_gemm_launch_config", "tb200_gguf_dequant", "tb200_gguf_gemv", "tb200_gguf_gemm",
    "tb200_gguf_dequant_v1", "tb200_gguf_gemv_v1", "tb200_gguf_gemm_v1",
    "tb200_gguf_gemv_static", "tb200_gguf_gemv_sharded", "tb200_gguf_gemv_sharded_sync", "tb200_peer_barrier",
    "tb200_peer_sync", "tb200_gguf_gemv_pair", "tb200_gguf_gemv_pair_sharded_sync",
    "tb200_peer_export", "tb200_peer_open", "tb200_peer_close",
    "tb200_gguf_gemv_list", "tb200_gguf_gemv_list_scratch_bytes", "tb200_peer_set_wait_limit",
    "tb200_gguf_schedule_legal", "tb200_gguf_schedule_record", "tb200_gguf_schedule_clear",
    "tb200_gguf_gemv_scheduled", "tb200_gguf_gemm_scheduled",
    "tb200_rmsnorm_bf16", "tb200_swiglu_bf16", "tb200_residual_add",
)


class TensorRuntimeError(RuntimeError):
    """Provider-side failure (status 3), like the reference's ``TensorRuntimeError``
    (src/tensor/providers/cuda/driver.py:11-16)."""

    def __init__(self, message: str, code: int = abi.ERROR_PROVIDER):
        super().__init__(message)
        self.code = code


class AbiError(TensorRuntimeError):
    """The call descriptor itself was malformed (status 1)."""


_lib = None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise TensorRuntimeError(
            f"{LIB_PATH} is missing: build the CUDA extension first (python -m tensor_b200.build). "
            "This package has no CPU or PyTorch fallback.")
    handle = ctypes.CDLL(LIB_PATH)
    missing = [name for name in EXPORTS if not hasattr(handle, name)]
    if missing:
        raise TensorRuntimeError(f"{LIB_PATH} does not export {missing}; rebuild it")
    i32, i64, vp = ctypes.c_int32, ctypes.c_int64, ctypes.c_void_p
    err = ctypes.POINTER(abi.TensorErrorV1)
    call = ctypes.POINTER(abi.TensorCallV1)
    handle.tb200_gguf_version.restype = i32
    handle.tb200_gguf_weight_bytes.restype = i64
    handle.tb200_gguf_weight_bytes.argtypes = [i32, i64, i64]
    handle.tb200_gguf_gemv_scratch_bytes.restype = i64
    handle.tb200_gguf_gemv_scratch_bytes.argtypes = [i32, i64, i64, i64]
    handle.tb200_gguf_gemv_plan.restype = i32
    handle.tb200_gguf_gemv_plan.argtypes = [i32, i64, i64, i64, i64, ctypes.POINTER(ctypes.c_int32)]
    handle.tb200_gguf_gemv_launch_config.restype = i32
    handle.tb200_gguf_gemv_launch_config.argtypes = [i32, i32, i64, i64, i64, i64, ctypes.POINTER(ctypes.c_int32)]
    handle.tb200_gguf_gemm_launch_config.restype = i32
    handle.tb200_gguf_gemm_launch_config.argtypes = [i32, i64, i64, i64, ctypes.POINTER(ctypes.c_int32)]
    handle.tb200_gguf_device_status.restype = i32
    handle.tb200_gguf_device_status.argtypes = [ctypes.POINTER(ctypes.c_uint32), err]
    handle.tb200_gguf_dequant.restype = i32
    handle.tb200_gguf_dequant.argtypes = [i32, vp, vp, i64, i64, vp, err]
    handle.tb200_gguf_gemv.restype = i32
    handle.tb200_gguf_gemv.argtypes = [i32, i32, vp, vp, vp, i64, i64, i64, vp, i64, i32, vp, err]
    handle.tb200_gguf_gemv_static.restype = i32
    handle.tb200_gguf_gemv_static.argtypes = [i32, i32, vp, vp, vp, i64, i64, i64, vp, err]
    handle.tb200_gguf_gemv_sharded.restype = i32
    handle.tb200_gguf_gemv_sharded.argtypes = [i32, i32, vp, vp, ctypes.POINTER(vp), i32, i64, i64, i64, i64, i64,
                                               vp, i64, i32, vp, err]
    handle.tb200_gguf_gemv_sharded_sync.restype = i32
    handle.tb200_gguf_gemv_sharded_sync.argtypes = [i32, i32, vp, vp, ctypes.POINTER(vp), i32, i64, i64, i64, i64, i64,
                                                    vp, i64, i32, ctypes.POINTER(vp), i32, i32, i32, vp, err]
    handle.tb200_gguf_gemv_pair.restype = i32
    handle.tb200_gguf_gemv_pair.argtypes = [i32, i32, vp, vp, i64, vp, i64, vp, i64, i64, vp, i64, i32, vp, err]
    handle.tb200_gguf_gemv_pair_sharded_sync.restype = i32
    handle.tb200_gguf_gemv_pair_sharded_sync.argtypes = [
        i32, i32, vp, vp, i64, vp, i64, ctypes.POINTER(vp), ctypes.POINTER(vp), i32, i64, i64, i64, i64, i64, vp, i64,
        i32, ctypes.POINTER(vp), i32, i32, i32, vp, err]
    handle.tb200_peer_sync.restype = i32
    handle.tb200_peer_sync.argtypes = [ctypes.POINTER(vp), i32, i32, i32, vp, err]
    handle.tb200_peer_barrier.restype = i32
    handle.tb200_peer_barrier.argtypes = [ctypes.POINTER(vp), i32, i32, vp, err]
    handle.tb200_peer_export.restype = i32
    handle.tb200_peer_export.argtypes = [vp, ctypes.c_char_p, ctypes.POINTER(i64), err]
    handle.tb200_peer_open.restype = i32
    handle.tb200_peer_open.argtypes = [ctypes.c_char_p, ctypes.POINTER(vp), err]
    handle.tb200_peer_close.restype = i32
    handle.tb200_peer_close.argtypes = [vp, err]
    handle.tb200_gguf_gemv_list_scratch_bytes.restype = i64
    handle.tb200_gguf_gemv_list_scratch_bytes.argtypes = [ctypes.POINTER(abi.TB200GemvItem), i32]
    handle.tb200_gguf_gemv_list.restype = i32
    handle.tb200_gguf_gemv_list.argtypes = [ctypes.POINTER(abi.TB200GemvItem), i32, vp, i64, i32, ctypes.POINTER(vp),
                                            i32, i32, i32, vp, err]
    sched = ctypes.POINTER(abi.TB200Schedule)
    handle.tb200_gguf_schedule_legal.restype = i32
    handle.tb200_gguf_schedule_legal.argtypes = [i32, i32, i64, i64, i64, i64, sched]
    handle.tb200_gguf_schedule_record.restype = i32
    handle.tb200_gguf_schedule_record.argtypes = [i32, i32, i64, i64, i64, sched]
    handle.tb200_gguf_schedule_clear.restype = None
    handle.tb200_gguf_gemv_scheduled.restype = i32
    handle.tb200_gguf_gemv_scheduled.argtypes = [i32, i32, vp, vp, vp, i64, i64, i64, vp, i64, sched, vp, err]
    handle.tb200_gguf_gemm_scheduled.restype = i32
    handle.tb200_gguf_gemm_scheduled.argtypes = [i32, i32, vp, vp, vp, i64, i64, i64, sched, vp, err]
    handle.tb200_rmsnorm_bf16.restype = i32
    handle.tb200_rmsnorm_bf16.argtypes = [vp, vp, vp, i64, i64, ctypes.c_float, vp, err]
    handle.tb200_swiglu_bf16.restype = i32
    handle.tb200_swiglu_bf16.argtypes = [vp, vp, i64, i64, vp, err]
    handle.tb200_residual_add.restype = i32
    handle.tb200_residual_add.argtypes = [vp, vp, i64, vp, err]
    handle.tb200_peer_set_wait_limit.restype = i32
    handle.tb200_peer_set_wait_limit.argtypes = [ctypes.c_uint64]
    handle.tb200_gguf_gemm.restype = i32
    handle.tb200_gguf_gemm.argtypes = [i32, i32, vp, vp, vp, i64, i64, i64, i32, vp, err]
    for name in ("tb200_gguf_dequant_v1", "tb200_gguf_gemv_v1", "tb200_gguf_gemm_v1"):
        fn = getattr(handle, name)
        fn.restype = i32
        fn.argtypes = [call, err]
    _lib = handle
    _apply_shipped_schedules()
    return _lib


def _apply_shipped_schedules() -> None:
    """Schedules found by a measured search on a B200 (``tensor_b200.schedule.search``) for shapes where
    the derived plan is not the fastest; recorded so that the ordinary entry points use them."""
    import json

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "schedules_b200.json")
    if not os.path.exists(path):
        return
    from . import schedule

    with open(path) as f:
        entries = json.load(f).get("entries", [])
    for e in entries:
        schedule.record(e["op"], e["format"], e["m"], e["n"], e["k"], e["best"])


def raise_for_status(status: int, error: abi.TensorErrorV1) -> None:
    """Map the C status codes onto the exception types the reference raises for the same
    conditions: binding problems are ValueError (src/tensor/runtime/executable.py:93-148),
    provider failures a RuntimeError subclass carrying ``.code``."""
    if status == abi.OK:
        return
    message = error.message.decode("utf-8", "replace")
    if status == abi.ERROR_ARGUMENT:
        raise ValueError(message)
    if status == abi.ERROR_ABI:
        raise AbiError(message, status)
    raise TensorRuntimeError(message, status)
