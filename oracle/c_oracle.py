"""ctypes binding of the plain-C oracle (``oracle/gguf_oracle.c``).

TEST INFRASTRUCTURE: used by the tests as a second checker and by the benchmark's
``cpu_baseline`` / ``--impl reference`` legs as the timed multi-threaded CPU port of
the reference arithmetic (``benchmarks/kernels/showcase/triton_kernels.py:133-222``).
"""

from __future__ import annotations

import ctypes
import os
import subprocess

import numpy as np

from .gguf_oracle import get_format, weight_bytes

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "_build", "libgguf_oracle.so")
_lib = None


def build(force: bool = False) -> str:
    """Compile the C oracle with the committed Makefile (gcc, OpenMP)."""
    src = os.path.join(_HERE, "gguf_oracle.c")
    stale = (not os.path.exists(_LIB_PATH)) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src)
    if force or stale:
        subprocess.run(["make", "-C", _HERE, "-B", "_build/libgguf_oracle.so"], check=True,
                       stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        u8p = ctypes.POINTER(ctypes.c_uint8)
        f32p = ctypes.POINTER(ctypes.c_float)
        i64 = ctypes.c_int64
        _lib.gguf_oracle_row_bytes.restype = i64
        _lib.gguf_oracle_row_bytes.argtypes = [ctypes.c_int, i64]
        _lib.gguf_oracle_threads.restype = ctypes.c_int
        _lib.gguf_oracle_set_threads.argtypes = [ctypes.c_int]
        _lib.gguf_oracle_dequant.argtypes = [ctypes.c_int, u8p, i64, i64, f32p]
        _lib.gguf_oracle_gemv.argtypes = [ctypes.c_int, u8p, i64, i64, f32p, i64, f32p]
        _lib.gguf_oracle_gemm.argtypes = [ctypes.c_int, u8p, i64, i64, f32p, i64, ctypes.c_int, f32p]
    return _lib


def _u8(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_uint8))


def _f32(a):
    return a.ctypes.data_as(ctypes.POINTER(ctypes.c_float))


def threads() -> int:
    return int(lib().gguf_oracle_threads())


def use_all_cores() -> int:
    """Run on every core this process may be scheduled on, whatever OMP_NUM_THREADS says (process
    launchers set it to 1 for their children); returns the thread count now in effect."""
    lib().gguf_oracle_set_threads(len(os.sched_getaffinity(0)))
    return threads()


def _raw(raw, fmt, n, k):
    raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
    if raw.size != weight_bytes(fmt, n, k):
        raise ValueError("raw byte count does not match [n, k]")
    return raw


def dequantize(raw, fmt, n: int, k: int) -> np.ndarray:
    f = get_format(fmt)
    raw = _raw(raw, f, n, k)
    out = np.empty((n, k), dtype=np.float32)
    status = lib().gguf_oracle_dequant(f.type_id, _u8(raw), n, k, _f32(out))
    if status:
        raise ValueError(f"gguf_oracle_dequant status {status}")
    return out


def gemv(x, raw, fmt, n: int, k: int) -> np.ndarray:
    f = get_format(fmt)
    raw = _raw(raw, f, n, k)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    out = np.empty((x.shape[0], n), dtype=np.float32)
    status = lib().gguf_oracle_gemv(f.type_id, _u8(raw), n, k, _f32(x), x.shape[0], _f32(out))
    if status:
        raise ValueError(f"gguf_oracle_gemv status {status}")
    return out


def gemm(x, raw, fmt, n: int, k: int, operand: str = "bf16") -> np.ndarray:
    """``x`` must already be rounded to the operand type (values held as fp32)."""
    f = get_format(fmt)
    raw = _raw(raw, f, n, k)
    x = np.ascontiguousarray(x, dtype=np.float32).reshape(-1, k)
    out = np.empty((x.shape[0], n), dtype=np.float32)
    mode = {"f32": 0, "bf16": 1}[operand]
    status = lib().gguf_oracle_gemm(f.type_id, _u8(raw), n, k, _f32(x), x.shape[0], mode, _f32(out))
    if status:
        raise ValueError(f"gguf_oracle_gemm status {status}")
    return out
