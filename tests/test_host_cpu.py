"""CPU-only checks of the host layer and of the C-ABI library's loading, exports and argument
validation (no compute: there is no GPU here, and the library has no CPU path)."""

import ctypes
import os
import re

import pytest

import tensor_b200 as tb
from tensor_b200 import abi
from tensor_b200._native import EXPORTS, LIB_PATH, lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    with open(os.path.join(ROOT, "include", "tensor_b200_gguf.h")) as f:
        declared = set(re.findall(r"\b(tb200_\w+)\s*\(", f.read()))
    assert declared, "header declares nothing?"
    assert declared == set(EXPORTS)
    handle = ctypes.CDLL(LIB_PATH)
    for name in declared:
        assert hasattr(handle, name), name


def test_host_constants_match_the_header():
    """The variant ids, peer flags and list length the Python layer passes are the header's."""
    from tensor_b200 import ops

    with open(os.path.join(ROOT, "include", "tensor_b200_gguf.h")) as f:
        defines = dict(re.findall(r"#define\s+(TB200_\w+)\s+(\d+)", f.read()))
    for name in ("auto", "simple", "fast", "mma", "tc", "dp4a"):
        assert ops._VARIANTS[name] == int(defines["TB200_VARIANT_" + name.upper()])
    assert ops.PEER_WAIT == int(defines["TB200_PEER_WAIT"]) and ops.PEER_SIGNAL == int(defines["TB200_PEER_SIGNAL"])
    assert ops.GEMV_LIST_MAX == int(defines["TB200_GEMV_LIST_MAX"])


def test_version_and_sizes():
    l = lib()
    assert l.tb200_gguf_version() >> 16 == 1
    assert l.tb200_gguf_weight_bytes(8, 4096, 4096) == 17825792
    assert l.tb200_gguf_weight_bytes(12, 18944, 3584) == 38191104
    assert l.tb200_gguf_weight_bytes(12, 3584, 18944) == 38191104
    assert l.tb200_gguf_weight_bytes(14, 12288, 4096) == 41287680
    assert l.tb200_gguf_weight_bytes(2, 4, 64) == 4 * 2 * 18
    assert l.tb200_gguf_weight_bytes(12, 4, 100) == -1
    assert l.tb200_gguf_weight_bytes(5, 4, 256) == -1


def _status(fn, *args):
    err = abi.TensorErrorV1()
    code = fn(*args, ctypes.byref(err))
    return code, err.message.decode()


def test_plain_entry_points_reject_bad_arguments_before_any_cuda_call():
    l = lib()
    ok_ptr = ctypes.c_void_p(1 << 20)
    code, msg = _status(l.tb200_gguf_gemv, 99, 13, ok_ptr, ok_ptr, ok_ptr, 1, 16, 256, None, 0, 0, None)
    assert code == abi.ERROR_ARGUMENT and "format" in msg
    code, msg = _status(l.tb200_gguf_gemv, 12, 13, ok_ptr, ok_ptr, ok_ptr, 1, 16, 100, None, 0, 0, None)
    assert code == abi.ERROR_ARGUMENT and "multiple" in msg
    code, msg = _status(l.tb200_gguf_gemv, 12, 6, ok_ptr, ok_ptr, ok_ptr, 1, 16, 256, None, 0, 0, None)
    assert code == abi.ERROR_ARGUMENT and "dtype" in msg
    code, msg = _status(l.tb200_gguf_gemv, 12, 13, ctypes.c_void_p((1 << 20) + 2), ok_ptr, ok_ptr, 1, 16, 256,
                        None, 0, 0, None)
    assert code == abi.ERROR_ARGUMENT and "aligned" in msg
    code, msg = _status(l.tb200_gguf_gemv, 12, 13, None, ok_ptr, ok_ptr, 1, 16, 256, None, 0, 0, None)
    assert code == abi.ERROR_ARGUMENT and "NULL" in msg
    code, msg = _status(l.tb200_gguf_gemm, 12, 10, ok_ptr, ok_ptr, ok_ptr, 256, 16, 256, 0, None)
    assert code == abi.ERROR_ARGUMENT and "bfloat16" in msg
    code, msg = _status(l.tb200_gguf_dequant, 12, ok_ptr, ok_ptr, -1, 256, None)
    assert code == abi.ERROR_ARGUMENT


def test_empty_problem_is_ok_without_a_device():
    l = lib()
    code, _ = _status(l.tb200_gguf_gemv, 12, 13, None, None, None, 0, 16, 256, None, 0, 0, None)
    assert code == abi.OK


def _call(arguments, abi_version=1, ordinal=0):
    call, keep = abi.make_call(arguments, ordinal, 0)
    call.abi_version = abi_version
    return call, keep


def test_descriptor_entry_points_validate_like_the_reference_wrappers():
    l = lib()
    buf = lambda n, dt: abi.buffer_argument(1 << 20, n, dt, 0)
    good = [buf(2 * 256, 13), buf(16 * 144, 3), buf(4 * 16, 11),
            abi.scalar_argument(1), abi.scalar_argument(16), abi.scalar_argument(256), abi.scalar_argument(12)]
    call, keep = _call(good, abi_version=2)
    code, msg = _status(l.tb200_gguf_gemv_v1, ctypes.byref(call))
    assert code == abi.ERROR_ABI and "ABI version" in msg
    call, keep = _call(good)
    call.struct_size = 64
    assert _status(l.tb200_gguf_gemv_v1, ctypes.byref(call))[0] == abi.ERROR_ABI
    # wrong byte size for w
    bad = list(good)
    bad[1] = buf(16 * 144 - 1, 3)
    call, keep = _call(bad)
    code, msg = _status(l.tb200_gguf_gemv_v1, ctypes.byref(call))
    assert code == abi.ERROR_ARGUMENT and "w holds" in msg
    # output dtype
    bad = list(good)
    bad[2] = buf(4 * 16, 10)
    call, keep = _call(bad)
    assert _status(l.tb200_gguf_gemv_v1, ctypes.byref(call))[0] == abi.ERROR_ARGUMENT
    # too few scalars
    call, keep = _call(good[:5])
    assert _status(l.tb200_gguf_gemv_v1, ctypes.byref(call))[0] == abi.ERROR_ARGUMENT
    # buffer on another device than the stream
    bad = list(good)
    bad[0] = abi.buffer_argument(1 << 20, 512, 13, 1)
    call, keep = _call(bad)
    code, msg = _status(l.tb200_gguf_gemv_v1, ctypes.byref(call))
    assert code == abi.ERROR_ARGUMENT and "device" in msg
    # scalar of a float dtype
    bad = list(good)
    bad[3] = abi.scalar_argument(1, 11)
    call, keep = _call(bad)
    assert _status(l.tb200_gguf_gemv_v1, ctypes.byref(call))[0] == abi.ERROR_ARGUMENT
    # NULL call
    assert _status(l.tb200_gguf_gemm_v1, None)[0] == abi.ERROR_ABI


def test_valid_call_without_gpu_fails_loudly():
    import torch

    if torch.cuda.is_available():
        pytest.skip("needs a box without a GPU")
    l = lib()
    ok_ptr = ctypes.c_void_p(1 << 20)
    code, msg = _status(l.tb200_gguf_gemv, 12, 13, ok_ptr, ok_ptr, ok_ptr, 1, 16, 256, None, 0, 0, None)
    assert code == abi.ERROR_PROVIDER and msg


def test_formats_and_kernel_factory_validation():
    assert tb.get_format(12) is tb.Q4_K and tb.get_format("Q6_K") is tb.Q6_K
    assert tb.Q8_0.row_bytes(4096) == 4352 and tb.Q4_0.bits_per_weight == 4.5
    with pytest.raises(ValueError):
        tb.get_format(13)
    with pytest.raises(ValueError):
        tb.Q4_K.row_bytes(300)
    with pytest.raises(ValueError):
        tb.gguf(1, 16, 256, 12, threads=128, device="cuda:0")  # a reference schedule key
    with pytest.raises(ValueError):
        tb.gguf(0, 16, 256, 12, device="cuda:0")
    with pytest.raises(ValueError):
        tb.gguf(256, 16, 256, 12, x_dtype="float16", device="cuda:0")  # GEMM wants bf16
    k = tb.gguf(1, 4096, 4096, 8, x_dtype="float16", device="cuda:0")
    assert k.op == "gemv" and k.weight_bytes == 17825792 and k.outputs == ["out"]
    assert [a["name"] for a in k.arguments] == ["x", "w", "out"]
    assert tb.gguf(256, 12288, 4096, 14, device="cuda:0").op == "gemm"


def test_ops_refuse_cpu_tensors():
    import torch

    x = torch.zeros(1, 256, dtype=torch.bfloat16)
    w = torch.zeros(16 * 144, dtype=torch.uint8)
    with pytest.raises(ValueError, match="CUDA"):
        tb.gemv(x, w, 12, 16, 256)
    with pytest.raises(ValueError, match="CUDA"):
        tb.dequantize(w, 12, 16, 256)
    k = tb.gguf(1, 16, 256, 12, device="cuda:0")
    with pytest.raises(ValueError):
        k.launch(x, w, torch.zeros(1, 16))
    with pytest.raises(TypeError):
        k.launch(x, w, None)
    with pytest.raises(ValueError):
        k._check((x, w))


# ---- N-sharded entry points: argument checks run before any device is touched -------------------

def _sharded(out_count=1, out_ld=64, col_offset=0, n=32, outs=None, fmt=12, k=256):
    import ctypes

    from tensor_b200 import abi
    from tensor_b200._native import lib

    table = (ctypes.c_void_p * 8)(*(outs if outs is not None else [0x1000] * 8))
    err = abi.TensorErrorV1()
    status = lib().tb200_gguf_gemv_sharded(fmt, 13, 0x1000, 0x1000, table, out_count, out_ld, col_offset, 1, n, k,
                                           None, 0, 0, None, ctypes.byref(err))
    return status, err.message.decode()


def test_sharded_gemv_rejects_bad_destinations():
    assert _sharded(out_count=0)[0] == 2
    assert _sharded(out_count=9)[0] == 2
    status, message = _sharded(out_ld=40, col_offset=16, n=32)
    assert status == 2 and "do not fit" in message
    assert _sharded(col_offset=-4)[0] == 2
    assert _sharded(outs=[0x1000, 0] + [0x1000] * 6, out_count=2)[0] == 2
    assert _sharded(fmt=99)[0] == 2
    # well-formed arguments get as far as the device check (no GPU here: provider error, never a CPU result)
    assert _sharded()[0] == 3


def test_peer_barrier_rejects_bad_ranks():
    import ctypes

    from tensor_b200 import abi
    from tensor_b200._native import lib

    table = (ctypes.c_void_p * 8)(*([0x1000] * 8))
    err = abi.TensorErrorV1()
    assert lib().tb200_peer_barrier(table, 2, 2, None, ctypes.byref(err)) == 2
    assert lib().tb200_peer_barrier(table, 0, 9, None, ctypes.byref(err)) == 2
    assert lib().tb200_peer_barrier(None, 0, 2, None, ctypes.byref(err)) == 2
    assert lib().tb200_peer_barrier(table, 0, 2, None, ctypes.byref(err)) == 3


def test_bump_allocator_gives_every_rank_the_same_offsets():
    from tensor_b200.peer import BumpAllocator

    a, b = BumpAllocator(4096), BumpAllocator(4096)
    sizes = [256, 100, 4, 1000]
    assert [a.take(s) for s in sizes] == [b.take(s) for s in sizes] == [0, 256, 512, 768]
    with pytest.raises(MemoryError):
        a.take(4096)


def test_gemv_pair_validates_before_touching_a_device():
    import ctypes

    from tensor_b200 import abi
    from tensor_b200._native import lib

    err = abi.TensorErrorV1()

    def call(fmt=12, n1=32, n2=32, k=256, variant=0):
        return lib().tb200_gguf_gemv_pair(fmt, 13, 0x1000, 0x1000, n1, 0x2000, n2, 0x3000, 1, k, None, 0, variant,
                                          None, ctypes.byref(err))

    assert call(fmt=7) == 2
    assert call(k=100) == 2
    assert call(n2=-1) == 2
    assert call(variant=6) == 2
    assert call() == 3  # well-formed: stops at the missing device, never computes on the CPU
