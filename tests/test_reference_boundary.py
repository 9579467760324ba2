"""The reference's side of the boundary, exercised against this build without a GPU.

The reference checkout (``src/tensor`` and ``packages/tensor-torch``) imports and runs with NumPy and
PyTorch alone.  These tests hand ITS OWN classes and functions to this build: its ctypes descriptor
classes (src/tensor/runtime/abi.py:50-97) to the ``*_v1`` entry points, its shape binding and launch
resolution (src/tensor/runtime/signature.py:137-216) and its artifact reader to manifests written by
``tensor_b200.tbin``, and ``tensor_torch.load`` (packages/tensor-torch/src/tensor_torch/loading.py:7-34,
registration.py:10-73) to one of our artifacts under fake tensors.  Skipped where the checkout is absent
(set TENSOR_REFERENCE, or keep a directory ``reference`` next to this repository)."""

import ctypes
import os
import sys

import numpy as np
import pytest

import tensor_b200
from tensor_b200 import tbin

REFERENCE = os.environ.get("TENSOR_REFERENCE") or os.path.normpath(
    os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference"))
PATHS = [os.path.join(REFERENCE, "src"), os.path.join(REFERENCE, "packages", "tensor-torch", "src")]

pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "src", "tensor")),
                                reason="reference checkout not available")


@pytest.fixture(scope="module")
def reference_on_path():
    for p in PATHS:
        sys.path.insert(0, p)
    yield
    for p in PATHS:
        sys.path.remove(p)


def _library():
    lib = ctypes.CDLL(tensor_b200.LIB_PATH)
    for name in ("tb200_gguf_dequant_v1", "tb200_gguf_gemv_v1", "tb200_gguf_gemm_v1"):
        fn = getattr(lib, name)
        fn.restype = ctypes.c_int32
        fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    return lib


def _call(rabi, buffers, scalars):
    """A CallDescriptor filled by hand with the reference's classes: kind-1 buffers (device address,
    byte size, dtype, CUDA device 0), then kind-2 int64 scalars, stream 0 of device 0."""
    args = (rabi.Argument * (len(buffers) + len(scalars)))()
    for arg, (address, nbytes, dtype) in zip(args, buffers):
        arg.kind, arg.dtype = 1, rabi.DTYPES[dtype]
        arg.buffer = rabi.BufferDescriptor(address, nbytes, None, None, 0, rabi.DTYPES[dtype], 2, 0)
    for arg, value in zip(args[len(buffers):], scalars):
        arg.kind, arg.dtype = 2, rabi.DTYPES["int64"]
        scalar = ctypes.c_int64(value)
        ctypes.memmove(ctypes.addressof(arg) + rabi.Argument.scalar.offset, ctypes.byref(scalar), 8)
    call = rabi.CallDescriptor(rabi.ABI_MAJOR, ctypes.sizeof(rabi.CallDescriptor), args, len(args), 0,
                               (ctypes.c_uint32 * 3)(1, 1, 1), (ctypes.c_uint32 * 3)(1, 1, 1), 0,
                               rabi.StreamDescriptor(2, 0, 0))
    return call, args


def test_reference_descriptor_classes_drive_the_c_abi(reference_on_path):
    from tensor.runtime import abi as rabi

    assert ctypes.sizeof(rabi.BufferDescriptor) == ctypes.sizeof(tensor_b200.abi.TensorBufferV1) == 48
    assert ctypes.sizeof(rabi.Argument) == 64 and ctypes.sizeof(rabi.CallDescriptor) == 72
    assert ctypes.sizeof(rabi.ErrorDescriptor) == 512
    lib = _library()
    m, n, k, q4_k = 1, 256, 512, 12
    wbytes = n * k // 256 * 144
    base = 1 << 20  # never dereferenced: every call below is rejected before a launch
    good = [(base, m * k * 2, "bfloat16"), (2 * base, wbytes, "uint8"), (3 * base, m * n * 4, "float32")]

    # a weight buffer one block short: an argument error that names the buffer, found before any CUDA call
    short = [good[0], (2 * base, wbytes - 144, "uint8"), good[2]]
    call, keep = _call(rabi, short, (m, n, k, q4_k))
    err = rabi.ErrorDescriptor()
    assert lib.tb200_gguf_gemv_v1(ctypes.byref(call), ctypes.byref(err)) == 2
    assert err.code == 2 and b"w holds" in err.message

    # a descriptor of another ABI major
    call, keep = _call(rabi, good, (m, n, k, q4_k))
    call.abi_version = 2
    assert lib.tb200_gguf_gemv_v1(ctypes.byref(call), ctypes.byref(err)) == 1

    # an unknown format id, and K that is not a whole number of blocks
    call, keep = _call(rabi, good, (m, n, k, 99))
    assert lib.tb200_gguf_gemv_v1(ctypes.byref(call), ctypes.byref(err)) == 2
    call, keep = _call(rabi, good, (m, n, k + 32, q4_k))
    assert lib.tb200_gguf_gemv_v1(ctypes.byref(call), ctypes.byref(err)) == 2

    # the dequantisation and the GEMM take the same descriptors
    call, keep = _call(rabi, [(2 * base, wbytes, "uint8"), (3 * base, n * k * 4 - 4, "float32")], (n, k, q4_k))
    assert lib.tb200_gguf_dequant_v1(ctypes.byref(call), ctypes.byref(err)) == 2
    call, keep = _call(rabi, [(base, 256 * k * 4, "float32"), good[1], (3 * base, 256 * n * 4, "float32")], (256, n, k, q4_k))
    assert lib.tb200_gguf_gemm_v1(ctypes.byref(call), ctypes.byref(err)) == 2  # the GEMM takes bfloat16 activations

    import torch

    if not torch.cuda.is_available():
        # a well-formed call on a machine without a device: a provider error, never a CPU result
        call, keep = _call(rabi, good, (m, n, k, q4_k))
        assert lib.tb200_gguf_gemv_v1(ctypes.byref(call), ctypes.byref(err)) == 3
        assert err.code == 3 and err.message


class _Shaped:
    """What bind_shapes needs of a buffer: a shape and a dtype that prints as the manifest's name."""

    def __init__(self, shape, dtype):
        self.shape, self.dtype = tuple(shape), dtype


def test_reference_binding_accepts_our_manifests(reference_on_path, tmp_path):
    from tensor.artifacts.format import read_artifact
    from tensor.runtime.abi import check_requirement
    from tensor.runtime.signature import bind_shapes, resolve_launch

    cases = [
        (tbin.build_gemv_tbin, ("q4_k", 4, 4096, 4096)),
        (tbin.build_gemv_f32_tbin, ("q6_k", 1, 512, 1024)),
        (tbin.build_gemv_f32_tbin, ("q8_0", 3, 300, 512)),
        (tbin.build_gemm_tbin, ("q6_k", 256, 256, 1024)),
    ]
    for i, (build, args) in enumerate(cases):
        path = str(tmp_path / f"k{i}.tbin")
        build(path, *args)
        manifest, files = read_artifact(path)
        check_requirement(manifest["runtime_abi"])
        assert files["kernel.cubin"].startswith(b"\x7fELF")
        supplied = {a["name"]: _Shaped(a["shape"], a["dtype"]) for a in manifest["arguments"]}
        symbols, values = bind_shapes(manifest, supplied)
        assert symbols == {} and set(values) == set(supplied)
        launch = resolve_launch(manifest["launch"], symbols)
        assert launch["grid"][0] >= 1 and launch["block"][0] % 32 == 0
        wrong = dict(supplied)
        first = manifest["arguments"][0]
        wrong[first["name"]] = _Shaped([d + 1 for d in first["shape"]], first["dtype"])
        with pytest.raises(ValueError):
            bind_shapes(manifest, wrong)
    # the artifact with the reference kernels' own signature: fp32 x, flat buffers, no declared outputs
    manifest, _ = read_artifact(str(tmp_path / "k1.tbin"))
    assert [(a["name"], a["dtype"], len(a["shape"])) for a in manifest["arguments"]] == [
        ("x", "float32", 1), ("w", "uint8", 1), ("out", "float32", 1)]
    assert manifest["outputs"] == [] and manifest["launch"]["shared_memory_bytes"] == 0


def test_tensor_torch_loads_our_artifact_under_fake_tensors(reference_on_path, tmp_path):
    import torch
    from torch._subclasses.fake_tensor import FakeTensorMode

    import tensor_torch

    m, n, k = 256, 384, 1024
    path = str(tmp_path / "gemm.tbin")
    tbin.build_gemm_tbin(path, "q4_k", m, n, k)
    kernel = tensor_torch.load(path)
    assert [d["name"] for d in kernel.inputs] == ["x", "w"] and [d["name"] for d in kernel.outputs] == ["out"]
    with FakeTensorMode():
        x = torch.empty((m, k), dtype=torch.bfloat16, device="cuda")
        w = torch.empty((n * k // 256 * 144,), dtype=torch.uint8, device="cuda")
        out = kernel._op([x, w], [])
        assert len(out) == 1 and tuple(out[0].shape) == (m, n) and out[0].dtype == torch.float32
        assert out[0].device.type == "cuda"
    # the fp32-signature artifact declares no outputs: the functional binding refuses it, as the
    # reference documents (kernel.py:28-30); its caller passes all three buffers to Executable.launch
    f32 = str(tmp_path / "f32.tbin")
    tbin.build_gemv_f32_tbin(f32, "q4_k", 1, 256, 512)
    with pytest.raises(ValueError):
        tensor_torch.load(f32)


def test_reference_module_system_installs_and_resolves_our_module(reference_on_path, tmp_path):
    """``tensor.json`` + prebuilt artifacts: installed, resolved for target sm_100 and loaded by tensor-torch
    through the reference's own package code, with no compiler on the consumer side."""
    import torch
    from torch._subclasses.fake_tensor import FakeTensorMode

    import tensor_torch
    from tensor.modules.archive import pack
    from tensor.modules.errors import ModuleError
    from tensor.modules.project import resolve_reference
    from tensor.modules.resolver import install

    from tensor_b200 import module

    root, cache = str(tmp_path / "gguf-b200"), str(tmp_path / "cache")
    shapes = [{"op": "gemv", "encoding": "q4_k", "m": 1, "n": 1024, "k": 2048},
              {"op": "gemv", "encoding": "q6_k", "m": 1, "n": 256, "k": 512, "x_dtype": "float32"},
              {"op": "gemm", "encoding": "q4_k", "m": 256, "n": 256, "k": 1024}]
    manifest = module.write_module(root, shapes)
    assert set(manifest["exports"]) == {"q4_k_gemv_m1_n1024_k2048", "q6_k_gemv_m1_n256_k512_f32", "q4_k_gemm_m256_n256_k1024"}
    assert install(root, cache_dir=cache)["status"] == "installed"
    for export in manifest["exports"]:
        found = resolve_reference(f"gguf-b200::{export}", project=root, module_cache=cache, target="sm_100")
        assert found["selection"] == "packaged" and found["target"] == "sm_100" and found["path"].endswith(export + ".tbin")
    with pytest.raises(ModuleError):
        resolve_reference("gguf-b200::q4_k_gemm_m256_n256_k1024", project=root, module_cache=cache, target="sm_90")
    kernel = tensor_torch.load("gguf-b200::q4_k_gemm_m256_n256_k1024", project=root, module_cache=cache, target="sm_100")
    with FakeTensorMode():
        x = torch.empty((256, 1024), dtype=torch.bfloat16, device="cuda")
        w = torch.empty((256 * 1024 // 256 * 144,), dtype=torch.uint8, device="cuda")
        (out,) = kernel._op([x, w], [])
        assert tuple(out.shape) == (256, 256) and out.dtype == torch.float32
    archive = str(tmp_path / "gguf-b200.tpack")
    pack(root, archive, cache_dir=cache)
    assert os.path.getsize(archive) > 0
