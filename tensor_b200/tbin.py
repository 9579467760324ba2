"""Package the hand-written sm_100a kernels as ``.tbin`` artifacts for the unchanged reference runtime.

A ``.tbin`` is the reference's executable bundle: a zip holding ``manifest.json``,
``kernel.cubin`` and ``kernel.tirx.json``, every member pinned by SHA-256
(``src/tensor/artifacts/format.py:35-357``).  The reference's CUDA provider loads it with
``cuModuleLoadData`` and launches ``entrypoint`` with ``cuLaunchKernel(grid, block, shared, stream,
params)`` where ``params`` are the device addresses of the manifest's buffers in ``abi`` order, or a
128-byte ``CUtensorMap`` for buffers listed in ``cuda_tensor_maps``
(``src/tensor/runtime/abi.py:196-274``, ``src/tensor/providers/cuda/device.py:211-229``).

Because the provider passes nothing but those parameters, every artifact is compiled for ONE static
shape: the launch plan the library would derive at run time is baked into the cubin as constants
(this is what the reference's compiler does per shape as well).  The manifest target is ``sm_100``
-- the reference's target pattern rejects ``sm_100a`` (``src/tensor/runtime/cuda_target.py:9``) --
while the cubin inside is built with ``-arch=sm_100a``; the driver enforces the feature match.

Kernel signature kept from the reference's kernels for this path: ``kernel_kernel(x, w, out)``
(+ an explicit ``scratch`` buffer when the plan splits K: the ABI allows no hidden workspace).
"""

from __future__ import annotations

import ctypes
import hashlib
import json
import os
import subprocess
import tempfile
import zipfile

from .formats import get_format

CSRC = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc")
ENTRYPOINT = "kernel_kernel"
ALIGNMENT = 64
_EMPTY_IR = json.dumps({"nodes": [], "note": "hand-written CUDA; no TIRx graph"}, sort_keys=True).encode()
# CUtensorMapDataType ids (src/tensor/runtime/tensor_map.py:4-17)
_TMA_U64, _TMA_BF16 = 4, 9


def _sha256(data: bytes) -> str:
    return hashlib.sha256(data).hexdigest()


def nvcc_version() -> str:
    from .build import _nvcc

    out = subprocess.run([_nvcc(), "--version"], capture_output=True, text=True).stdout
    for token in out.replace(",", " ").split():
        if token.startswith("V") and token[1:2].isdigit():
            return token[1:]
    return "unknown"


def make_manifest(*, grid, block, shared_memory_bytes, arguments, outputs, source: bytes,
                  tensor_maps=None, options=()):
    """Manifest v3 for a static-shape CUDA kernel (format.py:35-297)."""
    uses_bf16 = any(a["dtype"] == "bfloat16" for a in arguments)
    capabilities = ["contiguous", "executable_descriptors", "no_external_workspace"]
    if uses_bf16:
        capabilities.append("bfloat16_storage")
    if tensor_maps:
        capabilities.append("cuda_tensor_maps")
    manifest = {
        "format": "tensor.module", "format_version": 3, "kind": "cubin", "provider": "cuda",
        "target": "sm_100",
        "entrypoint": ENTRYPOINT,
        "launch": {"grid": list(grid), "block": list(block), "shared_memory_bytes": int(shared_memory_bytes)},
        "compiler": {"name": "nvcc", "version": nvcc_version(), "options": ["-arch=sm_100a", *options]},
        "runtime_abi": {"major": 1, "minor": 3 if uses_bf16 else 1, "required_capabilities": capabilities},
        "workspace": {"bytes": 0, "alignment": 1},
        "arguments": arguments,
        "abi": [{"kind": a["kind"], "name": a["name"], "dtype": a["dtype"]} for a in arguments],
        "outputs": list(outputs), "symbols": {},
        "source_sha256": _sha256(source),
        "tilelang_version": "none (hand-written CUDA)", "tvm_ffi_version": "none",
        "op_set": [],
    }
    if tensor_maps:
        manifest["cuda_tensor_maps"] = tensor_maps
    return manifest


def write_tbin(path: str, manifest: dict, cubin: bytes) -> str:
    if not cubin.startswith(b"\x7fELF"):
        raise ValueError("kernel image is not an ELF cubin")
    manifest = dict(manifest)
    manifest["files"] = {"kernel.cubin": _sha256(cubin), "kernel.tirx.json": _sha256(_EMPTY_IR)}
    with zipfile.ZipFile(path, "w", compression=zipfile.ZIP_DEFLATED) as z:
        for name, data in (("manifest.json", json.dumps(manifest, indent=1, sort_keys=True).encode()),
                           ("kernel.cubin", cubin), ("kernel.tirx.json", _EMPTY_IR)):
            info = zipfile.ZipInfo(name, date_time=(2026, 1, 1, 0, 0, 0))
            info.compress_type = zipfile.ZIP_DEFLATED
            z.writestr(info, data)
    return path


def compile_cubin(source: str) -> bytes:
    """nvcc -cubin of a translation unit that includes the library's kernel sources."""
    from .build import ARCH_FLAGS, _host_compiler, _nvcc

    with tempfile.TemporaryDirectory() as tmp:
        src = os.path.join(tmp, "kernel.cu")
        out = os.path.join(tmp, "kernel.cubin")
        with open(src, "w") as f:
            f.write(source)
        cmd = [_nvcc(), "-arch=sm_100a", "-cubin", "-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
               *_host_compiler(), "-I", CSRC, "-I", os.path.join(os.path.dirname(CSRC), "..", "include"),
               src, "-o", out]
        del ARCH_FLAGS
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode:
            raise RuntimeError(f"nvcc failed:\n{proc.stdout}\n{proc.stderr}")
        with open(out, "rb") as f:
            return f.read()


def _buffer(name, dtype, shape):
    return {"kind": "buffer", "name": name, "dtype": dtype, "shape": [int(s) for s in shape], "alignment": ALIGNMENT}


def _launch_config(encoding, m, n, k, scratch_bytes):
    """All launch constants of the pipelined GEMV at a shape (planned for a B200 when no GPU is present)."""
    from ._native import lib

    out = (ctypes.c_int32 * 32)()
    status = lib().tb200_gguf_gemv_launch_config(get_format(encoding).type_id, 13, m, n, k, scratch_bytes, out)
    if status:
        raise ValueError(f"the pipelined GEMV does not cover {encoding!r} m={m} n={n} k={k}")
    names = ("grid", "threads", "smem_bytes", "k_splits", "row_groups", "row_tiles", "sb_per_split", "nsb",
             "stages", "stride_s", "xs_stride", "off_stage", "off_xs", "off_sx", "off_red", "off_scl",
             "off_zero", "off_misc", "contiguous", "use_tma", "consumer_warps", "scratch_bytes", "ctas_per_sm",
             "counter_bytes", "red_bufs")
    return dict(zip(names, (int(v) for v in out)))


def build_gemv_tbin(path: str, encoding, m: int, n: int, k: int, x_dtype: str = "bfloat16",
                    allow_scratch: bool = True) -> dict:
    """Decode GEMV ``out[m, n] = x[m, k] . dequant(w)^T`` as a static-shape artifact.

    Arguments ``x, w, out`` (+ ``scratch``, uint8, zero-initialised by the caller once, when the plan
    splits K).  Returns the manifest.
    """
    fmt = get_format(encoding)
    if x_dtype not in ("bfloat16", "float16"):
        raise ValueError("the pipelined GEMV takes bfloat16 or float16 activations")
    cfg = _launch_config(fmt, m, n, k, (1 << 40) if allow_scratch else 0)
    split = cfg["k_splits"] > 1
    f16 = "true" if x_dtype == "float16" else "false"
    nt = 1 if m <= 8 else 2
    groups = "true" if m == 1 else "false"
    wparam = "const __grid_constant__ CUtensorMap w" if cfg["use_tma"] else "const uint8_t* w"
    fields = ", ".join(f"{cfg[key]}" for key in (
        "nsb", "sb_per_split", "k_splits", "row_groups", "row_tiles", "stages", "stride_s", "xs_stride",
        "off_stage", "off_xs", "off_sx", "off_red", "off_scl", "off_zero", "off_misc", "contiguous", "use_tma",
        "consumer_warps", "red_bufs"))
    source = f"""// generated by tensor_b200.tbin: Q-format {fmt.name}, m={m}, n={n}, k={k}, x={x_dtype}
#define TB200_TBIN_WRAPPER
#include "gemv_mma.cu"
extern "C" __global__ void __launch_bounds__({cfg['threads']}, {cfg['ctas_per_sm']})
kernel_kernel(const void* x, {wparam}, float* out{', unsigned char* scratch' if split else ''}) {{
  const tb200::GemvStatic s = {{{fields}}};
  tb200::gemv_static_entry<{fmt.type_id}, {f16}, {nt}, {groups}>(
      s, x, {'nullptr, &w' if cfg['use_tma'] else 'w, nullptr'}, out, {'scratch' if split else 'nullptr'},
      {m}, {n}LL, {k}, {cfg['counter_bytes']});
}}
"""
    cubin = compile_cubin(source)
    arguments = [_buffer("x", x_dtype, (m, k)), _buffer("w", "uint8", (fmt.weight_bytes(n, k),)),
                 _buffer("out", "float32", (m, n))]
    if split:
        arguments.append(_buffer("scratch", "uint8", (cfg["scratch_bytes"],)))
    maps = None
    if cfg["use_tma"]:
        rb = fmt.row_bytes(k)
        maps = {"w": {"data_type": _TMA_U64, "global_dims": [rb // 8, n], "global_strides": [rb],
                      "box_dims": [cfg["sb_per_split"] * fmt.nbytes // 8, 16], "element_strides": [1, 1],
                      "interleave": 0, "swizzle": 0, "l2_promotion": 2, "oob_fill": 0}}
    manifest = make_manifest(grid=(cfg["grid"], 1, 1), block=(cfg["threads"], 1, 1),
                             shared_memory_bytes=cfg["smem_bytes"], arguments=arguments, outputs=["out"],
                             source=source.encode(), tensor_maps=maps)
    write_tbin(path, manifest, cubin)
    return manifest


def build_gemv_f32_tbin(path: str, encoding, m: int, n: int, k: int) -> dict:
    """The GEMV with the reference kernels' exact signature and manifest shape for this path:
    ``kernel_kernel(const float* x, const uint8_t* w, float* out)`` over flat 64-byte aligned buffers
    ``x: float32 [m*k]``, ``w: uint8 [bytes]``, ``out: float32 [m*n]`` and NO declared outputs (the caller
    passes all three, as benchmarks/kernels/showcase/benchmark.py:293-295 does).  Any of the four
    formats, any batch; fp32 weights x fp32 activations, one warp per weight row."""
    fmt = get_format(encoding)
    if m < 1 or n < 1:
        raise ValueError("m and n must be positive")
    fmt.row_bytes(k)
    nb = 1 if m == 1 else (4 if m <= 4 else 8)
    warps = 8
    grid = ((n + warps - 1) // warps, (m + nb - 1) // nb, 1)
    source = f"""// generated by tensor_b200.tbin: {fmt.name} GEMV with fp32 activations, m={m}, n={n}, k={k}
#define TB200_TBIN_WRAPPER
#include "gemv_simple.cu"
extern "C" __global__ void __launch_bounds__({warps * 32})
kernel_kernel(const float* x, const uint8_t* w, float* out) {{
  tb200::gemv_simple_static_entry<{fmt.type_id}, float, {nb}>(x, w, out, {m}, {n}LL, {k});
}}
"""
    cubin = compile_cubin(source)
    arguments = [_buffer("x", "float32", (m * k,)), _buffer("w", "uint8", (fmt.weight_bytes(n, k),)),
                 _buffer("out", "float32", (m * n,))]
    manifest = make_manifest(grid=grid, block=(warps * 32, 1, 1), shared_memory_bytes=0, arguments=arguments,
                             outputs=[], source=source.encode())
    write_tbin(path, manifest, cubin)
    return manifest


def build_gemm_tbin(path: str, encoding, m: int, n: int, k: int) -> dict:
    """Prefill GEMM (tcgen05, bf16 operands) as a static-shape artifact: arguments ``x, w, out``;
    ``x`` is consumed through a TMA descriptor the runtime encodes from ``cuda_tensor_maps``."""
    from ._native import lib

    fmt = get_format(encoding)
    cfg = (ctypes.c_int32 * 8)()
    if lib().tb200_gguf_gemm_launch_config(fmt.type_id, m, n, k, cfg):
        raise ValueError(f"the tcgen05 GEMM does not cover {fmt.name} m={m} n={n} k={k}")
    grid_x, grid_y, threads, smem, tile_tok, block_k = (int(v) for v in cfg[:6])
    source = f"""// generated by tensor_b200.tbin: {fmt.name} GEMM, m={m}, n={n}, k={k}
#define TB200_TBIN_WRAPPER
#include "gemm_tcgen05.cu"
extern "C" __global__ void __launch_bounds__(tb200::kGemmThreads, 2)
kernel_kernel(const __grid_constant__ CUtensorMap x, const uint8_t* w, float* out) {{
  tb200::gemm_static_entry<{fmt.type_id}>(x, w, out, {m}, {n}, {k});
}}
"""
    cubin = compile_cubin(source)
    arguments = [_buffer("x", "bfloat16", (m, k)), _buffer("w", "uint8", (fmt.weight_bytes(n, k),)),
                 _buffer("out", "float32", (m, n))]
    maps = {"x": {"data_type": _TMA_BF16, "global_dims": [k, m], "global_strides": [2 * k],
                  "box_dims": [block_k, tile_tok], "element_strides": [1, 1],
                  "interleave": 0, "swizzle": 3, "l2_promotion": 2, "oob_fill": 0}}
    manifest = make_manifest(grid=(grid_x, grid_y, 1), block=(threads, 1, 1), shared_memory_bytes=smem,
                             arguments=arguments, outputs=["out"], source=source.encode(), tensor_maps=maps)
    write_tbin(path, manifest, cubin)
    return manifest
