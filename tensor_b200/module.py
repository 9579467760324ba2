"""Package the sm_100a artifacts as a module of the reference's package system.

A module is a directory with a ``tensor.json`` manifest whose exports name ``.tbin`` artifacts
(docs/modules.md in the reference; src/tensor/modules/module.py:27-120 resolves an export to the
artifact of the requested provider and target).  With the artifacts built ahead of time the consumer
side is compiler-free: ``tensor install``, then ``tensor_torch.load("gguf-b200::<export>")`` or
``Project(...).module(...).resolve(export, target="sm_100")``.  One export per static shape: the
artifacts bake their launch plan in (see ``tensor_b200.tbin``).
"""

from __future__ import annotations

import json
import os

from . import tbin
from .formats import get_format

CAPABILITIES = ["contiguous", "executable_descriptors", "no_external_workspace", "bfloat16_storage", "cuda_tensor_maps"]


def export_name(op: str, encoding, m: int, n: int, k: int, x_dtype: str = "bfloat16") -> str:
    """ASCII identifier of a shape, e.g. ``q4_k_gemv_m1_n18944_k3584`` (``_f32`` for fp32 activations)."""
    suffix = "_f32" if x_dtype == "float32" else ("_f16" if x_dtype == "float16" else "")
    return f"{get_format(encoding).name}_{op}_m{m}_n{n}_k{k}{suffix}"


def write_module(directory: str, shapes, name: str = "gguf-b200", version: str = "0.1.0") -> dict:
    """Build one artifact per entry of ``shapes`` -- dicts with ``op`` (``"gemv"`` / ``"gemm"``),
    ``encoding``, ``m``, ``n``, ``k`` and optionally ``x_dtype`` -- under ``directory/artifacts`` and write
    ``directory/tensor.json``.  Returns the manifest."""
    os.makedirs(os.path.join(directory, "artifacts"), exist_ok=True)
    exports = {}
    for shape in shapes:
        op, enc, m, n, k = shape["op"], shape["encoding"], int(shape["m"]), int(shape["n"]), int(shape["k"])
        x_dtype = shape.get("x_dtype", "bfloat16")
        export = export_name(op, enc, m, n, k, x_dtype)
        relative = f"artifacts/{export}.tbin"
        path = os.path.join(directory, relative)
        if op == "gemm":
            tbin.build_gemm_tbin(path, enc, m, n, k)
        elif x_dtype == "float32":
            tbin.build_gemv_f32_tbin(path, enc, m, n, k)
        elif op == "gemv":
            tbin.build_gemv_tbin(path, enc, m, n, k, x_dtype=x_dtype)
        else:
            raise ValueError(f"unknown op {op!r}")
        exports[export] = {"artifacts": [relative]}
    manifest = {"formatVersion": 1, "name": name, "version": version, "tensorAbi": 1, "exports": exports,
                "capabilities": CAPABILITIES}
    with open(os.path.join(directory, "tensor.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
    return manifest


__all__ = ["CAPABILITIES", "export_name", "write_module"]
