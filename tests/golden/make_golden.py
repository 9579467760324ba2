"""Generate the golden vectors that pin the CPU oracle to the reference.

Run once in a container that has the reference checkout (set ``TENSOR_REFERENCE`` to its
root) -- the GPU box does not have it, so the outputs are committed next to this script:

    TENSOR_REFERENCE=/path/to/tensor python tests/golden/make_golden.py

What it records, for seeded random blocks of each format the reference states
(GGML type ids 2 / 12 / 14 = Q4_0 / Q4_K / Q6_K):

* ``decode``: the fp32 values produced by the reference's own ``decode_ggml``
  (``benchmarks/kernels/showcase/triton_kernels.py:133-181``), executed with Triton's CPU
  interpreter through a four-line dump kernel defined below;
* ``gemv``: the output of the reference's ``gguf_gemv`` kernel (``triton_kernels.py:213-222``);
* ``gemm``: the output of the reference's fused ``gguf`` kernel (``triton_kernels.py:184-210``,
  fp16 operands, fp32 accumulate).

For all four formats (including Q8_0, which the reference never states) it also records
``gguf.quants.dequantize`` from the third-party ``gguf`` package as a second opinion.
"""

from __future__ import annotations

import os
import sys

os.environ["TRITON_INTERPRET"] = "1"

import numpy as np
import torch
import triton as tr
import triton.language as tl

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
# the reference checkout: TENSOR_REFERENCE, else a sibling directory `reference` next to this repository
sys.path.insert(0, os.environ.get("TENSOR_REFERENCE") or os.path.normpath(os.path.join(ROOT, "..", "reference")))

from benchmarks.kernels.showcase import triton_kernels as ref  # noqa: E402  (the reference)
from oracle import gguf_oracle as oracle  # noqa: E402

decode_ggml = ref.decode_ggml


@tr.jit
def dump_decode(W, O, N: tl.constexpr, K: tl.constexpr, Q: tl.constexpr, BK: tl.constexpr):
    rows = tl.program_id(0) + tl.zeros((1, 1), tl.int32)
    ks = tl.program_id(1) * BK + tl.arange(0, BK)[None, :]
    tl.store(O + rows * K + ks, decode_ggml(W, rows, ks, N, K, Q))


def main():
    from gguf import GGMLQuantizationType as T
    from gguf.quants import dequantize as third_party

    third = {"q4_0": T.Q4_0, "q8_0": T.Q8_0, "q4_k": T.Q4_K, "q6_k": T.Q6_K}
    out = {}
    n, k, m = 12, 512, 16
    for seed, name in enumerate(("q4_0", "q8_0", "q4_k", "q6_k")):
        fmt = oracle.get_format(name)
        raw = oracle.make_weights(fmt, n, k, seed=1000 + seed)
        # widen the scale distribution so decoded values exercise more of the fp32 range
        x1 = oracle.make_activations(1, k, seed=2000 + seed, dtype="f32")
        xm = oracle.make_activations(m, k, seed=3000 + seed, dtype="f32") * 0.2
        out[f"{name}_raw"] = raw
        out[f"{name}_x1"] = x1
        out[f"{name}_xm"] = xm
        out[f"{name}_gguf_py"] = third_party(raw.reshape(n, -1), third[name]).astype(np.float32)
        if name == "q8_0":
            continue  # not stated anywhere in the reference
        w = torch.from_numpy(raw.copy())
        dec = torch.empty((n, k), dtype=torch.float32)
        dump_decode[(n, k // 64)](w, dec, n, k, fmt.type_id, 64)
        out[f"{name}_decode"] = dec.numpy().copy()
        y = torch.full((n,), float("nan"), dtype=torch.float32)
        ref.gguf_gemv[(n // 4,)](torch.from_numpy(x1.reshape(-1).copy()), w, y, n, k, fmt.type_id, 4)
        out[f"{name}_gemv"] = y.numpy().copy()
        z = torch.full((m, n), float("nan"), dtype=torch.float32)
        bm, bn, bk = 16, 16, 32
        ref.gguf[(tr.cdiv(m, bm), tr.cdiv(n, bn))](
            torch.from_numpy(xm.reshape(-1).copy()), w, z, m, n, k, fmt.type_id, bm, bn, bk)
        out[f"{name}_gemm"] = z.numpy().copy()
    out["shape_n_k_m"] = np.array([n, k, m], dtype=np.int64)
    path = os.path.join(HERE, "reference_vectors.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
