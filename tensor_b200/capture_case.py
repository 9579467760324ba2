"""A small, self-contained launch sequence of one kernel, sized for a profiler capture.

    python -m tensor_b200.capture_case gemv <batch>            # Q4_K decode GEMV, W = 18944 x 3584
    python -m tensor_b200.capture_case gemm <format> <tokens>  # prefill GEMM, W = 12288 x 4096

A few launches over distinct weight copies (so that every launch streams from HBM: the copies
together exceed the L2) and a synchronize; a few hundred MB on the device, a fraction of a second of
GPU time.  Meant to be run plainly first and then under ``ncu -k regex:<kernel> -s 2 -c 2``.
"""

from __future__ import annotations

import sys

import torch

import tensor_b200 as tb
from tensor_b200 import synth


def main(argv) -> int:
    if len(argv) < 2 or argv[0] not in ("gemv", "gemm"):
        print(__doc__)
        return 2
    dev = torch.device("cuda", 0)
    if argv[0] == "gemv":
        m, n, k, fmt, copies = int(argv[1]), 18944, 3584, "q4_k", 5
        op = "gemv"
    else:
        fmt, m, n, k, copies = argv[1], int(argv[2]), 12288, 4096, 4
        op = "gemm"
    weights = [synth.make_weights(fmt, n, k, seed=i, device=dev) for i in range(copies)]
    x = synth.make_activations(m, k, seed=9, device=dev)
    out = torch.empty(m, n, device=dev)
    kernel = tb.gguf(m, n, k, fmt, op=op)
    for w in weights:
        kernel.launch(x, w, out)
    torch.cuda.synchronize()
    print("device status", tb.device_status())
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
