"""The allocation-free GEMV entry point (`tb200_gguf_gemv_static`), called through the C ABI.

It serves callers that can neither pass a scratch buffer nor let the library allocate one (launch
adapters that forward only declared buffers, hosts with their own memory arena, code inside a
stream capture): the split-K scratch is an array inside the library image.  The test runs a shape
whose plan splits K, twice in a row on the same stream, and requires each result to equal what the
regular entry point produces with caller-provided scratch.  This file sorts last on purpose: a run
that stops at the first failure has then already run every other test.
"""

import ctypes

import numpy as np
import pytest
import torch

import tensor_b200 as tb
from tensor_b200 import abi
from tensor_b200._native import lib

pytestmark = pytest.mark.gpu

STATIC_SCRATCH_BYTES = 4 << 20  # TB200_GEMV_STATIC_SCRATCH_BYTES in include/tensor_b200_gguf.h


def _call_static(fmt_id, x, w, out, m, n, k):
    err = abi.TensorErrorV1()
    status = lib().tb200_gguf_gemv_static(
        fmt_id, abi.DTYPE_IDS["bfloat16"], ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(w.data_ptr()),
        ctypes.c_void_p(out.data_ptr()), m, n, k, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream),
        ctypes.byref(err))
    return status, err.message.decode()


@pytest.mark.parametrize("m", [1, 4, 16])
def test_static_scratch_matches_regular_entry_point_twice(m):
    from tensor_b200 import synth

    dev = torch.device("cuda", 0)
    n, k = 3584, 18944  # short and wide: the plan splits K, so the scratch is really used
    plan = tb.gemv_plan("q4_k", m, n, k)
    assert plan["k_splits"] > 1 and 0 < plan["scratch_bytes"] <= STATIC_SCRATCH_BYTES
    w = synth.make_weights("q4_k", n, k, seed=3, device=dev)
    kern = tb.gguf(m, n, k, "q4_k", op="gemv")  # regular path with its own scratch
    for attempt in range(2):
        x = synth.make_activations(m, k, seed=10 + attempt, device=dev)
        want = kern(x, w)
        got = torch.full((m, n), float("nan"), device=dev)
        status, message = _call_static(12, x, w, got, m, n, k)
        assert status == 0, message
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        # same kernel, same plan, same summation order: tolerance as in the parity tests, and in
        # practice bit-identical
        rel = (got - want).norm() / want.norm()
        assert rel.item() < 1e-3
        assert torch.equal(got, want)
    assert tb.device_status() == 0


def test_static_scratch_rejects_oversized_shapes():
    dev = torch.device("cuda", 0)
    # a shape whose preferred plan wants more than the built-in 4 MiB
    m, n, k = 16, 16384, 65536
    plan = tb.gemv_plan("q4_k", m, n, k)
    if plan["scratch_bytes"] <= STATIC_SCRATCH_BYTES:
        pytest.skip("no oversized plan at this shape on this device")
    dummy = torch.zeros(64, dtype=torch.uint8, device=dev)
    out = torch.zeros(64, device=dev)
    status, message = _call_static(12, dummy, dummy, out, m, n, k)
    assert status == abi.ERROR_ARGUMENT and "4 MiB" in message
