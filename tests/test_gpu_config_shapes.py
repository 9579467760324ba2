"""The benchmark definition's full-size configurations, checked through properties that do not need
a CPU pass over the whole problem: a slice of weight rows computed by the any-shape kernel (rows
are independent, so a slice of the weight is a valid smaller problem with the same operand
contract), linearity in the activations, and the CPU oracle on a handful of rows."""

import numpy as np
import pytest
import torch

import tensor_b200 as tb
from oracle import c_oracle
from oracle import gguf_oracle as oracle
from tensor_b200 import synth

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda", 0)


def _row_slice(w, name, n, k, start, count):
    rb = tb.get_format(name).row_bytes(k)
    return w.reshape(-1)[start * rb:(start + count) * rb].clone()


def _rel(a, b):
    return float((a - b).norm() / b.norm())


@pytest.fixture(scope="module", autouse=True)
def _no_device_timeouts():
    yield
    assert tb.device_status() == 0


# prefill GEMM: N = 12288, K = 4096 at every M of the definition; 70B-class shapes at M = 4096
@pytest.mark.parametrize("name,m,n,k", [
    ("q4_k", 512, 12288, 4096), ("q4_k", 2048, 12288, 4096),
    ("q6_k", 512, 12288, 4096), ("q6_k", 2048, 12288, 4096),
    ("q4_k", 4096, 28672, 8192), ("q6_k", 4096, 8192, 28672),
])
def test_prefill_gemm_full_size(name, m, n, k):
    w = synth.make_weights(name, n, k, seed=5, device=dev())
    x = synth.make_activations(m, k, seed=6, device=dev())
    out = torch.full((m, n), float("nan"), device=dev())
    tb.gguf(m, n, k, name, op="gemm").launch(x, w, out)
    assert not torch.isnan(out).any()
    # three bands of 64 weight rows through the any-shape kernel (same bf16 operand contract)
    for start in (0, n // 2 - 32, n - 64):
        ws = _row_slice(w, name, n, k, start, 64)
        ref = tb.gemm(x, ws, name, 64, k, variant="simple")
        assert _rel(out[:, start:start + 64], ref) < 1e-4
    # the CPU oracle on the first 8 rows and 32 tokens
    ws = _row_slice(w, name, n, k, 0, 8).cpu().numpy()
    want = c_oracle.gemm(x[:32].float().cpu().numpy(), ws, name, 8, k, operand="bf16")
    assert oracle.rel_frobenius(out[:32, :8].cpu().numpy(), want) < 1e-3
    # zero activations give zeros (no stale accumulator state between launches)
    tb.gguf(m, n, k, name, op="gemm").launch(torch.zeros_like(x), w, out)
    assert torch.count_nonzero(out).item() == 0


# decode step of an 8B-class decoder: q/o, k/v, gate/up in Q4_K, down in Q6_K, batch 1 and 16
@pytest.mark.parametrize("m", [1, 16])
@pytest.mark.parametrize("name,n,k", [
    ("q4_k", 4096, 4096), ("q4_k", 1024, 4096), ("q4_k", 12288, 4096), ("q6_k", 4096, 12288),
])
def test_decode_step_projection(name, n, k, m):
    w = synth.make_weights(name, n, k, seed=7, device=dev())
    x = synth.make_activations(m, k, seed=8, device=dev())
    kern = tb.gguf(m, n, k, name, op="gemv")
    out = torch.full((m, n), float("nan"), device=dev())
    kern.launch(x, w, out)
    want = c_oracle.gemv(x.float().cpu().numpy(), w.cpu().numpy(), name, n, k)
    assert oracle.rel_frobenius(out.cpu().numpy(), want) < 1e-3
    # linearity: y(2.5 x) == 2.5 y(x) up to rounding (2.5 x is exact in bf16 only approximately,
    # so compare against the oracle of the rounded input instead of scaling the output)
    x2 = (x.float() * 2.5).to(torch.bfloat16)
    out2 = torch.full((m, n), float("nan"), device=dev())
    kern.launch(x2, w, out2)
    want2 = c_oracle.gemv(x2.float().cpu().numpy(), w.cpu().numpy(), name, n, k)
    assert oracle.rel_frobenius(out2.cpu().numpy(), want2) < 1e-3
    # N-sharded over 8 ranks: rank r's rows alone give its columns
    per = n // 8
    for r in (0, 5):
        ws = _row_slice(w, name, n, k, r * per, per)
        part = tb.gguf(m, per, k, name, op="gemv")(x, ws)
        assert _rel(part, out[:, r * per:(r + 1) * per]) < 2e-5
