"""The kernels either side of a decode projection (RMS normalisation, SwiGLU, residual add) and the
decoder MLP block that chains them with the GEMVs, against a float64 NumPy statement of the same
arithmetic.  Tolerances: the bf16 outputs are compared after rounding the reference to bf16 (one unit in
the last place allowed for the transcendental), the block's fp32 result to 1e-3 relative Frobenius error."""

import numpy as np
import pytest
import torch

import tensor_b200 as tb
from oracle import c_oracle
from oracle import gguf_oracle as oracle
from tensor_b200 import ops
from tensor_b200.projection import DecoderMlp

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda", 0)


def _bf16(a):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(torch.bfloat16).float().numpy()


@pytest.mark.parametrize("m,k", [(1, 4096), (4, 3584), (16, 1024)])
def test_rmsnorm(m, k):
    rng = np.random.default_rng(m + k)
    x = rng.standard_normal((m, k)).astype(np.float32) * 3
    w = (1 + 0.1 * rng.standard_normal(k)).astype(np.float32)
    got = ops.rmsnorm(torch.from_numpy(x).to(dev()), torch.from_numpy(w).to(dev()), 1e-6).float().cpu().numpy()
    x64 = x.astype(np.float64)
    want = x64 / np.sqrt((x64 ** 2).mean(axis=1, keepdims=True) + 1e-6) * w
    assert np.abs(got - _bf16(want)).max() <= np.abs(want).max() * 2 ** -7  # at most one bf16 step apart
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 4e-3  # bf16 rounding


@pytest.mark.parametrize("m,width", [(1, 18944), (4, 12288), (16, 256)])
def test_swiglu(m, width):
    rng = np.random.default_rng(m + width)
    gu = rng.standard_normal((m, 2 * width)).astype(np.float32) * 2
    got = ops.swiglu(torch.from_numpy(gu).to(dev())).float().cpu().numpy()
    g, u = gu[:, :width].astype(np.float64), gu[:, width:].astype(np.float64)
    want = g / (1 + np.exp(-g)) * u
    assert np.linalg.norm(got - want) / np.linalg.norm(want) < 4e-3


def test_residual_add():
    rng = np.random.default_rng(0)
    a = rng.standard_normal((4, 3584)).astype(np.float32)
    b = rng.standard_normal((4, 3584)).astype(np.float32)
    h = torch.from_numpy(a).to(dev())
    ops.residual_add(h, torch.from_numpy(b).to(dev()))
    assert np.array_equal(h.cpu().numpy(), a + b)


@pytest.mark.parametrize("m", [1, 4])
def test_decoder_mlp_block(m):
    hidden, inter = 1024, 2816
    rng = np.random.default_rng(m)
    raw = {name: oracle.make_weights("q4_k", n, k, seed=s) for s, (name, n, k) in
           enumerate((("gate", inter, hidden), ("up", inter, hidden), ("down", hidden, inter)))}
    norm_w = (1 + 0.1 * rng.standard_normal(hidden)).astype(np.float32)
    h0 = rng.standard_normal((m, hidden)).astype(np.float32)
    put = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev())
    block = DecoderMlp(put(raw["gate"]), put(raw["up"]), put(raw["down"]), put(norm_w), hidden, inter, m)
    h = put(h0.copy())
    for _ in range(2):  # twice on the same buffers: the second call starts from the first one's result
        block(h)
    torch.cuda.synchronize()
    got = h.cpu().numpy()
    # the same two steps on the CPU, with the same roundings of the intermediate activations to bf16
    ref = h0.astype(np.float64)
    for _ in range(2):
        normed = _bf16(ref / np.sqrt((ref ** 2).mean(axis=1, keepdims=True) + 1e-6) * norm_w)
        g = c_oracle.gemv(normed, raw["gate"], "q4_k", inter, hidden).astype(np.float64)
        u = c_oracle.gemv(normed, raw["up"], "q4_k", inter, hidden).astype(np.float64)
        act = _bf16(g / (1 + np.exp(-g)) * u)
        ref = ref + c_oracle.gemv(act, raw["down"], "q4_k", hidden, inter)
    assert np.isfinite(got).all()
    assert np.linalg.norm(got - ref) / np.linalg.norm(ref) < 1e-3
    assert tb.device_status() == 0
