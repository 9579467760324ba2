"""The CPU oracle against the reference's own outputs (committed golden vectors), against the
third-party gguf package, and the C restatement against the NumPy one."""

import os

import numpy as np
import pytest

from oracle import c_oracle
from oracle import gguf_oracle as oracle

GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))
N, K, M = (int(v) for v in GOLDEN["shape_n_k_m"])
REFERENCE_FORMATS = ("q4_0", "q4_k", "q6_k")  # the three the reference states
ALL_FORMATS = ("q4_0", "q8_0", "q4_k", "q6_k")


@pytest.mark.parametrize("name", REFERENCE_FORMATS)
def test_decode_bit_exact_vs_reference_triton(name):
    got = oracle.dequantize(GOLDEN[f"{name}_raw"], name, N, K)
    assert np.array_equal(got.view(np.uint32), GOLDEN[f"{name}_decode"].view(np.uint32))


@pytest.mark.parametrize("name", ALL_FORMATS)
def test_decode_bit_exact_vs_gguf_py_vectors(name):
    got = oracle.dequantize(GOLDEN[f"{name}_raw"], name, N, K)
    assert np.array_equal(got.view(np.uint32), GOLDEN[f"{name}_gguf_py"].view(np.uint32))


@pytest.mark.parametrize("name", ALL_FORMATS)
def test_c_oracle_decode_bit_exact(name):
    got = c_oracle.dequantize(GOLDEN[f"{name}_raw"], name, N, K)
    want = oracle.dequantize(GOLDEN[f"{name}_raw"], name, N, K)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("name", REFERENCE_FORMATS)
def test_gemv_vs_reference_triton(name):
    raw, x = GOLDEN[f"{name}_raw"], GOLDEN[f"{name}_x1"]
    want = GOLDEN[f"{name}_gemv"]
    for got in (oracle.gemv_ref(x, raw, name, N, K)[0], c_oracle.gemv(x, raw, name, N, K)[0]):
        assert oracle.rel_frobenius(got, want) < 1e-6


@pytest.mark.parametrize("name", REFERENCE_FORMATS)
def test_gemm_f16_operands_vs_reference_triton(name):
    raw, x = GOLDEN[f"{name}_raw"], GOLDEN[f"{name}_xm"]
    got = oracle.gemm_ref(x, raw, name, N, K, operand="f16")
    assert oracle.rel_frobenius(got, GOLDEN[f"{name}_gemm"]) < 1e-6


@pytest.mark.parametrize("name", ALL_FORMATS)
def test_gemm_bf16_c_vs_numpy(name):
    raw = GOLDEN[f"{name}_raw"]
    x = oracle.bf16_round(GOLDEN[f"{name}_xm"])
    got = c_oracle.gemm(x, raw, name, N, K, operand="bf16")
    want = oracle.gemm_ref(x, raw, name, N, K, operand="bf16", accumulate=np.float64)
    assert oracle.rel_frobenius(got, want) < 1e-6


@pytest.mark.parametrize("name", ALL_FORMATS)
def test_against_installed_gguf_py(name):
    gguf = pytest.importorskip("gguf")
    from gguf.quants import dequantize

    kinds = {"q4_0": gguf.GGMLQuantizationType.Q4_0, "q8_0": gguf.GGMLQuantizationType.Q8_0,
             "q4_k": gguf.GGMLQuantizationType.Q4_K, "q6_k": gguf.GGMLQuantizationType.Q6_K}
    n, k = 24, 1024
    raw = oracle.make_weights(name, n, k, seed=7)
    want = dequantize(raw.reshape(n, -1), kinds[name]).astype(np.float32)
    assert np.array_equal(oracle.dequantize(raw, name, n, k).view(np.uint32), want.view(np.uint32))
    assert np.array_equal(c_oracle.dequantize(raw, name, n, k).view(np.uint32), want.view(np.uint32))


def test_sizes_and_errors():
    assert oracle.row_bytes("q8_0", 4096) == 4352
    assert oracle.row_bytes("q4_k", 3584) == 2016
    assert oracle.row_bytes("q4_k", 18944) == 10656
    assert oracle.row_bytes("q6_k", 4096) == 3360
    assert oracle.weight_bytes("q4_k", 18944, 3584) == 38191104
    assert oracle.weight_bytes("q6_k", 12288, 4096) == 41287680
    with pytest.raises(ValueError):
        oracle.row_bytes("q4_k", 100)
    with pytest.raises(ValueError):
        oracle.dequantize(np.zeros(10, np.uint8), "q4_0", 1, 32)


def test_bf16_round_ties_to_even():
    vals = np.array([1.0, 1.00390625, 1.01171875, -1.00390625, 3.0e38, 0.0], dtype=np.float32)
    got = oracle.bf16_round(vals)
    # 1 + 2^-8 is a tie between 1.0 and 1 + 2^-7: even mantissa wins (1.0)
    assert got[1] == np.float32(1.0)
    # 1 + 3*2^-8 ties between 1+2^-7 and 1+2^-6: even is 1+2^-6
    assert got[2] == np.float32(1.015625)
    assert got[3] == np.float32(-1.0)
    torch = pytest.importorskip("torch")
    rnd = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    want = torch.from_numpy(rnd).to(torch.bfloat16).float().numpy()
    assert np.array_equal(oracle.bf16_round(rnd), want)


def test_synthetic_weights_are_finite():
    for name in ALL_FORMATS:
        w = oracle.dequantize(oracle.make_weights(name, 8, 512, seed=3), name, 8, 512)
        assert np.isfinite(w).all() and np.abs(w).max() > 0
