"""Parity of the CUDA path with the CPU oracle, through the C ABI, on a B200.

Gates: dequantisation bit-exact; GEMV / GEMM within 1e-3 relative Frobenius error of the oracle
that applies the same operand contract (GEMV: fp32 weights x activation-as-fp32; GEMM: both
operands rounded to bf16, fp32 accumulate).  Outputs are pre-filled with NaN so an element the
kernel never writes fails the comparison (the reference's idiom,
benchmarks/kernels/showcase/benchmark.py:520).
"""

import os

import numpy as np
import pytest
import torch

import tensor_b200 as tb
from oracle import c_oracle
from oracle import gguf_oracle as oracle

pytestmark = pytest.mark.gpu

TOL = 1e-3  # relative Frobenius error, the gate the benchmark definition states
FORMATS = ("q4_0", "q8_0", "q4_k", "q6_k")
GOLDEN = np.load(os.path.join(os.path.dirname(__file__), "golden", "reference_vectors.npz"))
TORCH_X = {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}


def dev():
    return torch.device("cuda", 0)


def to_dev(a: np.ndarray, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(dev())
    return t if dtype is None else t.to(dtype)


def nan_out(m, n):
    return torch.full((m, n), float("nan"), dtype=torch.float32, device=dev())


@pytest.fixture(scope="module", autouse=True)
def _no_device_timeouts():
    yield
    assert tb.device_status() == 0


# ---- dequantisation ---------------------------------------------------------------------------------

@pytest.mark.parametrize("name", FORMATS)
@pytest.mark.parametrize("n,k", [(1, 256), (12, 512), (37, 1024), (128, 4096)])
def test_dequant_bit_exact(name, n, k):
    raw = oracle.make_weights(name, n, k, seed=n * 1000 + k)
    want = oracle.dequantize(raw, name, n, k)
    got = tb.dequantize(to_dev(raw), name, n, k).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("name", ("q4_0", "q4_k", "q6_k"))
def test_dequant_matches_reference_golden_vectors(name):
    n, k, _ = (int(v) for v in GOLDEN["shape_n_k_m"])
    got = tb.dequantize(to_dev(GOLDEN[f"{name}_raw"]), name, n, k).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), GOLDEN[f"{name}_decode"].view(np.uint32))


def test_dequant_extreme_scale_fields():
    # largest / smallest / subnormal fp16 scales and all-ones quants
    for name in FORMATS:
        fmt = oracle.get_format(name)
        n, k = 4, 512
        raw = oracle.make_weights(name, n, k, seed=5).reshape(n, k // fmt.weights, fmt.nbytes)
        halfs = np.array([65504.0, 6.1e-5, 5.96e-8, 0.0], dtype=np.float16).view(np.uint8).reshape(4, 2)
        off = 208 if name == "q6_k" else 0
        for r in range(n):
            raw[r, :, off:off + 2] = halfs[r]
        raw = raw.reshape(-1)
        want = oracle.dequantize(raw, name, n, k)
        got = tb.dequantize(to_dev(raw), name, n, k).cpu().numpy()
        assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), name


# ---- GEMV ----------------------------------------------------------------------------------------------

def _gemv_case(name, m, n, k, xdt, variant, seed=0, scratch=True):
    raw = oracle.make_weights(name, n, k, seed=seed + 11)
    x = oracle.make_activations(m, k, seed=seed + 12, dtype=xdt)
    want = c_oracle.gemv(x, raw, name, n, k)
    kern = tb.gguf(m, n, k, name, x_dtype={"bf16": "bfloat16", "f16": "float16", "f32": "float32"}[xdt],
                   op="gemv", variant=variant)
    if not scratch:
        kern._scratch = None
    xd, wd = to_dev(x, TORCH_X[xdt]), to_dev(raw)
    out = nan_out(m, n)
    kern.launch(xd, wd, out)
    got = out.cpu().numpy()
    assert np.isfinite(got).all(), "output not fully written"
    err = oracle.rel_frobenius(got, want)
    assert err < TOL, err
    return kern, xd, wd, out, want, err


@pytest.mark.parametrize("name", FORMATS)
@pytest.mark.parametrize("m", [1, 3, 16, 19])
def test_gemv_simple_small(name, m):
    _gemv_case(name, m, 37, 512, "bf16", "simple")


@pytest.mark.parametrize("xdt", ["f16", "f32"])
def test_gemv_simple_activation_dtypes(xdt):
    _gemv_case("q8_0", 1, 64, 1024, xdt, "simple")
    _gemv_case("q6_k", 2, 24, 512, xdt, "simple")


@pytest.mark.parametrize("m", [1, 2, 4, 8, 9, 16])
@pytest.mark.parametrize("n,k", [(16, 256), (40, 512), (130, 2048), (1000, 3584)])
def test_gemv_fast_q4k_small(m, n, k):
    _, _, _, _, _, err = _gemv_case("q4_k", m, n, k, "bf16", "fast")
    assert err < 2e-5, err  # operands are exact; only summation order differs


@pytest.mark.parametrize("m", [1, 4, 16])
def test_gemv_fast_q4k_f16(m):
    _gemv_case("q4_k", m, 72, 1024, "f16", "fast")


@pytest.mark.parametrize("m", [1, 4, 16])
@pytest.mark.parametrize("n,k", [(18944, 3584), (3584, 18944)])
def test_gemv_fast_q4k_config_shapes(m, n, k):
    kern, xd, wd, out, want, _ = _gemv_case("q4_k", m, n, k, "bf16", "fast")
    # replay on the same scratch with changed and with zero activations (scratch must self-reset)
    xd2 = (xd.float() * -1.5).to(torch.bfloat16)
    out.fill_(float("nan"))
    kern.launch(xd2, wd, out)
    want2 = c_oracle.gemv(xd2.float().cpu().numpy(), wd.cpu().numpy(), "q4_k", n, k)
    assert oracle.rel_frobenius(out.cpu().numpy(), want2) < TOL
    out.fill_(float("nan"))
    kern.launch(torch.zeros_like(xd), wd, out)
    assert torch.count_nonzero(out).item() == 0


@pytest.mark.parametrize("name,m,n1,n2,k", [
    ("q4_k", 1, 18944, 18944, 3584),   # gate + up: one launch over both weights
    ("q4_k", 4, 2048, 1024, 3584),
    ("q4_k", 16, 1024, 2048, 2048),
    ("q4_k", 1, 40, 72, 512),          # first weight does not end on a 16-row tile: two launches
    ("q4_k", 4, 1792, 1792, 18944),    # K is split across CTAs: two launches
    ("q6_k", 2, 48, 80, 512),          # served by the fallback kernel
])
def test_gemv_pair_equals_two_gemvs(name, m, n1, n2, k):
    from tensor_b200 import ops, synth
    from tensor_b200.projection import QuantLinearPair

    w1 = synth.make_weights(name, n1, k, seed=1, device=dev())
    w2 = synth.make_weights(name, n2, k, seed=2, device=dev())
    x = synth.make_activations(m, k, seed=3, device=dev())
    pair = QuantLinearPair(w1, n1, w2, n2, name, k, m)
    pair.out.fill_(float("nan"))
    got = pair.forward(x)
    want = torch.cat([tb.gguf(m, n1, k, name, op="gemv")(x, w1), tb.gguf(m, n2, k, name, op="gemv")(x, w2)], dim=1)
    assert not torch.isnan(got).any()
    assert oracle.rel_frobenius(got.cpu().numpy(), want.cpu().numpy()) < 2e-5
    # against the oracle as well (first weight's columns first)
    ref = np.concatenate([c_oracle.gemv(x.float().cpu().numpy(), w.cpu().numpy(), name, n, k)
                          for w, n in ((w1, n1), (w2, n2))], axis=1)
    assert oracle.rel_frobenius(got.cpu().numpy(), ref) < TOL
    # twice on the same scratch
    got2 = pair.forward(x).clone()
    assert torch.equal(got2, got)


def test_gemv_fast_without_scratch_still_correct():
    _gemv_case("q4_k", 1, 512, 18944, "bf16", "auto", scratch=False)


def test_gemv_is_deterministic_and_batch_rows_agree():
    n, k = 3584, 18944
    raw = oracle.make_weights("q4_k", n, k, seed=3)
    x = oracle.make_activations(4, k, seed=4, dtype="bf16")
    wd, xd = to_dev(raw), to_dev(x, torch.bfloat16)
    kern = tb.gguf(4, n, k, "q4_k", op="gemv")
    a = kern(xd, wd).clone()
    b = kern(xd, wd).clone()
    assert torch.equal(a, b)


def test_gemv_auto_falls_back_for_unsupported_layouts():
    # float32 activations and m > 16 are outside the pipelined kernel; auto must still be right
    _gemv_case("q4_k", 1, 64, 512, "f32", "auto")
    _gemv_case("q4_k", 20, 64, 512, "bf16", "auto")
    with pytest.raises(ValueError):
        _gemv_case("q4_k", 20, 64, 512, "bf16", "fast")


# ---- GEMM ----------------------------------------------------------------------------------------------

def _gemm_case(name, m, n, k, variant, seed=0):
    raw = oracle.make_weights(name, n, k, seed=seed + 21)
    x = oracle.make_activations(m, k, seed=seed + 22, dtype="bf16")
    want = c_oracle.gemm(x, raw, name, n, k, operand="bf16")
    out = nan_out(m, n)
    tb.gemm(to_dev(x, torch.bfloat16), to_dev(raw), name, n, k, out=out, variant=variant)
    got = out.cpu().numpy()
    assert np.isfinite(got).all(), "output not fully written"
    err = oracle.rel_frobenius(got, want)
    assert err < TOL, err
    return err


@pytest.mark.parametrize("name", FORMATS)
def test_gemm_simple_small(name):
    _gemm_case(name, 33, 40, 512, "simple")


@pytest.mark.parametrize("name", ["q4_k", "q6_k"])
@pytest.mark.parametrize("m,n,k", [(256, 128, 256), (256, 256, 1024), (300, 200, 512), (17, 128, 2048),
                                   (512, 384, 4096)])
def test_gemm_tcgen05_small(name, m, n, k):
    err = _gemm_case(name, m, n, k, "fast")
    assert err < 1e-4, err  # same operands as the oracle; only accumulation order differs


@pytest.mark.parametrize("name", ["q4_k", "q6_k"])
@pytest.mark.parametrize("m,n,k", [(1024, 128, 256), (1100, 200, 1024), (2048, 384, 512), (1537, 128, 2048)])
def test_gemm_tcgen05_wide_token_tiles(name, m, n, k):
    # M >= 1024 runs 512 tokens per tile (two MMAs per decoded weight tile, two decode groups)
    err = _gemm_case(name, m, n, k, "fast")
    assert err < 1e-4, err


@pytest.mark.parametrize("name", ["q4_k", "q6_k"])
def test_gemm_tcgen05_config_shape(name):
    _gemm_case(name, 256, 12288, 4096, "fast")


def test_gemm_error_vs_fp32_operands_is_reported_scale():
    # bf16 operands against the full-precision product: about 2^-9 per operand (reference reports
    # the same quantity for its fp16 kernels, benchmark.py:544-551)
    n, k, m = 256, 1024, 256
    raw = oracle.make_weights("q6_k", n, k, seed=31)
    x = oracle.make_activations(m, k, seed=32, dtype="bf16")
    full = oracle.gemm_ref(x, raw, "q6_k", n, k, operand="f32", accumulate=np.float64)
    got = tb.gemm(to_dev(x, torch.bfloat16), to_dev(raw), "q6_k", n, k).cpu().numpy()
    assert oracle.rel_frobenius(got, full) < 5e-3


# ---- boundary behaviour ------------------------------------------------------------------------------

def test_binding_errors_are_value_errors():
    n, k = 16, 256
    w = torch.zeros(tb.weight_bytes("q4_k", n, k), dtype=torch.uint8, device=dev())
    x = torch.zeros(1, k, dtype=torch.bfloat16, device=dev())
    with pytest.raises(ValueError):
        tb.gemv(x, w[:-1], "q4_k", n, k)
    with pytest.raises(ValueError):
        tb.gemv(x, w, "q4_k", n, k, out=torch.zeros(1, n, dtype=torch.float16, device=dev()))
    with pytest.raises(ValueError):
        tb.gemm(x.to(torch.float16), w, "q4_k", n, k)
    kern = tb.gguf(1, n, k, "q4_k")
    with pytest.raises(ValueError):
        kern.launch(x.view(-1)[1:].clone()[: k - 1], w, torch.zeros(1, n, device=dev()))


def test_launch_on_a_side_stream_and_graph_replay():
    n, k, m = 1024, 2048, 1
    raw = oracle.make_weights("q4_k", n, k, seed=41)
    x = oracle.make_activations(m, k, seed=42, dtype="bf16")
    wd, xd = to_dev(raw), to_dev(x, torch.bfloat16)
    kern = tb.gguf(m, n, k, "q4_k")
    out = nan_out(m, n)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        kern.launch(xd, wd, out)  # warm-up outside capture
        side.synchronize()
        graph = torch.cuda.CUDAGraph()
        out.fill_(float("nan"))
        with torch.cuda.graph(graph, stream=side):
            kern.launch(xd, wd, out)
        xd.copy_((xd.float() * 2).to(torch.bfloat16))
        graph.replay()
    side.synchronize()
    want = c_oracle.gemv(xd.float().cpu().numpy(), raw, "q4_k", n, k)
    assert oracle.rel_frobenius(out.cpu().numpy(), want) < TOL
