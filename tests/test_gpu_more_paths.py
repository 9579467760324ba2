"""GPU paths that the main parity file does not reach: the specialised inner loops of the staged SIMT
GEMV at the shapes that select them, the first configuration of the benchmark definition at its own
size, the persistent tcgen05 / TMEM GEMV (an explicit variant), the list entry point, and a
cross-GPU wait that runs out.  Everything goes through the C ABI and is compared with the CPU oracle
(relative Frobenius error <= 1e-3, the gate of benchmarks/kernels/showcase/benchmark.py:466-470's
contract as the benchmark definition states it)."""

import ctypes

import numpy as np
import pytest
import torch

import tensor_b200 as tb
from oracle import c_oracle
from oracle import gguf_oracle as oracle
from tensor_b200 import abi, ops
from tensor_b200._native import lib

pytestmark = pytest.mark.gpu
TOL = 1e-3
TORCH_X = {"bf16": torch.bfloat16, "f16": torch.float16}


def dev():
    return torch.device("cuda", 0)


def to_dev(a, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(a)).to(dev())
    return t if dtype is None else t.to(dtype)


@pytest.fixture(scope="module", autouse=True)
def _no_device_timeouts():
    yield
    assert tb.device_status() == 0


def _case(name, m, n, k, xdt, variant, seed=0):
    raw = oracle.make_weights(name, n, k, seed=seed + 3)
    x = oracle.make_activations(m, k, seed=seed + 4, dtype=xdt)
    want = c_oracle.gemv(x, raw, name, n, k)
    out = torch.full((m, n), float("nan"), device=dev())
    kern = tb.gguf(m, n, k, name, x_dtype={"bf16": "bfloat16", "f16": "float16"}[xdt], op="gemv", variant=variant)
    kern.launch(to_dev(x, TORCH_X[xdt]), to_dev(raw), out)
    got = out.cpu().numpy()
    assert np.isfinite(got).all()
    err = oracle.rel_frobenius(got, want)
    assert err < TOL, err
    return err


# rows whose byte stride is a multiple of 16 and that fit the staged kernel's shared memory: the
# lane-owns-a-run inner loops for Q6_K, Q8_0 and Q4_0
@pytest.mark.parametrize("m", [1, 2, 4])
@pytest.mark.parametrize("k", [2048, 4096])
def test_staged_simt_gemv_q6k(m, k):
    _case("q6_k", m, 520, k, "bf16", "auto", seed=m + k)


@pytest.mark.parametrize("name", ["q8_0", "q4_0"])
@pytest.mark.parametrize("m", [1, 3])
def test_staged_simt_gemv_small_blocks(name, m):
    _case(name, m, 384, 4096, "bf16", "auto", seed=m)


def test_config1_q8_0_4096x4096_fp16():
    """The benchmark definition's first configuration at its own size."""
    _case("q8_0", 1, 4096, 4096, "f16", "auto")


def test_q6k_down_projection_shape():
    _case("q6_k", 1, 4096, 12288, "bf16", "auto")


# ---- Q6_K at batch 1: the integer dot-product kernel (what "auto" picks there) --------------------

@pytest.mark.parametrize("n,k,xdt", [(8, 2048, "bf16"), (520, 2048, "bf16"), (300, 4096, "f16"), (4096, 12288, "bf16"),
                                     (1000, 6144, "bf16"), (33, 18432, "f16"), (5000, 32768, "bf16")])
def test_q6k_batch1_integer_dot_product(n, k, xdt):
    """One, two, three, six, nine and sixteen warps per row (K = 2048 ... 32768), row counts that leave the last
    CTA and the last batch ragged; a second launch must give the same bits."""
    raw = oracle.make_weights("q6_k", n, k, seed=n + k)
    x = oracle.make_activations(1, k, seed=n + k + 1, dtype=xdt)
    want = c_oracle.gemv(x, raw, "q6_k", n, k)
    kern = tb.gguf(1, n, k, "q6_k", x_dtype={"bf16": "bfloat16", "f16": "float16"}[xdt], op="gemv")
    xd, wd = to_dev(x, TORCH_X[xdt]), to_dev(raw)
    results = []
    for _ in range(2):
        out = torch.full((1, n), float("nan"), device=dev())
        kern.launch(xd, wd, out)
        got = out.cpu().numpy()
        assert np.isfinite(got).all()
        assert oracle.rel_frobenius(got, want) < 3e-5  # operands are exact to 2^-21 of a run's largest activation
        results.append(got)
    assert np.array_equal(results[0], results[1])
    # scaled (by a power of two: exact in the activation type) and zero activations
    kern.launch(xd * -2, wd, out)
    assert oracle.rel_frobenius(out.cpu().numpy(), -2 * want) < 3e-5
    kern.launch(torch.zeros_like(xd), wd, out)
    assert float(out.abs().max()) == 0.0


@pytest.mark.parametrize("n,k,xdt", [(64, 256, "bf16"), (300, 1024, "f16"), (1000, 2304, "bf16"), (18944, 3584, "bf16"),
                                     (3584, 18944, "bf16"), (777, 32768, "f16")])
def test_q4k_batch1_integer_dot_product(n, k, xdt):
    """The same kernel on Q4_K blocks (an explicit variant): rows whose last warp holds fewer than eight blocks,
    one to sixteen warps per row."""
    raw = oracle.make_weights("q4_k", n, k, seed=n + k)
    x = oracle.make_activations(1, k, seed=n + k + 1, dtype=xdt)
    want = c_oracle.gemv(x, raw, "q4_k", n, k)
    kern = tb.gguf(1, n, k, "q4_k", x_dtype={"bf16": "bfloat16", "f16": "float16"}[xdt], op="gemv", variant="dp4a")
    xd, wd = to_dev(x, TORCH_X[xdt]), to_dev(raw)
    results = []
    for _ in range(2):
        out = torch.full((1, n), float("nan"), device=dev())
        kern.launch(xd, wd, out)
        got = out.cpu().numpy()
        assert np.isfinite(got).all()
        assert oracle.rel_frobenius(got, want) < 3e-5
        results.append(got)
    assert np.array_equal(results[0], results[1])
    kern.launch(torch.zeros_like(xd), wd, out)
    assert float(out.abs().max()) == 0.0


@pytest.mark.parametrize("encoding", ["q8_0", "q4_0"])
@pytest.mark.parametrize("n,k,xdt", [(64, 256, "bf16"), (300, 1024, "f16"), (1000, 2304, "bf16"), (4096, 4096, "bf16"),
                                     (4096, 12288, "f16"), (555, 32768, "bf16")])
def test_blocks_of_32_batch1_integer_dot_product(encoding, n, k, xdt):
    """Q8_0 and Q4_0 on the integer dot-product kernel (eight blocks of 32 stand for one block of 256): against
    the oracle, finite, bit-identical from launch to launch, and the same answer as the explicit variant."""
    raw = oracle.make_weights(encoding, n, k, seed=n + k)
    x = oracle.make_activations(1, k, seed=n + k + 1, dtype=xdt)
    want = c_oracle.gemv(x, raw, encoding, n, k)
    x_dtype = {"bf16": "bfloat16", "f16": "float16"}[xdt]
    xd, wd = to_dev(x, TORCH_X[xdt]), to_dev(raw)
    results = []
    for variant in ("dp4a", "dp4a", "auto"):
        kern = tb.gguf(1, n, k, encoding, x_dtype=x_dtype, op="gemv", variant=variant)
        out = torch.full((1, n), float("nan"), device=dev())
        kern.launch(xd, wd, out)
        got = out.cpu().numpy()
        assert np.isfinite(got).all()
        assert oracle.rel_frobenius(got, want) < 3e-5
        results.append(got)
    assert np.array_equal(results[0], results[1])
    kern.launch(torch.zeros_like(xd), wd, out)
    assert float(out.abs().max()) == 0.0
    # twice the activations (exact in bf16 / fp16): twice the result, bit for bit
    kern = tb.gguf(1, n, k, encoding, x_dtype=x_dtype, op="gemv", variant="dp4a")
    kern.launch((xd.float() * -2.0).to(xd.dtype), wd, out)
    assert np.array_equal(out.cpu().numpy(), results[0] * np.float32(-2.0))


@pytest.mark.parametrize("encoding,k", [("q6_k", 2048), ("q8_0", 256), ("q4_0", 768), ("q4_k", 512)])
@pytest.mark.parametrize("n", [1, 3, 149])
def test_integer_dot_product_few_rows_and_nan(encoding, k, n):
    """Fewer rows than a CTA has row streams, and one row more than there are SMs; a NaN among the activations
    reaches every output, as it does in the reference arithmetic."""
    raw = oracle.make_weights(encoding, n, k, seed=n + k)
    x = oracle.make_activations(1, k, seed=n + k + 1, dtype="bf16")
    want = c_oracle.gemv(x, raw, encoding, n, k)
    kern = tb.gguf(1, n, k, encoding, op="gemv", variant="dp4a")
    xd, wd = to_dev(x, torch.bfloat16), to_dev(raw)
    out = torch.full((1, n), float("nan"), device=dev())
    kern.launch(xd, wd, out)
    assert oracle.rel_frobenius(out.cpu().numpy(), want) < 3e-5
    xd[0, k // 2 + 5] = float("nan")
    kern.launch(xd, wd, out)
    assert bool(torch.isnan(out).all())
    assert tb.device_status() == 0


def test_q6k_batch1_tiny_and_huge_activations():
    """A run of 32 activations is scaled by its own power of two: magnitudes far apart between runs survive."""
    n, k = 64, 2048
    raw = oracle.make_weights("q6_k", n, k, seed=5)
    x = oracle.make_activations(1, k, seed=6, dtype="bf16")  # fp32 values that are exact in bf16
    x[:, :512] *= np.float32(2.0 ** -40)                      # powers of two keep them so
    x[:, 512:1024] *= np.float32(2.0 ** 30)
    xd = to_dev(x, torch.bfloat16)
    want = c_oracle.gemv(x, raw, "q6_k", n, k)
    out = torch.full((1, n), float("nan"), device=dev())
    tb.gguf(1, n, k, "q6_k", op="gemv").launch(xd, to_dev(raw), out)
    assert oracle.rel_frobenius(out.cpu().numpy(), want) < 3e-5


# ---- the persistent tcgen05 / TMEM kernel ---------------------------------------------------------

@pytest.mark.parametrize("m,n,k", [(1, 128, 256), (2, 128, 3584), (4, 300, 1024), (8, 1000, 2048), (16, 2048, 3584),
                                   (3, 18944, 3584), (16, 3584, 18944)])
def test_tensor_memory_gemv(m, n, k):
    raw = oracle.make_weights("q4_k", n, k, seed=m + n)
    x = oracle.make_activations(m, k, seed=m + n + 1, dtype="bf16")
    want = c_oracle.gemv(x, raw, "q4_k", n, k)
    xd, wd = to_dev(x, torch.bfloat16), to_dev(raw)
    lst = ops.GemvList([(xd, wd, "q4_k", n, k, torch.full((m, n), float("nan"), device=dev()))], variant="tc")
    for _ in range(2):  # the second launch runs on the scratch the first one left behind
        lst.outs[0].fill_(float("nan"))
        lst.launch()
        got = lst.outs[0].cpu().numpy()
        assert np.isfinite(got).all()
        err = oracle.rel_frobenius(got, want)
        assert err < 3e-5, err  # operands are exact; only summation order differs


@pytest.mark.parametrize("m,n,k", [(1, 128, 2048), (2, 300, 4096), (16, 520, 2048), (5, 4096, 12288)])
def test_tensor_memory_gemv_q6k(m, n, k):
    """Q6_K blocks are 2-byte aligned: every block offset inside the staged 16-byte window occurs."""
    raw = oracle.make_weights("q6_k", n, k, seed=m + n)
    x = oracle.make_activations(m, k, seed=m + n + 1, dtype="bf16")
    want = c_oracle.gemv(x, raw, "q6_k", n, k)
    out = torch.full((m, n), float("nan"), device=dev())
    lst = ops.GemvList([(to_dev(x, torch.bfloat16), to_dev(raw), "q6_k", n, k, out)], variant="tc")
    for _ in range(2):
        out.fill_(float("nan"))
        lst.launch()
        got = out.cpu().numpy()
        assert np.isfinite(got).all()
        assert oracle.rel_frobenius(got, want) < 3e-5


def test_tensor_memory_gemv_f16_activations():
    m, n, k = 4, 256, 1024
    raw = oracle.make_weights("q4_k", n, k, seed=9)
    x = oracle.make_activations(m, k, seed=10, dtype="f16")
    out = torch.full((m, n), float("nan"), device=dev())
    ops.GemvList([(to_dev(x, torch.float16), to_dev(raw), "q4_k", n, k, out)], variant="tc").launch()
    assert oracle.rel_frobenius(out.cpu().numpy(), c_oracle.gemv(x, raw, "q4_k", n, k)) < 3e-5


@pytest.mark.parametrize("variant", ["auto", "tc"])
def test_gemv_list_mixed_batches(variant):
    """Projections of different shapes and batches in one call; two of them share their activations."""
    shapes = [(1, 1024, 2048), (1, 640, 2048), (4, 640, 2048), (16, 512, 1024), (1, 384, 4096)]
    entries, wants = [], []
    shared = None
    for i, (m, n, k) in enumerate(shapes):
        raw = oracle.make_weights("q4_k", n, k, seed=50 + i)
        if i == 1:
            x, xd = shared
        else:
            x = oracle.make_activations(m, k, seed=60 + i, dtype="bf16")
            xd = to_dev(x, torch.bfloat16)
        if i == 0:
            shared = (x, xd)
        entries.append((xd, to_dev(raw), "q4_k", n, k, torch.full((m, n), float("nan"), device=dev())))
        wants.append(c_oracle.gemv(x, raw, "q4_k", n, k))
    lst = ops.GemvList(entries, variant=variant)
    for _ in range(2):
        for e in entries:
            e[5].fill_(float("nan"))
        lst.launch()
        for e, want in zip(entries, wants):
            got = e[5].cpu().numpy()
            assert np.isfinite(got).all()
            assert oracle.rel_frobenius(got, want) < TOL


@pytest.mark.parametrize("shared_scratch", [False, True])
def test_gemv_list_converts_batched_activations_first(shared_scratch):
    """An MLP at batch 1, 4 and 16 as one list (gate and up share their activations; the down projection splits
    K): with a scratch slice per launch the conversions of the batched activations run ahead of the first GEMV,
    with a buffer that only holds the largest need every conversion runs right before its GEMV; both must give
    the results of single launches, call after call."""
    entries, wants = [], []
    for m in (1, 4, 16):
        xs = {k: oracle.make_activations(m, k, seed=90 + m + k, dtype="bf16") for k in (1024, 6144)}
        xd = {k: to_dev(v, torch.bfloat16) for k, v in xs.items()}
        for j, (n, k) in enumerate(((768, 1024), (768, 1024), (256, 6144))):
            raw = oracle.make_weights("q4_k", n, k, seed=100 + 10 * m + j)
            entries.append((xd[k], to_dev(raw), "q4_k", n, k, torch.full((m, n), float("nan"), device=dev())))
            wants.append(c_oracle.gemv(xs[k], raw, "q4_k", n, k))
    lst = ops.GemvList(entries)
    if shared_scratch:
        largest = max(ops.gemv_scratch_bytes("q4_k", e[5].shape[0], e[3], e[4]) for e in entries)
        pair = ops.gemv_scratch_bytes("q4_k", 16, 1536, 1024)
        lst.scratch = torch.zeros(max(largest, pair, 256), dtype=torch.uint8, device=dev())
        assert lst.scratch.numel() < int(ops.lib().tb200_gguf_gemv_list_scratch_bytes(lst._items, len(entries)))
    for _ in range(3):
        for e in entries:
            e[5].fill_(float("nan"))
        lst.launch()
        for e, want in zip(entries, wants):
            got = e[5].cpu().numpy()
            assert np.isfinite(got).all()
            assert oracle.rel_frobenius(got, want) < TOL
    assert tb.device_status() == 0


def test_gemv_list_twelve_batched_items_and_mixed_kernels():
    """The longest list, every item batched (twelve conversions in one launch); then a list whose items go to
    four different kernels (pipelined Q4_K at batch 16, tensor-memory Q6_K at batch 16, integer dot-product Q8_0
    at batch 1, SIMT for fp32 activations), each with its own slice of the scratch."""
    entries, wants = [], []
    for i in range(12):
        m, n, k = (2, 4, 8, 16)[i % 4], 256 + 64 * i, (1024, 2048, 3584)[i % 3]
        raw = oracle.make_weights("q4_k", n, k, seed=200 + i)
        x = oracle.make_activations(m, k, seed=220 + i, dtype="bf16")
        entries.append((to_dev(x, torch.bfloat16), to_dev(raw), "q4_k", n, k, torch.full((m, n), float("nan"), device=dev())))
        wants.append(c_oracle.gemv(x, raw, "q4_k", n, k))
    lst = ops.GemvList(entries)
    for _ in range(2):
        for e in entries:
            e[5].fill_(float("nan"))
        lst.launch()
        for e, want in zip(entries, wants):
            assert oracle.rel_frobenius(e[5].cpu().numpy(), want) < TOL
    entries, wants = [], []
    for i, (name, m, n, k, xdt) in enumerate((("q4_k", 16, 512, 2048, "bf16"), ("q6_k", 16, 256, 2048, "bf16"),
                                              ("q8_0", 1, 300, 1024, "f16"), ("q4_k", 4, 128, 512, "f32"),
                                              ("q4_k", 16, 640, 3584, "bf16"))):
        raw = oracle.make_weights(name, n, k, seed=240 + i)
        x = oracle.make_activations(m, k, seed=250 + i, dtype=xdt)
        xd = to_dev(x, {"bf16": torch.bfloat16, "f16": torch.float16, "f32": torch.float32}[xdt])
        entries.append((xd, to_dev(raw), name, n, k, torch.full((m, n), float("nan"), device=dev())))
        wants.append(c_oracle.gemv(x, raw, name, n, k))
    lst = ops.GemvList(entries)
    for _ in range(2):
        for e in entries:
            e[5].fill_(float("nan"))
        lst.launch()
        for e, want in zip(entries, wants):
            assert oracle.rel_frobenius(e[5].cpu().numpy(), want) < TOL
    assert tb.device_status() == 0


def test_gemv_list_other_formats_fall_back():
    m, n, k = 2, 96, 512
    entries, wants = [], []
    for i, name in enumerate(("q6_k", "q6_k")):
        raw = oracle.make_weights(name, n, k, seed=70 + i)
        x = oracle.make_activations(m, k, seed=80 + i, dtype="bf16")
        entries.append((to_dev(x, torch.bfloat16), to_dev(raw), name, n, k, torch.full((m, n), float("nan"), device=dev())))
        wants.append(c_oracle.gemv(x, raw, name, n, k))
    ops.GemvList(entries).launch()
    for e, want in zip(entries, wants):
        assert oracle.rel_frobenius(e[5].cpu().numpy(), want) < TOL
    with pytest.raises(ValueError):
        ops.GemvList(entries, variant="tc").launch()


# ---- a cross-GPU wait that runs out ----------------------------------------------------------------

def test_peer_wait_runs_out_and_reports():
    """World of two whose second rank never shows up: both pads live on this GPU, nobody signals.
    The wait must give up after the limit, the status word must name the missing peer, and reading it
    must clear it.  Nothing faults or hangs: the kernel returns normally."""
    pads = torch.zeros(2 * 64, dtype=torch.int32, device=dev())
    table = [pads.data_ptr(), pads.data_ptr() + 256]
    tb.set_peer_wait_limit(2_000_000)  # 2 ms
    try:
        ops.peer_sync(table, 0, dev(), ops.PEER_SIGNAL)  # this rank announces once ...
        ops.peer_sync(table, 0, dev(), ops.PEER_WAIT)    # ... and waits for a peer that never will
        word = ctypes.c_uint32(0)
        error = abi.TensorErrorV1()
        status = lib().tb200_gguf_device_status(ctypes.byref(word), ctypes.byref(error))
        assert status == abi.ERROR_PROVIDER
        assert word.value == 0x90000 | 1
        assert b"bounded device-side wait" in error.message
        assert tb.device_status() == 0  # cleared by the read
    finally:
        tb.set_peer_wait_limit(0)
    # the context is still usable
    assert torch.ones(4, device=dev()).sum().item() == 4
