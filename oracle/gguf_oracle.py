"""CPU oracle for the GGUF quantised-matmul path (TEST INFRASTRUCTURE, not product code).

This module restates, in NumPy, the block arithmetic the reference states in
``benchmarks/kernels/showcase/triton_kernels.py:133-181`` (``decode_ggml`` for
GGML type ids 2 / 12 / 14 = Q4_0 / Q4_K / Q6_K), the operand contracts of its
fused GEMM (``triton_kernels.py:184-210``: operands rounded to the MMA type,
fp32 accumulate) and GEMV (``triton_kernels.py:213-222``: fp32 weight x fp32
activation), and the closures the showcase harness validates against
(``benchmarks/kernels/showcase/benchmark.py:466-477``).

Q8_0 (type id 8) does not appear anywhere in the reference; its arithmetic is
the GGML format definition (34-byte blocks: fp16 ``d`` then 32 int8 quants,
``w = d * q``), so for Q8_0 parity with the reference is unpinned and only
pinned against the third-party ``gguf`` package.

The functions here are the checker.  Only tests, the smoke check and the
``cpu_baseline`` leg of the benchmark may import this module; the CUDA path
never routes through it.

Pinning: ``tests/golden/make_golden.py`` runs the reference's own Triton
kernels in Triton's CPU interpreter and stores their outputs;
``tests/test_oracle.py`` checks this module against those vectors and against
``gguf.quants.dequantize``.
"""

from __future__ import annotations

from dataclasses import dataclass

import numpy as np


@dataclass(frozen=True)
class BlockFormat:
    """One GGUF block encoding: ``weights`` values are stored in ``nbytes`` bytes."""

    name: str
    type_id: int  # GGML type id, the ``encoding`` of showcase/benchmark.py:122
    weights: int
    nbytes: int


Q4_0 = BlockFormat("q4_0", 2, 32, 18)
Q8_0 = BlockFormat("q8_0", 8, 32, 34)
Q4_K = BlockFormat("q4_k", 12, 256, 144)
Q6_K = BlockFormat("q6_k", 14, 256, 210)

FORMATS = {f.name: f for f in (Q4_0, Q8_0, Q4_K, Q6_K)}
BY_TYPE_ID = {f.type_id: f for f in FORMATS.values()}


def get_format(fmt) -> BlockFormat:
    if isinstance(fmt, BlockFormat):
        return fmt
    if isinstance(fmt, str):
        return FORMATS[fmt.lower()]
    return BY_TYPE_ID[int(fmt)]


def row_bytes(fmt, k: int) -> int:
    """Bytes of one weight row of ``k`` channels (triton_kernels.py:136,144,164)."""
    f = get_format(fmt)
    if k % f.weights:
        raise ValueError(f"K={k} is not a multiple of the {f.name} block of {f.weights}")
    return k // f.weights * f.nbytes


def weight_bytes(fmt, n: int, k: int) -> int:
    return n * row_bytes(fmt, k)


# --------------------------------------------------------------------------
# bf16 / fp16 rounding helpers (the MMA operand contract)
# --------------------------------------------------------------------------

def bf16_round(a: np.ndarray) -> np.ndarray:
    """Round fp32 to the nearest bfloat16 (ties to even); result kept as fp32."""
    a = np.ascontiguousarray(a, dtype=np.float32)
    bits = a.view(np.uint32).astype(np.uint64)
    lsb = (bits >> 16) & 1
    rounded = ((bits + 0x7FFF + lsb) >> 16) << 16
    out = rounded.astype(np.uint32).view(np.float32)
    nan = np.isnan(a)
    if nan.any():
        out = out.copy()
        out[nan] = np.nan
    return out.reshape(a.shape)


def bf16_bits(a: np.ndarray) -> np.ndarray:
    """fp32 -> uint16 bfloat16 bit patterns (RNE)."""
    return (bf16_round(a).view(np.uint32) >> 16).astype(np.uint16)


def bf16_from_bits(bits: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(bits, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def f16_round(a: np.ndarray) -> np.ndarray:
    return np.asarray(a, dtype=np.float32).astype(np.float16).astype(np.float32)


def round_operand(a: np.ndarray, operand: str) -> np.ndarray:
    if operand == "bf16":
        return bf16_round(a)
    if operand == "f16":
        return f16_round(a)
    if operand == "f32":
        return np.asarray(a, dtype=np.float32)
    raise ValueError(operand)


# --------------------------------------------------------------------------
# Dequantisation (fp32), one function per format
# --------------------------------------------------------------------------

def _blocks(raw: np.ndarray, fmt: BlockFormat, n: int, k: int) -> np.ndarray:
    raw = np.ascontiguousarray(raw, dtype=np.uint8).reshape(-1)
    need = weight_bytes(fmt, n, k)
    if raw.size != need:
        raise ValueError(f"{fmt.name}: expected {need} bytes for [{n},{k}], got {raw.size}")
    return raw.reshape(n, k // fmt.weights, fmt.nbytes)


def _f16_field(blocks: np.ndarray, offset: int) -> np.ndarray:
    """Little-endian fp16 at ``offset`` of every block, widened to fp32."""
    lo = blocks[..., offset].astype(np.uint16)
    hi = blocks[..., offset + 1].astype(np.uint16)
    return (lo | (hi << 8)).view(np.float16).astype(np.float32)


def dequant_q4_0(raw, n, k):
    """triton_kernels.py:135-142: ``w = (nibble - 8) * d``; weights 0..15 of a
    block are the low nibbles of bytes 2..17, weights 16..31 the high nibbles."""
    b = _blocks(raw, Q4_0, n, k)
    d = _f16_field(b, 0)
    q = b[..., 2:18]
    nib = np.concatenate([q & 15, q >> 4], axis=-1).astype(np.int32) - 8
    return (nib.astype(np.float32) * d[..., None]).reshape(n, k)


def dequant_q8_0(raw, n, k):
    """GGML format definition (not in the reference): ``w = d * int8``."""
    b = _blocks(raw, Q8_0, n, k)
    d = _f16_field(b, 0)
    q = b[..., 2:34].view(np.int8).astype(np.float32)
    return (q * d[..., None]).reshape(n, k)


def q4_k_scales(b: np.ndarray):
    """The sixteen 6-bit fields of a Q4_K block (triton_kernels.py:152-156).

    Returns (sc, mn), each ``[..., 8]`` int32 for the 8 groups of 32 weights.
    """
    s = b[..., 4:16].astype(np.int32)
    s0, s1, s2 = s[..., 0:4], s[..., 4:8], s[..., 8:12]
    sc = np.concatenate([s0 & 63, (s2 & 15) | ((s0 >> 6) << 4)], axis=-1)
    mn = np.concatenate([s1 & 63, (s2 >> 4) | ((s1 >> 6) << 4)], axis=-1)
    return sc, mn


def dequant_q4_k(raw, n, k):
    """triton_kernels.py:143-162: ``w = d*sc*nibble - dmin*mn``.

    Group g (32 weights) of a super-block uses bytes ``16 + (g//2)*32 .. +32``,
    low nibbles for even g and high nibbles for odd g.  Both products are
    exact in fp32; the subtraction rounds once.
    """
    b = _blocks(raw, Q4_K, n, k)
    d = _f16_field(b, 0)
    dmin = _f16_field(b, 2)
    sc, mn = q4_k_scales(b)
    qs = b[..., 16:144].reshape(*b.shape[:-1], 4, 32)
    nib = np.stack([qs & 15, qs >> 4], axis=-2).reshape(*b.shape[:-1], 8, 32)
    scale = d[..., None] * sc.astype(np.float32)
    minimum = dmin[..., None] * mn.astype(np.float32)
    w = scale[..., None] * nib.astype(np.float32) - minimum[..., None]
    return w.astype(np.float32).reshape(n, k)


def dequant_q6_k(raw, n, k):
    """triton_kernels.py:163-180: ``w = (q - 32) * sc * d`` with
    ``q = ql nibble | (qh 2 bits << 4)``, int8 sub-scale per 16 weights."""
    b = _blocks(raw, Q6_K, n, k)
    ql = b[..., 0:128].reshape(*b.shape[:-1], 2, 64).astype(np.int32)
    qh = b[..., 128:192].reshape(*b.shape[:-1], 2, 32).astype(np.int32)
    sc = b[..., 192:208].view(np.int8).astype(np.float32)
    d = _f16_field(b, 208)
    quarters = []
    for quarter in range(4):
        lo = ql[..., (quarter % 2) * 32:(quarter % 2) * 32 + 32]
        lo = (lo >> (quarter // 2 * 4)) & 15
        hi = (qh >> (quarter * 2)) & 3
        quarters.append(lo | (hi << 4))
    q = np.stack(quarters, axis=-2)  # [..., half, quarter, lane]
    q = q.reshape(*b.shape[:-1], 256) - 32
    scale = np.repeat(sc, 16, axis=-1)
    w = q.astype(np.float32) * scale * d[..., None]
    return w.astype(np.float32).reshape(n, k)


_DEQUANT = {"q4_0": dequant_q4_0, "q8_0": dequant_q8_0, "q4_k": dequant_q4_k, "q6_k": dequant_q6_k}


def dequantize(raw, fmt, n: int, k: int) -> np.ndarray:
    """Raw GGUF bytes of an ``[n, k]`` row-major weight -> fp32 ``[n, k]``."""
    return _DEQUANT[get_format(fmt).name](raw, n, k)


# --------------------------------------------------------------------------
# GEMV / GEMM contracts
# --------------------------------------------------------------------------

def gemv_ref(x: np.ndarray, raw, fmt, n: int, k: int, accumulate=np.float32) -> np.ndarray:
    """Decode GEMV oracle: ``out[b, n] = sum_k f32(x[b,k]) * dequant(W)[n,k]``.

    benchmark.py:468-470 / triton_kernels.py:218-221: the activation is used as
    fp32 (fp16 / bf16 activations widen exactly) and the decoded weight is fp32.
    """
    x = np.asarray(x, dtype=np.float32).reshape(-1, k)
    w = dequantize(raw, fmt, n, k)
    return (x.astype(accumulate) @ w.astype(accumulate).T).astype(np.float32)


def gemm_ref(x: np.ndarray, raw, fmt, n: int, k: int, operand: str = "bf16",
             accumulate=np.float32) -> np.ndarray:
    """Prefill GEMM oracle: both operands rounded to the MMA operand type, fp32
    accumulate (benchmark.py:471-477 with ``.half()``; triton_kernels.py:201-207).
    ``operand="f32"`` gives the full-precision product the reference reports
    its ``relative_l2_error_vs_fp32_operands`` against (benchmark.py:544-551).
    """
    x = round_operand(np.asarray(x, dtype=np.float32).reshape(-1, k), operand)
    w = round_operand(dequantize(raw, fmt, n, k), operand)
    return (x.astype(accumulate) @ w.astype(accumulate).T).astype(np.float32)


def rel_frobenius(actual: np.ndarray, expected: np.ndarray) -> float:
    """``||a - e||_F / ||e||_F`` in float64 (benchmark.py:548-550)."""
    a = np.asarray(actual, dtype=np.float64)
    e = np.asarray(expected, dtype=np.float64)
    return float(np.linalg.norm(a - e) / max(np.linalg.norm(e), 1e-12))


# --------------------------------------------------------------------------
# Seeded synthetic inputs with the value distributions of the benchmark configs
# --------------------------------------------------------------------------

def _f16_bytes(values: np.ndarray) -> np.ndarray:
    return np.ascontiguousarray(values.astype(np.float16)).view(np.uint8).reshape(*values.shape, 2)


def make_weights(fmt, n: int, k: int, seed: int) -> np.ndarray:
    """Raw bytes of a random ``[n, k]`` weight in format ``fmt``.

    fp16 scale fields are drawn from the stated distributions and then viewed
    as bytes (never random bytes, which would contain NaN/Inf); quants and
    packed 6-bit scales are uniform bytes.
      Q8_0: d = |N(0,1)|*0.02, int8 quants uniform in [-127,127]
      Q4_0: d = |N(0,1)|*0.02, nibbles uniform
      Q4_K: d, dmin = |N(0,1)|*0.01, 12 scale bytes + 128 quant bytes uniform
      Q6_K: ql/qh uniform, int8 sub-scales uniform in [-64,63], d = |N(0,1)|*0.005
    """
    f = get_format(fmt)
    rng = np.random.default_rng(seed)
    nb = k // f.weights
    if k % f.weights:
        raise ValueError("K must be a multiple of the block size")
    b = np.empty((n, nb, f.nbytes), dtype=np.uint8)
    if f is Q8_0:
        b[..., 0:2] = _f16_bytes(np.abs(rng.standard_normal((n, nb), dtype=np.float32)) * 0.02)
        b[..., 2:34] = rng.integers(-127, 128, size=(n, nb, 32), dtype=np.int8).view(np.uint8)
    elif f is Q4_0:
        b[..., 0:2] = _f16_bytes(np.abs(rng.standard_normal((n, nb), dtype=np.float32)) * 0.02)
        b[..., 2:18] = rng.integers(0, 256, size=(n, nb, 16), dtype=np.uint8)
    elif f is Q4_K:
        b[..., 0:2] = _f16_bytes(np.abs(rng.standard_normal((n, nb), dtype=np.float32)) * 0.01)
        b[..., 2:4] = _f16_bytes(np.abs(rng.standard_normal((n, nb), dtype=np.float32)) * 0.01)
        b[..., 4:144] = rng.integers(0, 256, size=(n, nb, 140), dtype=np.uint8)
    else:
        b[..., 0:192] = rng.integers(0, 256, size=(n, nb, 192), dtype=np.uint8)
        b[..., 192:208] = rng.integers(-64, 64, size=(n, nb, 16), dtype=np.int8).view(np.uint8)
        b[..., 208:210] = _f16_bytes(np.abs(rng.standard_normal((n, nb), dtype=np.float32)) * 0.005)
    return b.reshape(-1)


def make_activations(m: int, k: int, seed: int, dtype: str = "bf16") -> np.ndarray:
    """``[m, k]`` activations ~ N(0,1), already rounded to ``dtype``, held as fp32."""
    rng = np.random.default_rng(seed)
    return round_operand(rng.standard_normal((m, k), dtype=np.float32), dtype)
