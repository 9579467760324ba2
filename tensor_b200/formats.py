"""GGUF block formats on the quantised-matmul path.

Ids are GGML type ids, the ``encoding`` argument of the reference's
``gguf(m, n, k, encoding)`` (benchmarks/kernels/showcase/kernels.py:114-119,
benchmarks/kernels/showcase/benchmark.py:122).  Rows are ``k / weights`` consecutive blocks
(benchmarks/kernels/showcase/triton_kernels.py:136,144,164).
"""

from __future__ import annotations

from dataclasses import dataclass


@dataclass(frozen=True)
class BlockFormat:
    name: str
    type_id: int
    weights: int  # values per block
    nbytes: int   # bytes per block

    def row_bytes(self, k: int) -> int:
        if k < 0 or k % self.weights:
            raise ValueError(f"K={k} is not a multiple of the {self.name} block of {self.weights}")
        return k // self.weights * self.nbytes

    def weight_bytes(self, n: int, k: int) -> int:
        if n < 0:
            raise ValueError(f"N={n} is negative")
        return n * self.row_bytes(k)

    @property
    def bits_per_weight(self) -> float:
        return 8.0 * self.nbytes / self.weights


Q4_0 = BlockFormat("q4_0", 2, 32, 18)
Q8_0 = BlockFormat("q8_0", 8, 32, 34)
Q4_K = BlockFormat("q4_k", 12, 256, 144)
Q6_K = BlockFormat("q6_k", 14, 256, 210)

_BY_NAME = {f.name: f for f in (Q4_0, Q8_0, Q4_K, Q6_K)}
_BY_ID = {f.type_id: f for f in _BY_NAME.values()}


def get_format(encoding) -> BlockFormat:
    """Accepts a BlockFormat, a name ("q4_k") or a GGML type id (12)."""
    if isinstance(encoding, BlockFormat):
        return encoding
    try:
        if isinstance(encoding, str):
            return _BY_NAME[encoding.lower()]
        return _BY_ID[int(encoding)]
    except (KeyError, TypeError, ValueError):
        raise ValueError(f"unknown GGUF encoding {encoding!r}; expected one of "
                         f"{sorted(_BY_NAME)} or type ids {sorted(_BY_ID)}") from None
