"""``gguf(m, n, k, encoding)``: the reference's operator for this path, backed by sm_100a kernels.

The reference builds its GGUF kernels with ``gguf(m, n, k, encoding, **schedule)``
(benchmarks/kernels/showcase/kernels.py:114-119), which returns the GEMV for ``m == 1`` and the
tensor-core GEMM otherwise, and launches them as ``kernel.launch(x, w, out)`` over flat,
64-byte-aligned buffers (src/tensor/runtime/executable.py:87-154).  ``GgufKernel`` keeps that
surface: same argument names and order, same validation points (arity, dtype, element counts,
alignment, one device), ``ValueError`` / ``TypeError`` for binding problems and a ``RuntimeError``
subclass for provider failures.
"""

from __future__ import annotations

import torch

from . import ops
from .formats import get_format

ARGUMENTS = ("x", "w", "out")
ALIGNMENT = 64  # the reference's kernels declare 64-byte aligned buffers
_X_DTYPES = {"bfloat16": torch.bfloat16, "float16": torch.float16, "float32": torch.float32,
             torch.bfloat16: torch.bfloat16, torch.float16: torch.float16, torch.float32: torch.float32}
GEMV_MAX_ROWS = 16


class GgufKernel:
    def __init__(self, m: int, n: int, k: int, encoding, x_dtype="bfloat16", op: str | None = None,
                 variant="auto", device=None):
        self.format = get_format(encoding)
        if m < 1 or n < 1:
            raise ValueError(f"m and n must be positive, got m={m}, n={n}")
        self.format.row_bytes(k)  # validates K
        self.m, self.n, self.k = int(m), int(n), int(k)
        try:
            self.x_dtype = _X_DTYPES[x_dtype]
        except KeyError:
            raise ValueError(f"unsupported activation dtype {x_dtype!r}") from None
        if op is None:
            op = "gemv" if m <= GEMV_MAX_ROWS else "gemm"
        if op not in ("gemv", "gemm"):
            raise ValueError(f"op must be 'gemv' or 'gemm', got {op!r}")
        if op == "gemm" and self.x_dtype != torch.bfloat16:
            raise ValueError("the prefill GEMM takes bfloat16 activations")
        self.op = op
        self.variant = variant
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._scratch = None
        if op == "gemv" and torch.cuda.is_available():
            with torch.cuda.device(self.device):
                need = ops.gemv_scratch_bytes(self.format, self.m, self.n, self.k, variant=variant, x_dtype=self.x_dtype)
            if need:
                self._scratch = torch.zeros(need, dtype=torch.uint8, device=self.device)

    # -- metadata, named like the manifest fields of the reference artifact ---------------------
    @property
    def arguments(self):
        return [
            {"kind": "buffer", "name": "x", "dtype": str(self.x_dtype).split(".")[-1],
             "shape": [self.m, self.k], "alignment": ALIGNMENT},
            {"kind": "buffer", "name": "w", "dtype": "uint8",
             "shape": [self.format.weight_bytes(self.n, self.k)], "alignment": ALIGNMENT},
            {"kind": "buffer", "name": "out", "dtype": "float32", "shape": [self.m, self.n],
             "alignment": ALIGNMENT},
        ]

    @property
    def outputs(self):
        return ["out"]

    @property
    def weight_bytes(self) -> int:
        return self.format.weight_bytes(self.n, self.k)

    @property
    def flops(self) -> int:
        return 2 * self.m * self.n * self.k

    # -- binding checks (executable.py:93-148) -----------------------------------------------------
    def _check(self, buffers):
        if len(buffers) != len(ARGUMENTS):
            raise ValueError(f"expected {len(ARGUMENTS)} arguments {ARGUMENTS}, got {len(buffers)}")
        expected = {"x": (self.x_dtype, self.m * self.k), "w": (torch.uint8, self.weight_bytes),
                    "out": (torch.float32, self.m * self.n)}
        for name, t in zip(ARGUMENTS, buffers):
            if not isinstance(t, torch.Tensor):
                raise TypeError(f"argument {name!r} must be a torch.Tensor")
        for name, t in zip(ARGUMENTS, buffers):
            dtype, count = expected[name]
            if t.dtype != dtype:
                raise ValueError(f"argument {name!r} has dtype {t.dtype}, expected {dtype}")
            if t.numel() != count:
                raise ValueError(f"argument {name!r} has {t.numel()} elements, expected {count}")
            if not t.is_cuda or t.device != self.device:
                raise ValueError(f"argument {name!r} is on {t.device}, the kernel is bound to {self.device}")
            if not t.is_contiguous():
                raise ValueError(f"argument {name!r} must be contiguous")
            if t.data_ptr() % ALIGNMENT:
                raise ValueError(f"argument {name!r} is not aligned to {ALIGNMENT} bytes")

    def launch(self, x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, stream=None) -> torch.Tensor:
        """Enqueue on ``stream`` (default: torch's current stream of the device); asynchronous."""
        self._check((x, w, out))
        if self.op == "gemv":
            ops.gemv(x, w, self.format, self.n, self.k, out=out, scratch=self._scratch,
                     variant=self.variant, stream=stream)
        else:
            ops.gemm(x, w, self.format, self.n, self.k, out=out, variant=self.variant, stream=stream)
        return out

    def __call__(self, x: torch.Tensor, w: torch.Tensor, stream=None) -> torch.Tensor:
        out = torch.empty((self.m, self.n), dtype=torch.float32, device=self.device)
        return self.launch(x, w, out, stream=stream)


def gguf(m: int, n: int, k: int, encoding, **schedule) -> GgufKernel:
    """Same call as the reference's ``gguf(m, n, k, encoding, **schedule)``.  The reference's
    schedule axes (``threads``, ``unroll``, ``block_m`` ...; benchmark.py:214-237) tune a TileLang
    template and have no meaning here; ``x_dtype``, ``op``, ``variant`` and ``device`` are accepted,
    anything else is rejected so a stale schedule dict does not pass silently."""
    allowed = {"x_dtype", "op", "variant", "device"}
    unknown = set(schedule) - allowed
    if unknown:
        raise ValueError(f"unknown schedule keys {sorted(unknown)}; this backend accepts {sorted(allowed)}")
    return GgufKernel(m, n, k, encoding, **schedule)
