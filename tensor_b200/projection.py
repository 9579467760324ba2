"""Quantised projections: one GGUF weight resident in HBM, applied to activations.

This is the caller-side unit of the path: what a decoder runtime holds per ``q/k/v/o/gate/up/down``
matrix.  A projection owns its raw GGUF bytes on one GPU (optionally only the rows of one
tensor-parallel rank), the kernel bound to its shape, the scratch the GEMV may use, and output
buffers, so a call enqueues kernels and nothing else.

Multi-GPU (one process per GPU): weights are column-sharded along N.  GGUF rows are contiguous byte
spans, so rank ``r`` of ``g`` simply owns rows ``[r*N/g, (r+1)*N/g)`` -- no block is split and the
result is bit-identical to the unsharded one.  ``forward`` then all-gathers the fp32 outputs over
NCCL (NVLink / NVSwitch); activations are replicated.
"""

from __future__ import annotations

import torch

from .formats import get_format
from .kernel import GEMV_MAX_ROWS, GgufKernel


def shard_rows(n: int, rank: int, world: int) -> tuple[int, int]:
    """Rows ``[start, stop)`` of an N-row weight owned by ``rank`` (N must divide evenly)."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"rank {rank} outside world of {world}")
    if n % world:
        raise ValueError(f"N={n} does not split evenly over {world} ranks")
    per = n // world
    return rank * per, (rank + 1) * per


def shard_weight_bytes(raw, encoding, n: int, k: int, rank: int, world: int):
    """The byte span of ``rank``'s rows inside the raw ``[n, k]`` weight (a view, no copy)."""
    fmt = get_format(encoding)
    start, stop = shard_rows(n, rank, world)
    rb = fmt.row_bytes(k)
    flat = raw.reshape(-1)
    if flat.shape[0] != fmt.weight_bytes(n, k):
        raise ValueError("raw byte count does not match [n, k]")
    return flat[start * rb:stop * rb]


def all_gather_columns(out_local: torch.Tensor, gathered: torch.Tensor, out: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather ``out_local[m, n_local]`` of every rank into ``out[m, world * n_local]``.

    ``gathered`` is a ``[world, m, n_local]`` staging buffer (``all_gather_into_tensor`` concatenates
    along dim 0); rank r's columns land at ``[r * n_local, (r + 1) * n_local)`` of every output row.
    Works with any backend (NCCL on GPUs, gloo in the CPU tests).
    """
    import torch.distributed as dist

    world, m, n_local = gathered.shape
    dist.all_gather_into_tensor(gathered.view(world * m, n_local), out_local.view(m, n_local), group=group)
    if m == 1:
        out.view(-1).copy_(gathered.view(-1))
    else:
        out.view(m, world, n_local).copy_(gathered.permute(1, 0, 2))
    return out


class QuantLinear:
    """``y[m, N] = x[m, K] . dequant(W[N, K])^T`` for a fixed batch ``m``.

    ``raw`` holds the bytes of this rank's rows (``n_local = N / world``).  With ``world > 1`` a
    ``torch.distributed`` process group must be initialised; ``forward`` returns the full ``[m, N]``
    output on every rank.
    """

    def __init__(self, raw: torch.Tensor, encoding, n: int, k: int, m: int, x_dtype="bfloat16",
                 op: str | None = None, variant="auto", rank: int = 0, world: int = 1, group=None):
        self.format = get_format(encoding)
        self.n, self.k, self.m = int(n), int(k), int(m)
        self.rank, self.world, self.group = rank, world, group
        start, stop = shard_rows(self.n, rank, world)
        self.n_local = stop - start
        if not raw.is_cuda or raw.dtype != torch.uint8:
            raise ValueError("raw must be a uint8 CUDA tensor holding this rank's rows")
        if raw.numel() != self.format.weight_bytes(self.n_local, self.k):
            raise ValueError(f"raw holds {raw.numel()} bytes; {self.n_local} rows of K={k} in "
                             f"{self.format.name} need {self.format.weight_bytes(self.n_local, self.k)}")
        self.raw = raw.contiguous()
        self.device = raw.device
        self.kernel = GgufKernel(self.m, self.n_local, self.k, self.format, x_dtype=x_dtype, op=op,
                                 variant=variant, device=self.device)
        self.out_local = torch.empty((self.m, self.n_local), dtype=torch.float32, device=self.device)
        if world > 1:
            # all_gather_into_tensor concatenates along dim 0: gather [world, m, n_local]
            self._gathered = torch.empty((world, self.m, self.n_local), dtype=torch.float32, device=self.device)
            self.out = torch.empty((self.m, self.n), dtype=torch.float32, device=self.device)
        else:
            self._gathered = None
            self.out = self.out_local

    @property
    def weight_bytes_local(self) -> int:
        return self.raw.numel()

    @property
    def weight_bytes_total(self) -> int:
        return self.format.weight_bytes(self.n, self.k)

    def forward(self, x: torch.Tensor, raw: torch.Tensor | None = None) -> torch.Tensor:
        """Enqueue on the current stream; returns the (reused) ``[m, N]`` fp32 output buffer.
        ``raw`` substitutes another weight of the same shape (e.g. the next layer's)."""
        self.kernel.launch(x, self.raw if raw is None else raw, self.out_local)
        if self.world > 1:
            all_gather_columns(self.out_local, self._gathered, self.out, group=self.group)
        return self.out

    __call__ = forward


class HostProjection:
    """Host-buffer front end: activations arrive in (pinned) host memory and results are returned
    in host memory; weights stay resident on the GPU.  One call = H2D copy of ``x``, the kernel(s),
    D2H copy of ``y``, and a stream synchronise."""

    def __init__(self, linear: QuantLinear):
        self.linear = linear
        kern = linear.kernel
        self.x_dev = torch.empty((linear.m, linear.k), dtype=kern.x_dtype, device=linear.device)
        self.y_host = torch.empty((linear.m, linear.n), dtype=torch.float32).pin_memory()

    @property
    def h2d_bytes(self) -> int:
        return self.x_dev.numel() * self.x_dev.element_size()

    @property
    def d2h_bytes(self) -> int:
        return self.y_host.numel() * 4

    def __call__(self, x_host: torch.Tensor) -> torch.Tensor:
        self.x_dev.copy_(x_host, non_blocking=True)
        y = self.linear.forward(self.x_dev)
        self.y_host.copy_(y, non_blocking=True)
        torch.cuda.current_stream(self.linear.device).synchronize()
        return self.y_host


__all__ = ["GEMV_MAX_ROWS", "HostProjection", "QuantLinear", "all_gather_columns", "shard_rows",
           "shard_weight_bytes"]
