"""Quantised projections: one GGUF weight resident in HBM, applied to activations.

This is the caller-side unit of the path: what a decoder runtime holds per ``q/k/v/o/gate/up/down``
matrix.  A projection owns its raw GGUF bytes on one GPU (optionally only the rows of one
tensor-parallel rank), the kernel bound to its shape, the scratch the GEMV may use, and output
buffers, so a call enqueues kernels and nothing else.

Multi-GPU (one process per GPU): weights are column-sharded along N.  GGUF rows are contiguous byte
spans, so rank ``r`` of ``g`` simply owns rows ``[r*N/g, (r+1)*N/g)`` -- no block is split and the
result is bit-identical to the unsharded one of the same launch plan.  Activations are replicated;
every rank ends with the full ``[m, N]`` output, either through the kernels' own stores into every
rank's peer-mapped output (:class:`FusedGatherGroup`, the decode path) or through an NCCL all-gather
(:class:`QuantLinear`, :class:`GatherGroup`).
"""

from __future__ import annotations

import torch

from . import ops
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


class QuantLinearPair:
    """Two projections that read the same activations (gate and up of an MLP), applied in ONE kernel
    launch: ``forward(x)`` returns the ``[m, n1 + n2]`` concatenation, first weight's columns
    first.  A decode GEMV pays several microseconds of launch, staging and tail whatever its size;
    the pair pays them once.  Single GPU (N-sharded runs use :class:`FusedGatherGroup`)."""

    def __init__(self, raw1: torch.Tensor, n1: int, raw2: torch.Tensor, n2: int, encoding, k: int, m: int,
                 variant="auto"):
        self.format = get_format(encoding)
        self.n1, self.n2, self.k, self.m = int(n1), int(n2), int(k), int(m)
        for name, raw, n in (("raw1", raw1, n1), ("raw2", raw2, n2)):
            if not raw.is_cuda or raw.dtype != torch.uint8 or raw.numel() != self.format.weight_bytes(n, k):
                raise ValueError(f"{name} must be the uint8 CUDA tensor of a [{n}, {k}] {self.format.name} weight")
        if raw1.device != raw2.device:
            raise ValueError("both weights must live on the same device")
        self.raw1, self.raw2 = raw1.contiguous(), raw2.contiguous()
        self.device = raw1.device
        self.variant = variant
        self.out = torch.empty((self.m, self.n1 + self.n2), dtype=torch.float32, device=self.device)
        with torch.cuda.device(self.device):
            need = ops.gemv_scratch_bytes(self.format, self.m, self.n1 + self.n2, self.k)
        self._scratch = torch.zeros(need, dtype=torch.uint8, device=self.device) if need else None

    @property
    def weight_bytes_total(self) -> int:
        return self.raw1.numel() + self.raw2.numel()

    def forward(self, x: torch.Tensor, raw1: torch.Tensor | None = None, raw2: torch.Tensor | None = None):
        """Enqueue on the current stream; ``raw1`` / ``raw2`` substitute other weights of the same shapes."""
        return ops.gemv_pair(x, self.raw1 if raw1 is None else raw1, self.n1,
                             self.raw2 if raw2 is None else raw2, self.n2, self.format, self.k,
                             out=self.out, scratch=self._scratch, variant=self.variant)

    __call__ = forward


class GatherGroup:
    """Several projections that consume the same step's activations and whose outputs are needed
    together (e.g. gate and up of one MLP): their local outputs live back to back in one buffer and
    ONE all-gather moves them all, instead of one collective per projection.  Decode messages are
    a few KB to a few hundred KB, so the collective's launch latency, not its bandwidth, is what
    the step pays for."""

    def __init__(self, linears):
        self.linears = list(linears)
        first = self.linears[0]
        self.world, self.group, self.device = first.world, first.group, first.device
        if any(l.world != self.world or l.device != self.device for l in self.linears):
            raise ValueError("projections of a group must share the device and the process group")
        if self.world > 1:
            sizes = [l.m * l.n_local for l in self.linears]
            # every slice starts on a 256-byte boundary (the kernels want 64-byte aligned outputs)
            starts, total = [], 0
            for size in sizes:
                starts.append(total)
                total += -(-size // 64) * 64
            self._local = torch.empty(total, dtype=torch.float32, device=self.device)
            self._gathered = torch.empty((self.world, total), dtype=torch.float32, device=self.device)
            self._spans = []
            for l, size, offset in zip(self.linears, sizes, starts):
                # the kernel writes straight into its slice of the group buffer
                l.out_local = self._local[offset:offset + size].view(l.m, l.n_local)
                self._spans.append((offset, size))

    def forward(self, xs, raws=None):
        """``xs[i]`` is the activation of projection i (``raws[i]`` optionally replaces its weight);
        returns the list of full ``[m, N]`` outputs."""
        for i, l in enumerate(self.linears):
            l.kernel.launch(xs[i], l.raw if raws is None or raws[i] is None else raws[i], l.out_local)
        if self.world > 1:
            import torch.distributed as dist

            dist.all_gather_into_tensor(self._gathered, self._local.view(1, -1), group=self.group)
            for l, (offset, size) in zip(self.linears, self._spans):
                part = self._gathered[:, offset:offset + size].view(self.world, l.m, l.n_local)
                l.out.view(l.m, self.world, l.n_local).copy_(part.permute(1, 0, 2))
        return [l.out for l in self.linears]

    __call__ = forward


class FusedGatherGroup:
    """The same contract as :class:`GatherGroup` without a collective call: every projection's kernel
    stores its columns into every rank's ``[m, N]`` output over NVLink (peer-mapped memory from a
    :class:`tensor_b200.peer.PeerArena`), and the ordering between ranks rides in the same launches:
    the group's first GEMV waits for the peers' previous signal before it reads its activations,
    its last GEMV signals the peers once every output is stored.  A decode step moves a few KB per
    projection, so what the step pays for is latency: no extra launch, and the wait sits behind the
    kernel's weight prefetch.  With ``fold_sync=False`` one barrier kernel follows the group instead.

    Whatever reads the outputs must run after a wait: the next group's first GEMV (folded), or
    :meth:`wait` for any other consumer.

    Every output exists twice and calls alternate between the two copies: a peer signals when its
    kernel ends, not when the consumer of its result has finished reading, so a rank that is one
    call ahead must not store into the buffer its peer may still be reading.  With two copies the
    stores of call t + 2 reuse the buffer of call t, and they start only after this rank has seen the
    peer's signal of call t + 1, which the peer enqueues after everything it did with call t's
    result (stream order).  ``forward`` returns the tensors of the copy it wrote; a CUDA graph
    replays the copy it captured, so capture an even number of calls per replayed sequence."""

    def __init__(self, linears, arena, fold_sync: bool = True, shared_input: bool = False):
        """``shared_input``: the first two projections read the same activations (``xs[0]``; gate and
        up) and go out as one grouped launch."""
        self.linears = list(linears)
        self.arena = arena
        self.fold_sync = fold_sync
        self.shared_input = bool(shared_input) and len(self.linears) >= 2
        first = self.linears[0]
        self.world, self.rank, self.device = first.world, first.rank, first.device
        if arena.world != self.world or arena.rank != self.rank or arena.device != self.device:
            raise ValueError("the arena belongs to another rank, world or device")
        self._targets = [[], []]  # per copy, per projection: the output's address on every rank
        self._outs = [[], []]
        for l in self.linears:
            if l.world != self.world or l.device != self.device:
                raise ValueError("projections of a group must share the device and the process group")
            if l.kernel.op != "gemv":
                raise ValueError("the fused gather covers decode GEMVs (m <= 16)")
            for copy in range(2):
                offset = arena.take(l.m * l.n * 4)
                self._outs[copy].append(arena.view(offset, (l.m, l.n)))
                self._targets[copy].append(arena.ptrs(offset))
            l.out = self._outs[0][-1]
        self._copy = 1  # the first call writes copy 0
        self._pads = arena.pad_ptrs()
        self._pair_scratch = None
        if self.shared_input:
            a, b = self.linears[0], self.linears[1]
            if (a.format, a.k, a.m, a.n) != (b.format, b.k, b.m, b.n):
                raise ValueError("a grouped launch needs two weights of the same format, shape and batch")
            with torch.cuda.device(self.device):
                need = ops.gemv_scratch_bytes(a.format, a.m, a.n_local + b.n_local, a.k)
            if need:
                self._pair_scratch = torch.zeros(need, dtype=torch.uint8, device=self.device)

    def outputs(self, copy: int):
        """The ``[m, N]`` tensors of one of the two copies."""
        return list(self._outs[copy])

    def forward(self, xs, raws=None):
        self._copy ^= 1
        targets, outs = self._targets[self._copy], self._outs[self._copy]
        last = len(self.linears) - 1
        for i, l in enumerate(self.linears):
            l.out = outs[i]
            raw = l.raw if raws is None or raws[i] is None else raws[i]
            sync = 0
            if self.fold_sync and self.world > 1:
                sync = (ops.PEER_WAIT if i == 0 else 0) | (ops.PEER_SIGNAL if i == last else 0)
            if self.shared_input and i == 1:
                continue  # went out with projection 0
            if self.shared_input and i == 0:
                b = self.linears[1]
                raw_b = b.raw if raws is None or raws[1] is None else raws[1]
                if self.fold_sync and self.world > 1 and last == 1:
                    sync |= ops.PEER_SIGNAL
                ops.gemv_pair_sharded(xs[0], raw, l.n_local, raw_b, b.n_local, l.format, l.k, targets[0],
                                      targets[1], l.n, l.rank * l.n_local, b.rank * b.n_local,
                                      scratch=self._pair_scratch, variant=l.kernel.variant,
                                      pad_ptrs=self._pads if sync else None, rank=self.rank, sync=sync)
                continue
            ops.gemv_sharded(xs[i], raw, l.format, l.n_local, l.k, targets[i], l.n, l.rank * l.n_local,
                             scratch=l.kernel._scratch, variant=l.kernel.variant,
                             pad_ptrs=self._pads if sync else None, rank=self.rank, sync=sync)
        if self.world > 1 and not self.fold_sync:
            ops.peer_barrier(self._pads, self.rank, self.device)
        return list(outs)

    def wait(self) -> None:
        """Enqueue the wait a consumer other than the next group needs (no-op after a barrier)."""
        if self.world > 1 and self.fold_sync:
            ops.peer_sync(self._pads, self.rank, self.device, ops.PEER_WAIT)

    __call__ = forward


class ShardedGemvList:
    """Independent projections of one rank of an N-sharded run, issued with one call: a decoder
    layer's q/k/v, o, gate/up, down, or one MLP at several batches.  ``specs`` is a list of
    ``(x, raw_local, encoding, n, k)``: ``raw_local`` holds this rank's ``n / world`` rows of the
    ``[n, k]`` weight, ``x`` the replicated ``[m, k]`` activations.  Every rank ends with every full
    ``[m, n]`` output: the kernels store their columns into all ranks' outputs (peer-mapped memory of
    ``arena``), the first launch of a call waits for the peers' previous signal, the last one signals.
    Outputs exist twice and calls alternate between the copies (see :class:`FusedGatherGroup`; on one GPU the
    second copy lets a step's results be read out while the next step computes).
    With ``world == 1`` no arena is needed and the outputs are ordinary tensors."""

    def __init__(self, specs, arena=None, rank: int = 0, world: int = 1, variant="auto"):
        self.rank, self.world = rank, world
        self.device = specs[0][0].device
        if world > 1 and arena is None:
            raise ValueError("an N-sharded list needs a PeerArena")
        self._outs = [[], []]
        entries = [[], []]
        self.weight_bytes_local = 0
        for x, raw, encoding, n, k in specs:
            fmt = get_format(encoding)
            start, stop = shard_rows(n, rank, world)
            n_local = stop - start
            if raw.numel() != fmt.weight_bytes(n_local, k):
                raise ValueError(f"raw holds {raw.numel()} bytes; {n_local} rows of K={k} need {fmt.weight_bytes(n_local, k)}")
            m = x.numel() // k
            self.weight_bytes_local += raw.numel()
            for copy in range(2):
                if world > 1:
                    offset = arena.take(m * n * 4)
                    out = arena.view(offset, (m, n))
                    dest = (arena.ptrs(offset), n, start)
                else:
                    out = torch.empty((m, n), dtype=torch.float32, device=self.device)
                    dest = out
                self._outs[copy].append(out)
                entries[copy].append((x, raw, fmt, n_local, k, dest))
        pads = arena.pad_ptrs() if world > 1 else None
        sync = (ops.PEER_WAIT | ops.PEER_SIGNAL) if world > 1 else 0
        self._lists = [ops.GemvList(e, pad_ptrs=pads, rank=rank, sync=sync, variant=variant) for e in entries if e]
        self._copy = len(self._lists) - 1

    def outputs(self, copy: int = 0):
        return list(self._outs[copy])

    def rebind(self, index: int, x=None, w=None) -> None:
        for lst in self._lists:
            lst.rebind(index, x=x, w=w)

    def forward(self, stream=None):
        """Enqueue the projections; returns the ``[m, n]`` outputs of the copy this call writes."""
        self._copy = (self._copy + 1) % len(self._lists)
        self._lists[self._copy].launch(stream)
        return list(self._outs[self._copy])

    def wait(self, pads, stream=None) -> None:
        """For a consumer that is not the next call of a list: wait until the peers' stores have landed."""
        if self.world > 1:
            ops.peer_sync(pads, self.rank, self.device, ops.PEER_WAIT, stream)

    __call__ = forward


class DecoderMlp:
    """One decoder MLP at decode batch ``m`` on one GPU, every step a kernel of this library chained
    without launch gaps: ``h += down(silu(gate(n)) * up(n))`` with ``n = rmsnorm(h)``.  ``h`` is the fp32
    residual stream ``[m, hidden]`` (updated in place); gate and up share their activations and run as one
    grouped GEMV; the normalised activations and the SwiGLU product are the bf16 inputs of the
    projections.  The steps between the projections are what a real step pays for besides the GEMVs
    (the reference states them as matmul epilogues and a normalisation kernel:
    packages/tensor-nn/src/tensor_nn/kernels/linear.py:6-100, normalization.py)."""

    def __init__(self, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, norm_weight: torch.Tensor,
                 hidden: int, intermediate: int, m: int, gate_up_format="q4_k", down_format="q4_k", eps: float = 1e-6):
        self.hidden, self.intermediate, self.m, self.eps = int(hidden), int(intermediate), int(m), float(eps)
        self.device = gate.device
        self.norm_weight = norm_weight
        self.normed = torch.empty((m, hidden), dtype=torch.bfloat16, device=self.device)
        self.pair = QuantLinearPair(gate, intermediate, up, intermediate, gate_up_format, hidden, m)
        self.act = torch.empty((m, intermediate), dtype=torch.bfloat16, device=self.device)
        self.down = QuantLinear(down, down_format, hidden, intermediate, m)

    def forward(self, h: torch.Tensor) -> torch.Tensor:
        ops.rmsnorm(h, self.norm_weight, self.eps, out=self.normed)
        gate_up = self.pair.forward(self.normed)
        ops.swiglu(gate_up, out=self.act)
        ops.residual_add(h, self.down.forward(self.act))
        return h

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


__all__ = ["DecoderMlp", "FusedGatherGroup", "GEMV_MAX_ROWS", "GatherGroup", "HostProjection", "QuantLinear", "QuantLinearPair",
           "ShardedGemvList", "all_gather_columns", "shard_rows", "shard_weight_bytes"]
