"""Host-side operators over torch CUDA tensors.  PyTorch supplies device memory and streams; the
arithmetic is entirely in the C library (``tensor_b200/csrc``), reached through the reference's
descriptor calling convention (``*_v1`` entry points of include/tensor_b200_gguf.h)."""

from __future__ import annotations

import ctypes

import torch

from . import abi
from ._native import lib, raise_for_status
from .formats import get_format

_TORCH_DTYPE_IDS = {torch.uint8: 3, torch.float16: 10, torch.float32: 11, torch.bfloat16: 13}
_VARIANTS = {"auto": 0, "simple": 1, "fast": 2, "mma": 3, "tc": 4, "dp4a": 5, 0: 0, 1: 1, 2: 2, 3: 3, 4: 4, 5: 5}
_X_DTYPE_NAMES = {"float16": 10, "float32": 11, "bfloat16": 13, torch.float16: 10, torch.float32: 11, torch.bfloat16: 13}
GEMV_LIST_MAX = 12


def _require_cuda(name: str, t: torch.Tensor) -> None:
    if not isinstance(t, torch.Tensor):
        raise TypeError(f"{name} must be a torch.Tensor, got {type(t).__name__}")
    if not t.is_cuda:
        raise ValueError(f"{name} must live on a CUDA device (this path has no CPU fallback)")
    if not t.is_contiguous():
        raise ValueError(f"{name} must be contiguous")


def _buffer(name: str, t: torch.Tensor, shape=None) -> abi.TensorArgumentV1:
    try:
        dtype = _TORCH_DTYPE_IDS[t.dtype]
    except KeyError:
        raise ValueError(f"{name} has unsupported dtype {t.dtype}") from None
    return abi.buffer_argument(t.data_ptr(), t.numel() * t.element_size(), dtype, t.device.index,
                               shape if shape is not None else tuple(t.shape))


def _stream_handle(device: torch.device, stream) -> int:
    if stream is None:
        return torch.cuda.current_stream(device).cuda_stream
    if isinstance(stream, int):
        return stream
    return stream.cuda_stream


def _same_device(*tensors) -> torch.device:
    device = tensors[0].device
    for t in tensors[1:]:
        if t is not None and t.device != device:
            raise ValueError("all buffers of a call must live on the same device")
    return device


def _invoke(fn, arguments, device, stream) -> None:
    call, keep = abi.make_call(arguments, device.index, _stream_handle(device, stream))
    error = abi.TensorErrorV1()
    status = fn(ctypes.byref(call), ctypes.byref(error))
    del keep
    raise_for_status(status, error)


def weight_bytes(encoding, n: int, k: int) -> int:
    return get_format(encoding).weight_bytes(n, k)


def gemv_scratch_bytes(encoding, m: int, n: int, k: int, variant="auto", x_dtype="bfloat16") -> int:
    """Scratch the GEMV can use at this shape on the current device (0: never splits K).  The tensor-memory
    kernel (``variant="tc"``) keeps its converted activations and partial sums there and cannot run without it."""
    fmt = get_format(encoding)
    if _VARIANTS[variant] == _VARIANTS["tc"]:
        item = abi.TB200GemvItem()
        item.format, item.x_dtype = fmt.type_id, _X_DTYPE_NAMES[x_dtype]
        item.m, item.n, item.k, item.out_count, item.out_ld = m, n, k, 1, n
        return int(lib().tb200_gguf_gemv_list_scratch_bytes(ctypes.byref(item), 1))
    return int(lib().tb200_gguf_gemv_scratch_bytes(fmt.type_id, m, n, k))


def gemv_plan(encoding, m: int, n: int, k: int, scratch_bytes: int = 1 << 40) -> dict:
    """The launch plan of the pipelined GEMV at this shape (see ``tb200_gguf_gemv_plan``)."""
    out = (ctypes.c_int32 * 8)()
    status = lib().tb200_gguf_gemv_plan(get_format(encoding).type_id, m, n, k, scratch_bytes, out)
    if status:
        raise ValueError(f"no plan for format {encoding!r}, m={m}, n={n}, k={k}")
    keys = ("pipelined", "k_splits", "row_groups", "sb_per_split", "stages", "smem_bytes",
            "scratch_bytes", "ctas_per_sm")
    plan = dict(zip(keys, (int(v) for v in out)))
    plan["pipelined"] = bool(plan["pipelined"])
    return plan


def device_status() -> int:
    """Synchronise and return the sticky device status word (0 = no bounded wait gave up)."""
    word = ctypes.c_uint32(0)
    error = abi.TensorErrorV1()
    status = lib().tb200_gguf_device_status(ctypes.byref(word), ctypes.byref(error))
    raise_for_status(status, error)
    return int(word.value)


def dequantize(w: torch.Tensor, encoding, n: int, k: int, out: torch.Tensor | None = None,
               stream=None) -> torch.Tensor:
    """fp32 ``[n, k]`` decode of raw GGUF bytes; bit-identical to the reference's ``decode_ggml``
    (benchmarks/kernels/showcase/triton_kernels.py:133-181)."""
    fmt = get_format(encoding)
    _require_cuda("w", w)
    if w.dtype != torch.uint8:
        raise ValueError(f"w must be uint8 raw blocks, got {w.dtype}")
    if w.numel() != fmt.weight_bytes(n, k):
        raise ValueError(f"w holds {w.numel()} bytes; [{n}, {k}] in {fmt.name} needs {fmt.weight_bytes(n, k)}")
    if out is None:
        out = torch.empty((n, k), dtype=torch.float32, device=w.device)
    _require_cuda("out", out)
    device = _same_device(w, out)
    args = [_buffer("w", w, (w.numel(),)), _buffer("out", out, (n, k)),
            abi.scalar_argument(n), abi.scalar_argument(k), abi.scalar_argument(fmt.type_id)]
    _invoke(lib().tb200_gguf_dequant_v1, args, device, stream)
    return out


def _matmul_args(x, w, out, fmt, m, n, k):
    _require_cuda("x", x)
    _require_cuda("w", w)
    _require_cuda("out", out)
    if w.dtype != torch.uint8:
        raise ValueError(f"w must be uint8 raw blocks, got {w.dtype}")
    if x.numel() != m * k:
        raise ValueError(f"x holds {x.numel()} elements; [{m}, {k}] needs {m * k}")
    if w.numel() != fmt.weight_bytes(n, k):
        raise ValueError(f"w holds {w.numel()} bytes; [{n}, {k}] in {fmt.name} needs {fmt.weight_bytes(n, k)}")
    if out.dtype != torch.float32 or out.numel() != m * n:
        raise ValueError(f"out must be float32 with {m * n} elements")
    return [_buffer("x", x, (m, k)), _buffer("w", w, (w.numel(),)), _buffer("out", out, (m, n))]


def _infer_m(x: torch.Tensor, k: int) -> int:
    if k <= 0 or x.numel() % k:
        raise ValueError(f"x with {x.numel()} elements is not a whole number of rows of K={k}")
    return x.numel() // k


def gemv(x: torch.Tensor, w: torch.Tensor, encoding, n: int, k: int, out: torch.Tensor | None = None,
         scratch: torch.Tensor | None = None, variant="auto", stream=None) -> torch.Tensor:
    """Decode GEMV ``out[m, n] = x[m, k] . dequant(w)^T`` (fp32 weights, fp32 accumulate).

    ``scratch`` (uint8, zero-initialised once, reused across calls on one stream) lets the kernel
    split K across CTAs for short-and-wide weights; without it a non-splitting kernel is used.
    """
    fmt = get_format(encoding)
    m = _infer_m(x, k)
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    args = _matmul_args(x, w, out, fmt, m, n, k)
    device = _same_device(x, w, out, scratch)
    if scratch is not None:
        _require_cuda("scratch", scratch)
        if scratch.dtype != torch.uint8:
            raise ValueError("scratch must be uint8")
        args.append(_buffer("scratch", scratch, (scratch.numel(),)))
    args += [abi.scalar_argument(m), abi.scalar_argument(n), abi.scalar_argument(k),
             abi.scalar_argument(fmt.type_id), abi.scalar_argument(_VARIANTS[variant])]
    _invoke(lib().tb200_gguf_gemv_v1, args, device, stream)
    return out


def gemm(x: torch.Tensor, w: torch.Tensor, encoding, n: int, k: int, out: torch.Tensor | None = None,
         variant="auto", stream=None) -> torch.Tensor:
    """Prefill GEMM ``out[m, n] = x[m, k] . dequant(w)^T`` with bf16 operands, fp32 accumulate."""
    fmt = get_format(encoding)
    m = _infer_m(x, k)
    if x.dtype != torch.bfloat16:
        raise ValueError(f"the GEMM takes bfloat16 activations, got {x.dtype}")
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=x.device)
    args = _matmul_args(x, w, out, fmt, m, n, k)
    device = _same_device(x, w, out)
    args += [abi.scalar_argument(m), abi.scalar_argument(n), abi.scalar_argument(k),
             abi.scalar_argument(fmt.type_id), abi.scalar_argument(_VARIANTS[variant])]
    _invoke(lib().tb200_gguf_gemm_v1, args, device, stream)
    return out


_X_DTYPE_IDS = {torch.float16: 10, torch.float32: 11, torch.bfloat16: 13}


PEER_WAIT, PEER_SIGNAL = 1, 2


def gemv_sharded(x: torch.Tensor, w: torch.Tensor, encoding, n: int, k: int, out_ptrs, out_ld: int,
                 col_offset: int, scratch: torch.Tensor | None = None, variant="auto", stream=None,
                 pad_ptrs=None, rank: int = 0, sync: int = 0) -> None:
    """The GEMV of one rank of an N-sharded projection: ``w`` holds this rank's ``n`` rows and the
    ``[m, n]`` result goes to columns ``col_offset .. col_offset + n`` of every ``[m, out_ld]`` fp32
    matrix whose device address is in ``out_ptrs`` (own output first, then the other ranks' outputs
    as mapped by :class:`tensor_b200.peer.PeerArena`).  ``sync`` folds the cross-GPU ordering into
    the launch (``PEER_WAIT`` before the activations are read, ``PEER_SIGNAL`` after the last
    store) over the signal pads ``pad_ptrs`` (rank order).  See ``tb200_gguf_gemv_sharded_sync``."""
    fmt = get_format(encoding)
    m = _infer_m(x, k)
    _require_cuda("x", x)
    _require_cuda("w", w)
    if w.dtype != torch.uint8 or w.numel() != fmt.weight_bytes(n, k):
        raise ValueError(f"w must hold the {fmt.weight_bytes(n, k)} raw bytes of [{n}, {k}] in {fmt.name}")
    try:
        x_dtype = _X_DTYPE_IDS[x.dtype]
    except KeyError:
        raise ValueError(f"unsupported activation dtype {x.dtype}") from None
    if sync and pad_ptrs is None:
        raise ValueError("sync needs the signal pads")
    device = _same_device(x, w, scratch)
    ptrs = [int(p) for p in out_ptrs]
    table = (ctypes.c_void_p * max(len(ptrs), 1))(*ptrs)
    pads = [int(p) for p in (pad_ptrs or [])]
    pad_table = (ctypes.c_void_p * max(len(pads), 1))(*pads)
    error = abi.TensorErrorV1()
    with torch.cuda.device(device):
        status = lib().tb200_gguf_gemv_sharded_sync(
            fmt.type_id, x_dtype, x.data_ptr(), w.data_ptr(), table, len(ptrs), out_ld, col_offset, m, n, k,
            scratch.data_ptr() if scratch is not None else None, scratch.numel() if scratch is not None else 0,
            _VARIANTS[variant], pad_table if pads else None, rank, max(len(pads), 1), sync,
            _stream_handle(device, stream), ctypes.byref(error))
    raise_for_status(status, error)


def peer_sync(pad_ptrs, rank: int, device: torch.device, mode: int = PEER_WAIT | PEER_SIGNAL, stream=None) -> None:
    """Enqueue one or both halves of the cross-GPU barrier (``tb200_peer_sync``) on ``stream``;
    ``pad_ptrs[i]`` is the address of rank i's signal pad as mapped in this process."""
    ptrs = [int(p) for p in pad_ptrs]
    table = (ctypes.c_void_p * max(len(ptrs), 1))(*ptrs)
    error = abi.TensorErrorV1()
    with torch.cuda.device(device):
        status = lib().tb200_peer_sync(table, rank, len(ptrs), mode, _stream_handle(device, stream),
                                       ctypes.byref(error))
    raise_for_status(status, error)


def peer_barrier(pad_ptrs, rank: int, device: torch.device, stream=None) -> None:
    """Signal and wait (``tb200_peer_barrier``)."""
    peer_sync(pad_ptrs, rank, device, PEER_WAIT | PEER_SIGNAL, stream)


class GemvList:
    """Several independent decode GEMVs bound once and launched with one C call
    (``tb200_gguf_gemv_list``): what a decoder layer issues back to back (q/k/v, gate/up), or one
    projection at several batches.  ``variant="tc"`` runs them as ONE persistent tcgen05 launch.  Each entry is ``(x, w, encoding, n, k, out)`` with ``out`` either
    an fp32 ``[m, n]`` tensor or ``(device addresses, row length, column offset)`` for an N-sharded
    rank that stores its columns into every rank's output.  Entries must not depend on one another;
    entries that pass the same ``x`` tensor share its conversion.  The descriptors are kept, so a
    launch is one C call; ``rebind(i, w=..., x=...)`` swaps buffers of the same shape."""

    def __init__(self, entries, pad_ptrs=None, rank: int = 0, sync: int = 0, variant="auto"):
        if not 1 <= len(entries) <= GEMV_LIST_MAX:
            raise ValueError(f"a list holds 1..{GEMV_LIST_MAX} projections, got {len(entries)}")
        self._items = (abi.TB200GemvItem * len(entries))()
        self._keep = []
        self.device = entries[0][0].device
        self.outs = []
        for i, (x, w, encoding, n, k, out) in enumerate(entries):
            fmt = get_format(encoding)
            m = _infer_m(x, k)
            _require_cuda("x", x)
            _require_cuda("w", w)
            if w.dtype != torch.uint8 or w.numel() != fmt.weight_bytes(n, k):
                raise ValueError(f"entry {i}: w must hold the {fmt.weight_bytes(n, k)} raw bytes of [{n}, {k}] in {fmt.name}")
            try:
                x_dtype = _X_DTYPE_IDS[x.dtype]
            except KeyError:
                raise ValueError(f"entry {i}: unsupported activation dtype {x.dtype}") from None
            if x.device != self.device or w.device != self.device:
                raise ValueError("all buffers of a list must live on the same device")
            item = self._items[i]
            item.format, item.x_dtype = fmt.type_id, x_dtype
            item.x, item.w = x.data_ptr(), w.data_ptr()
            item.m, item.n, item.k = m, n, k
            if isinstance(out, torch.Tensor):
                _require_cuda("out", out)
                if out.dtype != torch.float32 or out.numel() != m * n or out.device != self.device:
                    raise ValueError(f"entry {i}: out must be float32 with {m * n} elements on {self.device}")
                item.outs[0] = out.data_ptr()
                item.out_count, item.out_ld = 1, n
            else:
                ptrs, ld, col = out
                if not 1 <= len(ptrs) <= 8 or ld < col + n:
                    raise ValueError(f"entry {i}: bad destinations")
                for d, ptr in enumerate(ptrs):
                    item.outs[d] = int(ptr) + 4 * col
                item.out_count, item.out_ld = len(ptrs), ld
            self._keep.append((x, w, out))
            self.outs.append(out)
        with torch.cuda.device(self.device):
            need = int(lib().tb200_gguf_gemv_list_scratch_bytes(self._items, len(entries)))
        self.scratch = torch.zeros(max(need, 256), dtype=torch.uint8, device=self.device)
        self._pads = [int(p) for p in (pad_ptrs or [])]
        self._pad_table = (ctypes.c_void_p * max(len(self._pads), 1))(*self._pads)
        self.rank, self.sync = rank, sync if self._pads else 0
        self.variant = _VARIANTS[variant]

    def rebind(self, index: int, x: torch.Tensor | None = None, w: torch.Tensor | None = None) -> None:
        """Point entry ``index`` at other activations / weights of the same shape and dtype."""
        item = self._items[index]
        old_x, old_w, out = self._keep[index]
        if x is not None:
            if x.shape != old_x.shape or x.dtype != old_x.dtype or x.device != self.device:
                raise ValueError("rebind needs activations of the same shape, dtype and device")
            item.x = x.data_ptr()
        if w is not None:
            if w.numel() != old_w.numel() or w.dtype != torch.uint8 or w.device != self.device:
                raise ValueError("rebind needs a weight of the same byte size")
            item.w = w.data_ptr()
        self._keep[index] = (old_x if x is None else x, old_w if w is None else w, out)

    def launch(self, stream=None) -> None:
        error = abi.TensorErrorV1()
        with torch.cuda.device(self.device):
            status = lib().tb200_gguf_gemv_list(
                self._items, len(self._items), self.scratch.data_ptr(), self.scratch.numel(), self.variant,
                self._pad_table if self._pads else None, self.rank, max(len(self._pads), 1), self.sync,
                _stream_handle(self.device, stream), ctypes.byref(error))
        raise_for_status(status, error)

    __call__ = launch


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float = 1e-6, out: torch.Tensor | None = None, stream=None):
    """``out[r] = bf16(x[r] * rsqrt(mean(x[r]^2) + eps) * weight)`` for fp32 ``x [m, k]`` (``tb200_rmsnorm_bf16``):
    the residual stream turned into the activations of the next projection."""
    _require_cuda("x", x)
    _require_cuda("weight", weight)
    if x.dtype != torch.float32 or weight.dtype != torch.float32 or x.dim() != 2 or weight.numel() != x.shape[1]:
        raise ValueError("rmsnorm takes float32 x [m, k] and float32 weight [k]")
    m, k = x.shape
    if out is None:
        out = torch.empty((m, k), dtype=torch.bfloat16, device=x.device)
    _require_cuda("out", out)
    if out.dtype != torch.bfloat16 or out.numel() != m * k:
        raise ValueError("out must be bfloat16 [m, k]")
    device = _same_device(x, weight, out)
    error = abi.TensorErrorV1()
    with torch.cuda.device(device):
        status = lib().tb200_rmsnorm_bf16(x.data_ptr(), weight.data_ptr(), out.data_ptr(), m, k, float(eps),
                                          _stream_handle(device, stream), ctypes.byref(error))
    raise_for_status(status, error)
    return out


def swiglu(gate_up: torch.Tensor, out: torch.Tensor | None = None, stream=None):
    """``out = bf16(silu(gate) * up)`` for the fp32 ``[m, 2 * width]`` output of a grouped gate + up launch
    (gate in the first ``width`` columns); ``tb200_swiglu_bf16``."""
    _require_cuda("gate_up", gate_up)
    if gate_up.dtype != torch.float32 or gate_up.dim() != 2 or gate_up.shape[1] % 2:
        raise ValueError("swiglu takes float32 [m, 2 * width]")
    m, width = gate_up.shape[0], gate_up.shape[1] // 2
    if out is None:
        out = torch.empty((m, width), dtype=torch.bfloat16, device=gate_up.device)
    _require_cuda("out", out)
    if out.dtype != torch.bfloat16 or out.numel() != m * width:
        raise ValueError("out must be bfloat16 [m, width]")
    device = _same_device(gate_up, out)
    error = abi.TensorErrorV1()
    with torch.cuda.device(device):
        status = lib().tb200_swiglu_bf16(gate_up.data_ptr(), out.data_ptr(), m, width, _stream_handle(device, stream),
                                         ctypes.byref(error))
    raise_for_status(status, error)
    return out


def residual_add(stream_buffer: torch.Tensor, delta: torch.Tensor, stream=None):
    """``stream_buffer += delta`` (fp32, in place); ``tb200_residual_add``."""
    _require_cuda("stream_buffer", stream_buffer)
    _require_cuda("delta", delta)
    if stream_buffer.dtype != torch.float32 or delta.dtype != torch.float32 or stream_buffer.numel() != delta.numel():
        raise ValueError("residual_add takes two float32 tensors of the same size")
    device = _same_device(stream_buffer, delta)
    error = abi.TensorErrorV1()
    with torch.cuda.device(device):
        status = lib().tb200_residual_add(stream_buffer.data_ptr(), delta.data_ptr(), stream_buffer.numel(),
                                          _stream_handle(device, stream), ctypes.byref(error))
    raise_for_status(status, error)
    return stream_buffer


def set_peer_wait_limit(nanoseconds: int) -> None:
    """How long kernels wait for another GPU's signal before giving up (0: the default, two seconds)."""
    lib().tb200_peer_set_wait_limit(int(nanoseconds))


def gemv_pair(x: torch.Tensor, w1: torch.Tensor, n1: int, w2: torch.Tensor, n2: int, encoding, k: int,
              out: torch.Tensor | None = None, scratch: torch.Tensor | None = None, variant="auto",
              stream=None) -> torch.Tensor:
    """Two weights over the same activations in one launch: ``out[m, n1 + n2]`` holds
    ``x . dequant(w1)^T`` in its first ``n1`` columns and ``x . dequant(w2)^T`` in the rest
    (``tb200_gguf_gemv_pair``).  ``scratch``: as for :func:`gemv` at the shape ``(m, n1 + n2, k)``."""
    fmt = get_format(encoding)
    m = _infer_m(x, k)
    _require_cuda("x", x)
    _require_cuda("w1", w1)
    _require_cuda("w2", w2)
    for name, w, n in (("w1", w1, n1), ("w2", w2, n2)):
        if w.dtype != torch.uint8 or w.numel() != fmt.weight_bytes(n, k):
            raise ValueError(f"{name} must hold the {fmt.weight_bytes(n, k)} raw bytes of [{n}, {k}] in {fmt.name}")
    try:
        x_dtype = _X_DTYPE_IDS[x.dtype]
    except KeyError:
        raise ValueError(f"unsupported activation dtype {x.dtype}") from None
    if out is None:
        out = torch.empty((m, n1 + n2), dtype=torch.float32, device=x.device)
    _require_cuda("out", out)
    if out.dtype != torch.float32 or out.numel() != m * (n1 + n2):
        raise ValueError(f"out must be float32 with {m * (n1 + n2)} elements")
    device = _same_device(x, w1, w2, out, scratch)
    error = abi.TensorErrorV1()
    with torch.cuda.device(device):
        status = lib().tb200_gguf_gemv_pair(
            fmt.type_id, x_dtype, x.data_ptr(), w1.data_ptr(), n1, w2.data_ptr(), n2, out.data_ptr(), m, k,
            scratch.data_ptr() if scratch is not None else None, scratch.numel() if scratch is not None else 0,
            _VARIANTS[variant], _stream_handle(device, stream), ctypes.byref(error))
    raise_for_status(status, error)
    return out


def gemv_pair_sharded(x: torch.Tensor, w1: torch.Tensor, n1: int, w2: torch.Tensor, n2: int, encoding, k: int,
                      out1_ptrs, out2_ptrs, out_ld: int, col_offset1: int, col_offset2: int,
                      scratch: torch.Tensor | None = None, variant="auto", stream=None, pad_ptrs=None,
                      rank: int = 0, sync: int = 0) -> None:
    """:func:`gemv_pair` for one rank of an N-sharded pair of projections: the two weights' columns go
    to their own windows of every rank's two outputs (``tb200_gguf_gemv_pair_sharded_sync``)."""
    fmt = get_format(encoding)
    m = _infer_m(x, k)
    for name, t in (("x", x), ("w1", w1), ("w2", w2)):
        _require_cuda(name, t)
    for name, w, n in (("w1", w1, n1), ("w2", w2, n2)):
        if w.dtype != torch.uint8 or w.numel() != fmt.weight_bytes(n, k):
            raise ValueError(f"{name} must hold the {fmt.weight_bytes(n, k)} raw bytes of [{n}, {k}] in {fmt.name}")
    try:
        x_dtype = _X_DTYPE_IDS[x.dtype]
    except KeyError:
        raise ValueError(f"unsupported activation dtype {x.dtype}") from None
    if len(out1_ptrs) != len(out2_ptrs):
        raise ValueError("both outputs need the same number of destinations")
    if sync and pad_ptrs is None:
        raise ValueError("sync needs the signal pads")
    device = _same_device(x, w1, w2, scratch)
    count = len(out1_ptrs)
    table1 = (ctypes.c_void_p * max(count, 1))(*[int(p) for p in out1_ptrs])
    table2 = (ctypes.c_void_p * max(count, 1))(*[int(p) for p in out2_ptrs])
    pads = [int(p) for p in (pad_ptrs or [])]
    pad_table = (ctypes.c_void_p * max(len(pads), 1))(*pads)
    error = abi.TensorErrorV1()
    with torch.cuda.device(device):
        status = lib().tb200_gguf_gemv_pair_sharded_sync(
            fmt.type_id, x_dtype, x.data_ptr(), w1.data_ptr(), n1, w2.data_ptr(), n2, table1, table2, count, out_ld,
            col_offset1, col_offset2, m, k, scratch.data_ptr() if scratch is not None else None,
            scratch.numel() if scratch is not None else 0, _VARIANTS[variant], pad_table if pads else None, rank,
            max(len(pads), 1), sync, _stream_handle(device, stream), ctypes.byref(error))
    raise_for_status(status, error)
