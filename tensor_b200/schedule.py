"""Schedule spaces, legality, measured search and profiles for the pipelined kernels.

The reference chooses the launch configuration of its generated projection kernels by searching a
schedule space behind a correctness gate and storing the winner per shape
(src/tensor/compiler/cuda/schedules.py:3-52 for the spaces and ``projection_legal``,
src/tensor/compiler/search.py:29-159 for the search, src/tensor/compiler/tuning.py:207-268 for the
measurement).  The kernels here are written by hand, so a schedule is a small set of launch choices
instead of a code-generation recipe, but the workflow is the same: enumerate, keep what is legal,
run each candidate, reject any whose result differs from the reference result of the default
schedule, time the rest with CUDA events over weights that do not fit L2, keep the fastest, and
record it so the ordinary entry points use it for that shape.
"""

from __future__ import annotations

import ctypes
import itertools
import json
import statistics

from . import abi
from ._native import lib, raise_for_status
from .formats import get_format

OP_GEMV, OP_GEMM = 1, 2
_OPS = {"gemv": OP_GEMV, "gemm": OP_GEMM}
AXES = ("k_splits", "ctas_per_sm", "convert_ahead", "overlap", "gemm_shape")

#: decode GEMV: CTAs along K per 16-row tile, CTAs per SM, where batched activations are converted
DECODE_SPACE = {"k_splits": (1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 12, 14, 16), "ctas_per_sm": (1, 2), "convert_ahead": (1, 2)}
#: prefill GEMM: <256-token tiles per CTA, decode warp groups>
PREFILL_SPACE = {"gemm_shape": (11, 12, 22)}


def projection_space(phase: str, m: int = 1) -> dict:
    """The axes worth searching for a phase (``"decode"`` or ``"prefill"``), like the reference's
    ``projection_space``; at batch 1 there is nothing to convert ahead of the launch."""
    if phase == "decode":
        space = dict(DECODE_SPACE)
        if m == 1:
            space["convert_ahead"] = (2,)
        return {"gemv": space}
    if phase == "prefill":
        return {"gemm": dict(PREFILL_SPACE)}
    raise ValueError("requires prefill or decode schedule space")


def _struct(config: dict) -> abi.TB200Schedule:
    s = abi.TB200Schedule()
    for axis in AXES:
        setattr(s, axis, int(config.get(axis, 0)))
    return s


def legal(op: str, encoding, m: int, n: int, k: int, config: dict, scratch_bytes: int = 1 << 40) -> bool:
    """Whether the kernel can run ``config`` at this shape (shared memory, scratch, non-empty K ranges ...);
    the role of the reference's ``projection_legal``.  Needs no GPU: judged for a B200 when none is present."""
    return bool(lib().tb200_gguf_schedule_legal(_OPS[op], get_format(encoding).type_id, m, n, k, scratch_bytes,
                                                ctypes.byref(_struct(config))))


def candidates(op: str, encoding, m: int, n: int, k: int, space: dict | None = None):
    """Every legal point of the space, the all-derived schedule ``{}`` first."""
    if space is None:
        space = projection_space("decode" if op == "gemv" else "prefill", m)[op]
    yield {}
    axes = list(space)
    for values in itertools.product(*(space[a] for a in axes)):
        config = dict(zip(axes, values))
        if legal(op, encoding, m, n, k, config):
            yield config


def record(op: str, encoding, m: int, n: int, k: int, config: dict) -> None:
    """Make ``config`` the default for this exact shape in this process."""
    status = lib().tb200_gguf_schedule_record(_OPS[op], get_format(encoding).type_id, m, n, k, ctypes.byref(_struct(config)))
    if status:
        raise ValueError("cannot record a schedule for this operation or format")


def clear() -> None:
    """Forget every recorded schedule (the shipped ones included): everything is derived again."""
    lib().tb200_gguf_schedule_clear()


def run_scheduled(op: str, x, w, encoding, n: int, k: int, config: dict, out, scratch=None, stream=None):
    """One launch with a pinned schedule (``tb200_gguf_gemv_scheduled`` / ``tb200_gguf_gemm_scheduled``)."""
    import torch

    from .ops import _X_DTYPE_IDS, _stream_handle

    fmt = get_format(encoding)
    m = x.numel() // k
    error = abi.TensorErrorV1()
    sched = _struct(config)
    with torch.cuda.device(x.device):
        handle = _stream_handle(x.device, stream)
        if op == "gemv":
            status = lib().tb200_gguf_gemv_scheduled(
                fmt.type_id, _X_DTYPE_IDS[x.dtype], x.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k,
                scratch.data_ptr() if scratch is not None else None, scratch.numel() if scratch is not None else 0,
                ctypes.byref(sched), handle, ctypes.byref(error))
        else:
            status = lib().tb200_gguf_gemm_scheduled(fmt.type_id, _X_DTYPE_IDS[x.dtype], x.data_ptr(), w.data_ptr(),
                                                     out.data_ptr(), m, n, k, ctypes.byref(sched), handle, ctypes.byref(error))
    raise_for_status(status, error)
    return out


def search(op: str, encoding, m: int, n: int, k: int, device=None, space: dict | None = None, tolerance: float = 1e-3,
           repeats: int = 5, l2_bytes: int = 126 << 20, seed: int = 0) -> dict:
    """Time every legal schedule on the current GPU and return ``{"best": config, "us": ..., "rows": [...]}``.

    Correctness gate first: a candidate whose output differs from the default schedule's by more than
    ``tolerance`` (relative Frobenius norm) is rejected and never timed.  Timing: CUDA events around
    a CUDA graph that walks enough distinct weight copies to exceed three times the L2 cache, median of
    ``repeats`` replays (the reference conditions L2 between samples, tuning.py:15-82)."""
    import torch

    from . import synth
    from .ops import gemv_scratch_bytes

    fmt = get_format(encoding)
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    copies = max(2, -(-3 * l2_bytes // fmt.weight_bytes(n, k)))
    ws = [synth.make_weights(fmt, n, k, seed=seed + c, device=device) for c in range(copies)]
    x = synth.make_activations(m, k, seed=seed + 1000, device=device)
    need = gemv_scratch_bytes(fmt, m, n, k) if op == "gemv" else 0
    # a split finer than the default plan's needs more partial-sum space
    scratch = torch.zeros(max(need, 4096 + 64 * m * n * 4), dtype=torch.uint8, device=device) if op == "gemv" else None
    out = torch.empty((m, n), dtype=torch.float32, device=device)
    reference = run_scheduled(op, x, ws[0], fmt, n, k, {}, torch.empty_like(out), scratch).clone()
    stream = torch.cuda.Stream(device)
    rows = []
    for config in candidates(op, fmt, m, n, k, space):
        try:
            got = run_scheduled(op, x, ws[0], fmt, n, k, config, out, scratch).clone()
        except ValueError:
            continue  # legal on paper, refused at this scratch size
        error = float((got - reference).norm() / reference.norm())
        if not error <= tolerance:
            rows.append({"config": config, "rejected": f"relative error {error:.2e}"})
            continue
        with torch.cuda.stream(stream):
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=stream):
                for w in ws:
                    run_scheduled(op, x, w, fmt, n, k, config, out, scratch, stream=stream)
            graph.replay()
            samples = []
            for _ in range(repeats):
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record(stream)
                graph.replay()
                e1.record(stream)
                stream.synchronize()
                samples.append(e0.elapsed_time(e1) * 1e3 / copies)
        rows.append({"config": config, "us": statistics.median(samples), "error": error})
    timed = [r for r in rows if "us" in r]
    best = min(timed, key=lambda r: r["us"])
    return {"op": op, "format": fmt.name, "m": m, "n": n, "k": k, "best": best["config"], "us": best["us"],
            "default_us": timed[0]["us"], "rows": rows}


class Profile:
    """Searched schedules per shape, as a JSON file; ``apply`` records them in the library
    (the reference's ``ScheduleProfile``)."""

    def __init__(self, entries=None):
        self.entries = list(entries or [])

    def add(self, result: dict) -> None:
        self.entries = [e for e in self.entries if (e["op"], e["format"], e["m"], e["n"], e["k"]) !=
                        (result["op"], result["format"], result["m"], result["n"], result["k"])]
        self.entries.append({key: result[key] for key in ("op", "format", "m", "n", "k", "best", "us", "default_us")})

    def save(self, path: str) -> None:
        with open(path, "w") as f:
            json.dump({"version": 1, "entries": self.entries}, f, indent=1, sort_keys=True)

    @classmethod
    def load(cls, path: str) -> "Profile":
        with open(path) as f:
            data = json.load(f)
        if data.get("version") != 1:
            raise ValueError("unknown schedule profile version")
        return cls(data["entries"])

    def apply(self) -> int:
        for e in self.entries:
            record(e["op"], e["format"], e["m"], e["n"], e["k"], e["best"])
        return len(self.entries)


__all__ = ["AXES", "DECODE_SPACE", "PREFILL_SPACE", "Profile", "candidates", "clear", "legal", "projection_space",
           "record", "run_scheduled", "search"]
