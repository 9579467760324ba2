"""Peer-mapped device memory for the GPUs of one box (one process per GPU).

An N-sharded projection finishes with every rank holding the full ``[m, N]`` output.  Instead of a
collective after the kernel, the GEMV stores its columns into every rank's output directly
(``tb200_gguf_gemv_sharded``) and a small barrier kernel (``tb200_peer_barrier``) orders the
stores before the readers.  Both need each rank's buffers mapped into every other process: a
:class:`PeerArena` is one torch allocation per rank, exported with CUDA IPC, opened once by every
peer, and carved up identically on every rank (a bump allocator), so that a buffer is named by
its offset and ``ptrs(offset)`` lists its address on every rank.

``torch.distributed`` carries the handles (``all_gather_object``); the default process group or a
sub-group of ranks on the same box may be used.  The reference has no multi-GPU path; its
per-device sessions (src/tensor/providers/cuda/device.py:30-39) are what one rank corresponds to.
"""

from __future__ import annotations

import ctypes

import torch

from . import abi
from ._native import lib, raise_for_status

SIGNAL_PAD_BYTES = 256
_ALIGN = 256


class BumpAllocator:
    """Offsets inside an arena; every rank issues the same requests in the same order and so
    obtains the same offsets."""

    def __init__(self, capacity: int, align: int = _ALIGN):
        self.capacity, self.align, self.used = int(capacity), int(align), 0

    def take(self, nbytes: int) -> int:
        if nbytes < 0:
            raise ValueError("negative size")
        start = -(-self.used // self.align) * self.align
        if start + nbytes > self.capacity:
            raise MemoryError(f"peer arena exhausted: {nbytes} bytes wanted at offset {start} of {self.capacity}")
        self.used = start + nbytes
        return start


def export_handle(t: torch.Tensor):
    """(64-byte IPC handle, byte offset of ``t`` inside its allocation)."""
    handle = ctypes.create_string_buffer(64)
    offset = ctypes.c_int64(0)
    error = abi.TensorErrorV1()
    with torch.cuda.device(t.device):
        status = lib().tb200_peer_export(t.data_ptr(), handle, ctypes.byref(offset), ctypes.byref(error))
    raise_for_status(status, error)
    return handle.raw, int(offset.value)


def open_handle(handle: bytes, device: torch.device) -> int:
    base = ctypes.c_void_p(0)
    error = abi.TensorErrorV1()
    with torch.cuda.device(device):
        status = lib().tb200_peer_open(handle, ctypes.byref(base), ctypes.byref(error))
    raise_for_status(status, error)
    return int(base.value)


def close_handle(base: int, device: torch.device) -> None:
    error = abi.TensorErrorV1()
    with torch.cuda.device(device):
        status = lib().tb200_peer_close(base, ctypes.byref(error))
    raise_for_status(status, error)


class PeerArena:
    """``capacity`` bytes on every rank of ``group``, each rank's mapped into all the others."""

    def __init__(self, capacity: int, device: torch.device, rank: int, world: int, group=None):
        import torch.distributed as dist

        self.device, self.rank, self.world, self.group = torch.device(device), rank, world, group
        self.local = torch.zeros(int(capacity), dtype=torch.uint8, device=self.device)
        self._alloc = BumpAllocator(capacity)
        self.bases = [0] * world
        self._opened = []
        self.bases[rank] = self.local.data_ptr()
        if world > 1:
            torch.cuda.synchronize(self.device)  # the zero fill has landed before anyone maps it
            mine = export_handle(self.local)
            everyone = [None] * world
            dist.all_gather_object(everyone, mine, group=group)
            for r, (handle, offset) in enumerate(everyone):
                if r == rank:
                    continue
                base = open_handle(handle, self.device)
                self._opened.append(base)
                self.bases[r] = base + offset
            dist.barrier(group=group)  # every rank has mapped every arena: stores may begin
        self.pad_offset = self._alloc.take(SIGNAL_PAD_BYTES)

    def take(self, nbytes: int) -> int:
        """Offset of a new ``nbytes`` region (the same on every rank)."""
        return self._alloc.take(nbytes)

    def view(self, offset: int, shape, dtype=torch.float32) -> torch.Tensor:
        """This rank's copy of the region at ``offset`` as a tensor."""
        count = 1
        for s in shape:
            count *= int(s)
        nbytes = count * torch.empty((), dtype=dtype).element_size()
        return self.local[offset:offset + nbytes].view(dtype).view(*shape)

    def ptrs(self, offset: int, own_first: bool = True):
        """Addresses of the region on every rank, as seen from this process."""
        order = list(range(self.world))
        if own_first:
            order = [self.rank] + [r for r in order if r != self.rank]
        return [self.bases[r] + offset for r in order]

    def pad_ptrs(self):
        """Signal pads in rank order (what ``tb200_peer_barrier`` takes)."""
        return [self.bases[r] + self.pad_offset for r in range(self.world)]

    def close(self) -> None:
        for base in self._opened:
            close_handle(base, self.device)
        self._opened = []


__all__ = ["BumpAllocator", "PeerArena", "SIGNAL_PAD_BYTES", "close_handle", "export_handle", "open_handle"]
