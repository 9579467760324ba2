"""Reader for GGUF container files: the on-disk source of the raw blocks this library multiplies.

The reference plans GGUF model loading as a benchmark of its own
(research/plans/v1-benchmarks.md:287-358) and leaves the reader to the AKAS package; its showcase
feeds the kernels synthetic blocks.  A real deployment starts from a ``.gguf`` file, so this module
reads one: header, metadata key/values, tensor directory, and the tensor data as zero-copy views.  The
format is the public GGUF v3 layout (little endian): magic ``GGUF``, uint32 version, uint64 tensor
count, uint64 metadata count, the metadata pairs, the tensor infos (name, rank, dimensions innermost
first, GGML type id, offset into the data section), padding to ``general.alignment`` (default 32),
then the data.  A quantised weight ``[N, K]`` is stored with dimensions ``(K, N)`` and N * K / block *
bytes raw bytes, rows contiguous: exactly the buffer ``tb200_gguf_gemv`` / ``tb200_gguf_gemm`` take.
"""

from __future__ import annotations

import mmap
import struct

import numpy as np

from .formats import get_format

MAGIC = b"GGUF"
# GGML type ids of unquantised tensors (bytes per element); quantised ids come from tensor_b200.formats
PLAIN_TYPES = {0: ("float32", 4), 1: ("float16", 2), 30: ("bfloat16", 2), 24: ("int8", 1), 26: ("int32", 4)}
QUANTISED = (2, 8, 12, 14)
_SCALARS = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<?", 10: "<Q", 11: "<q", 12: "<d"}


class GgufError(ValueError):
    """The file is not a GGUF container this reader understands."""


class _Cursor:
    def __init__(self, data):
        self.data, self.pos = data, 0

    def take(self, fmt):
        size = struct.calcsize(fmt)
        if self.pos + size > len(self.data):
            raise GgufError("truncated file")
        (value,) = struct.unpack_from(fmt, self.data, self.pos)
        self.pos += size
        return value

    def string(self):
        length = self.take("<Q")
        if self.pos + length > len(self.data):
            raise GgufError("truncated string")
        raw = bytes(self.data[self.pos:self.pos + length])
        self.pos += length
        return raw.decode("utf-8", "replace")

    def value(self, kind):
        if kind in _SCALARS:
            return self.take(_SCALARS[kind])
        if kind == 8:
            return self.string()
        if kind == 9:
            item, count = self.take("<I"), self.take("<Q")
            if count > (1 << 28):
                raise GgufError("implausible array length")
            return [self.value(item) for _ in range(count)]
        raise GgufError(f"unknown metadata value type {kind}")


class GgufTensor:
    """One entry of the tensor directory.  ``shape`` is row-major (outermost first), i.e. ``(N, K)`` for
    a weight; ``data`` is a read-only uint8 view of the tensor's bytes inside the mapped file."""

    def __init__(self, name, shape, type_id, data):
        self.name, self.shape, self.type_id, self.data = name, tuple(shape), type_id, data

    @property
    def quantised(self) -> bool:
        return self.type_id in QUANTISED

    @property
    def format(self):
        if not self.quantised:
            raise GgufError(f"{self.name} is not in a block format this library multiplies (GGML type {self.type_id})")
        return get_format(self.type_id)

    def as_numpy(self) -> np.ndarray:
        """Unquantised tensors as an array of their own dtype (bfloat16 as uint16 bit patterns)."""
        if self.type_id not in PLAIN_TYPES:
            raise GgufError(f"{self.name} is quantised; use .data (raw blocks)")
        dtype = PLAIN_TYPES[self.type_id][0]
        return self.data.view(np.uint16 if dtype == "bfloat16" else dtype).reshape(self.shape)

    def to_device(self, device):
        """The raw blocks as a uint8 CUDA tensor (what the kernels take); a projection is then
        ``tensor_b200.gguf(m, N, K, tensor.format)`` with ``N, K = tensor.shape``."""
        import torch

        return torch.from_numpy(np.array(self.data, copy=True)).to(device)


class GgufFile:
    """``GgufFile(path)`` maps the file; ``.metadata`` is the key/value dictionary, ``.tensors`` the
    directory by name.  Keep the object alive while views of its data are in use; ``close()`` unmaps."""

    def __init__(self, path: str):
        self._file = open(path, "rb")
        try:
            self._map = mmap.mmap(self._file.fileno(), 0, access=mmap.ACCESS_READ)
        except ValueError:
            self._file.close()
            raise GgufError("empty file") from None
        data = memoryview(self._map)
        cur = _Cursor(data)
        if bytes(data[:4]) != MAGIC:
            self.close()
            raise GgufError("not a GGUF file (bad magic)")
        cur.pos = 4
        self.version = cur.take("<I")
        if self.version not in (2, 3):
            self.close()
            raise GgufError(f"unsupported GGUF version {self.version}")
        tensor_count, kv_count = cur.take("<Q"), cur.take("<Q")
        if tensor_count > (1 << 24) or kv_count > (1 << 24):
            self.close()
            raise GgufError("implausible header counts")
        self.metadata = {}
        for _ in range(kv_count):
            key = cur.string()
            self.metadata[key] = cur.value(cur.take("<I"))
        infos = []
        for _ in range(tensor_count):
            name = cur.string()
            rank = cur.take("<I")
            if rank > 4:
                self.close()
                raise GgufError(f"{name}: rank {rank}")
            dims = [cur.take("<Q") for _ in range(rank)]  # innermost first
            infos.append((name, dims, cur.take("<I"), cur.take("<Q")))
        self.alignment = int(self.metadata.get("general.alignment", 32))
        if self.alignment < 1 or self.alignment & (self.alignment - 1):
            self.close()
            raise GgufError("alignment is not a power of two")
        self.data_offset = -(-cur.pos // self.alignment) * self.alignment
        whole = np.frombuffer(data, dtype=np.uint8)
        self.tensors = {}
        for name, dims, type_id, offset in infos:
            count = 1
            for d in dims:
                count *= d
            if type_id in QUANTISED:
                fmt = get_format(type_id)
                if not dims or dims[0] % fmt.weights:
                    self.close()
                    raise GgufError(f"{name}: innermost dimension {dims[:1]} is not a whole number of {fmt.name} blocks")
                nbytes = count // fmt.weights * fmt.nbytes
            elif type_id in PLAIN_TYPES:
                nbytes = count * PLAIN_TYPES[type_id][1]
            else:
                nbytes = None  # a block format this library does not multiply: listed, data not sliced
            start = self.data_offset + offset
            if offset % self.alignment or (nbytes is not None and start + nbytes > len(whole)):
                self.close()
                raise GgufError(f"{name}: data range outside the file or misaligned")
            view = whole[start:start + nbytes] if nbytes is not None else whole[start:start]
            self.tensors[name] = GgufTensor(name, list(reversed(dims)), type_id, view)

    def projections(self):
        """The tensors the kernels can multiply directly: rank-2 weights in Q4_0 / Q8_0 / Q4_K / Q6_K."""
        return {name: t for name, t in self.tensors.items() if t.quantised and len(t.shape) == 2}

    def close(self) -> None:
        self.tensors = {}
        try:
            self._map.close()
        except (AttributeError, BufferError):
            pass  # views still alive keep the mapping; it goes with them
        self._file.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


__all__ = ["GgufError", "GgufFile", "GgufTensor"]
