"""Compiler-free consumer of a ``.tbin``, written against the CUDA driver API the way the reference's
provider consumes one (``src/tensor/providers/cuda/device.py:211-229,359-386``): verify the payload
hashes, ``cuModuleLoadData``, ``cuModuleGetFunction(entrypoint)``, opt in to the dynamic shared memory,
encode ``cuda_tensor_maps`` with ``cuTensorMapEncodeTiled``, and ``cuLaunchKernel(grid, block, shared,
stream, params)`` with one parameter per ``abi`` entry (the buffer's device address, or the 128-byte
tensor map).  Test infrastructure: the reference checkout is not present on the GPU box."""

import ctypes as c
import hashlib
import json
import zipfile


class TbinKernel:
    def __init__(self, path):
        self.cuda = c.CDLL("libcuda.so.1")
        with zipfile.ZipFile(path) as z:
            self.manifest = json.loads(z.read("manifest.json"))
            files = {n: z.read(n) for n in self.manifest["files"]}
        for name, data in files.items():
            assert hashlib.sha256(data).hexdigest() == self.manifest["files"][name], name
        self.image = files["kernel.cubin"]
        self.module = c.c_void_p()
        self._check(self.cuda.cuModuleLoadData(c.byref(self.module), self.image), "cuModuleLoadData")
        self.function = c.c_void_p()
        self._check(self.cuda.cuModuleGetFunction(c.byref(self.function), self.module,
                                                  self.manifest["entrypoint"].encode()), "cuModuleGetFunction")
        shared = self.manifest["launch"]["shared_memory_bytes"]
        if shared > 48 * 1024:
            self._check(self.cuda.cuFuncSetAttribute(self.function, 8, shared), "cuFuncSetAttribute")

    def _check(self, status, what):
        if status:
            raise RuntimeError(f"{what} failed with CUDA error {status}")

    def _tensor_map(self, spec, pointer):
        rank = len(spec["global_dims"])
        dims = (c.c_uint64 * rank)(*spec["global_dims"])
        strides = (c.c_uint64 * max(1, rank - 1))(*spec["global_strides"])
        box = (c.c_uint32 * rank)(*spec["box_dims"])
        elem = (c.c_uint32 * rank)(*spec["element_strides"])
        storage = c.create_string_buffer(128 + 63)
        address = (c.addressof(storage) + 63) & ~63
        fn = self.cuda.cuTensorMapEncodeTiled
        fn.argtypes = [c.c_void_p, c.c_int, c.c_uint32, c.c_void_p, c.POINTER(c.c_uint64), c.POINTER(c.c_uint64),
                       c.POINTER(c.c_uint32), c.POINTER(c.c_uint32), c.c_int, c.c_int, c.c_int, c.c_int]
        self._check(fn(address, spec["data_type"], rank, pointer, dims, strides, box, elem, spec["interleave"],
                       spec["swizzle"], spec["l2_promotion"], spec["oob_fill"]), "cuTensorMapEncodeTiled")
        return storage, address

    def launch(self, stream_handle, **buffers):
        """``buffers``: name -> torch CUDA tensor, one per manifest argument."""
        keep, params = [], []
        maps = self.manifest.get("cuda_tensor_maps", {})
        for item in self.manifest["abi"]:
            t = buffers[item["name"]]
            assert t.data_ptr() % 64 == 0
            if item["name"] in maps:
                storage, address = self._tensor_map(maps[item["name"]], t.data_ptr())
                keep.append(storage)
                params.append(address)
            else:
                slot = c.c_uint64(t.data_ptr())
                keep.append(slot)
                params.append(c.addressof(slot))
        array = (c.c_void_p * len(params))(*params)
        g, b = self.manifest["launch"]["grid"], self.manifest["launch"]["block"]
        fn = self.cuda.cuLaunchKernel
        fn.argtypes = [c.c_void_p] + [c.c_uint] * 6 + [c.c_uint, c.c_void_p, c.c_void_p, c.c_void_p]
        self._check(fn(self.function, g[0], g[1], g[2], b[0], b[1], b[2],
                       self.manifest["launch"]["shared_memory_bytes"], c.c_void_p(stream_handle), array, None),
                    "cuLaunchKernel")
        return keep
