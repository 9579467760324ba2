"""Build libtensor_b200_gguf.so in-tree with nvcc for sm_100a.

    python -m tensor_b200.build [--force]

Each .cu under csrc/ is compiled to an object in parallel and linked into
``tensor_b200/lib/libtensor_b200_gguf.so`` (static cudart, no libcuda link dependency: driver
entry points are resolved at run time).  ``-Xptxas -v`` output is kept in ``lib/ptxas.log``.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB_DIR = os.path.join(HERE, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libtensor_b200_gguf.so")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xptxas", "-v",
          "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found; the CUDA extension cannot be built")


def _host_compiler() -> list[str]:
    # An environment CC may point at a compiler nvcc does not accept; prefer the system g++.
    return ["-ccbin", "/usr/bin/g++"] if os.path.exists("/usr/bin/g++") else []


def sources() -> list[str]:
    return sorted(f for f in os.listdir(CSRC) if f.endswith(".cu"))


def _fingerprint() -> str:
    h = hashlib.sha256()
    for name in sorted(os.listdir(CSRC)) + ["../../include/tensor_b200_gguf.h"]:
        path = os.path.join(CSRC, name)
        if os.path.isfile(path):
            h.update(name.encode())
            with open(path, "rb") as f:
                h.update(f.read())
    h.update(" ".join(ARCH_FLAGS + COMMON).encode())
    return h.hexdigest()


def _compile(name: str) -> tuple[str, str]:
    obj = os.path.join(LIB_DIR, name[:-3] + ".o")
    cmd = [_nvcc(), *ARCH_FLAGS, *COMMON, *_host_compiler(), "-I", INCLUDE, "-c",
           os.path.join(CSRC, name), "-o", obj]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode:
        raise RuntimeError(f"nvcc failed for {name}:\n{proc.stdout}\n{proc.stderr}")
    return obj, proc.stderr


def build(force: bool = False, verbose: bool = False) -> str:
    if os.environ.get("TB200_GEMV_TRACE"):
        # diagnostic build: the GEMV kernels record a per-CTA timeline and print it at process exit
        for flag in ("-DTB200_GEMV_TRACE", "-DTB200_TC_TRACE"):
            if flag not in COMMON:
                COMMON.append(flag)
    os.makedirs(LIB_DIR, exist_ok=True)
    stamp = os.path.join(LIB_DIR, "build.sha256")
    fp = _fingerprint()
    if not force and os.path.exists(LIB_PATH) and os.path.exists(stamp):
        with open(stamp) as f:
            if f.read().strip() == fp:
                return LIB_PATH
    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 1)) as pool:
        results = list(pool.map(_compile, sources()))
    with open(os.path.join(LIB_DIR, "ptxas.log"), "w") as log:
        for _, text in results:
            log.write(text)
    objs = [o for o, _ in results]
    cmd = [_nvcc(), *ARCH_FLAGS, "-shared", *_host_compiler(), "-o", LIB_PATH, *objs]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode:
        raise RuntimeError(f"link failed:\n{proc.stdout}\n{proc.stderr}")
    for o in objs:
        os.remove(o)
    with open(stamp, "w") as f:
        f.write(fp)
    if verbose:
        print("built", LIB_PATH)
    return LIB_PATH


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
