"""``.tbin`` packaging of the sm_100a kernels for the unchanged reference runtime.

CPU: artifacts are built with nvcc (no GPU needed), their envelope is checked member by member and,
where the reference checkout is available (set TENSOR_REFERENCE), validated by the reference's own
``read_artifact`` / capability check.  GPU: the artifact is consumed the way the reference's provider
does (driver API only) and compared with the oracle."""

import hashlib
import json
import os
import sys
import zipfile

import numpy as np
import pytest

from tensor_b200 import tbin

# the reference checkout: TENSOR_REFERENCE, else a sibling directory `reference` next to this repository
REFERENCE = os.environ.get("TENSOR_REFERENCE") or os.path.normpath(
    os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "..", "reference"))


def _check_envelope(path):
    with zipfile.ZipFile(path) as z:
        names = set(z.namelist())
        manifest = json.loads(z.read("manifest.json"))
        assert names == {"manifest.json", *manifest["files"]}
        for name, digest in manifest["files"].items():
            assert hashlib.sha256(z.read(name)).hexdigest() == digest
        assert z.read("kernel.cubin").startswith(b"\x7fELF")
        assert "nodes" in json.loads(z.read("kernel.tirx.json"))
    assert manifest["format"] == "tensor.module" and manifest["format_version"] == 3
    assert manifest["target"] == "sm_100" and manifest["kind"] == "cubin" and manifest["provider"] == "cuda"
    assert manifest["workspace"] == {"bytes": 0, "alignment": 1}
    assert [a["name"] for a in manifest["arguments"]][:3] == ["x", "w", "out"]
    assert manifest["outputs"] == ["out"]
    block = manifest["launch"]["block"]
    assert block[0] * block[1] * block[2] <= 1024
    return manifest


@pytest.mark.parametrize("m,n,k", [(1, 256, 512), (4, 4096, 4096), (1, 3584, 18944)])
def test_gemv_artifact_envelope(tmp_path, m, n, k):
    path = str(tmp_path / "gemv.tbin")
    tbin.build_gemv_tbin(path, "q4_k", m, n, k)
    manifest = _check_envelope(path)
    split = len(manifest["arguments"]) == 4
    if split:
        assert manifest["arguments"][3]["name"] == "scratch" and manifest["arguments"][3]["dtype"] == "uint8"
    for name, spec in manifest.get("cuda_tensor_maps", {}).items():
        size = {4: 8, 9: 2}[spec["data_type"]]
        total = size
        for d in spec["global_dims"]:
            total *= d
        arg = next(a for a in manifest["arguments"] if a["name"] == name)
        elems = 1
        for d in arg["shape"]:
            elems *= d
        assert total == elems * {"uint8": 1, "bfloat16": 2}[arg["dtype"]]  # map covers the whole buffer
        assert all(1 <= b <= 256 for b in spec["box_dims"])


def test_gemm_artifact_envelope_and_reference_reader(tmp_path):
    path = str(tmp_path / "gemm.tbin")
    tbin.build_gemm_tbin(path, "q6_k", 256, 256, 1024)
    manifest = _check_envelope(path)
    assert manifest["cuda_tensor_maps"]["x"]["box_dims"] == [64, 256]
    if not os.path.isdir(os.path.join(REFERENCE, "src", "tensor")):
        pytest.skip("reference checkout not available")
    sys.path.insert(0, os.path.join(REFERENCE, "src"))
    try:
        from tensor.artifacts.format import read_artifact
        from tensor.runtime.abi import check_requirement

        read, files = read_artifact(path)
        check_requirement(read["runtime_abi"])
        assert read["entrypoint"] == "kernel_kernel" and files["kernel.cubin"].startswith(b"\x7fELF")
        gemv_path = str(tmp_path / "gemv.tbin")
        tbin.build_gemv_tbin(gemv_path, "q4_k", 1, 3584, 18944)
        read_artifact(gemv_path)
    finally:
        sys.path.remove(os.path.join(REFERENCE, "src"))


@pytest.mark.gpu
@pytest.mark.parametrize("m,n,k", [(1, 2048, 3584), (1, 3584, 18944), (4, 1024, 4096), (16, 512, 2048)])
def test_gemv_artifact_runs_like_the_provider_would(tmp_path, m, n, k):
    import torch

    from oracle import c_oracle
    from oracle import gguf_oracle as oracle
    from tbin_runner import TbinKernel

    dev = torch.device("cuda", 0)
    torch.cuda.init()
    torch.zeros(1, device=dev)
    path = str(tmp_path / "gemv.tbin")
    manifest = tbin.build_gemv_tbin(path, "q4_k", m, n, k)
    kern = TbinKernel(path)
    raw = oracle.make_weights("q4_k", n, k, seed=1)
    x = oracle.make_activations(m, k, seed=2, dtype="bf16")
    bufs = {"x": torch.from_numpy(x).to(dev).to(torch.bfloat16), "w": torch.from_numpy(raw).to(dev),
            "out": torch.full((m, n), float("nan"), device=dev)}
    if len(manifest["arguments"]) == 4:
        bufs["scratch"] = torch.zeros(manifest["arguments"][3]["shape"][0], dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    for _ in range(2):  # second launch reuses the scratch
        keep = kern.launch(stream, **bufs)
        torch.cuda.synchronize()
        del keep
    got = bufs["out"].cpu().numpy()
    assert np.isfinite(got).all()
    assert oracle.rel_frobenius(got, c_oracle.gemv(x, raw, "q4_k", n, k)) < 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("name", ["q4_k", "q6_k"])
def test_gemm_artifact_runs_like_the_provider_would(tmp_path, name):
    import torch

    from oracle import c_oracle
    from oracle import gguf_oracle as oracle
    from tbin_runner import TbinKernel

    dev = torch.device("cuda", 0)
    torch.zeros(1, device=dev)
    m, n, k = 300, 384, 1024
    path = str(tmp_path / "gemm.tbin")
    tbin.build_gemm_tbin(path, name, m, n, k)
    kern = TbinKernel(path)
    raw = oracle.make_weights(name, n, k, seed=3)
    x = oracle.make_activations(m, k, seed=4, dtype="bf16")
    bufs = {"x": torch.from_numpy(x).to(dev).to(torch.bfloat16), "w": torch.from_numpy(raw).to(dev),
            "out": torch.full((m, n), float("nan"), device=dev)}
    keep = kern.launch(torch.cuda.current_stream().cuda_stream, **bufs)
    torch.cuda.synchronize()
    del keep
    got = bufs["out"].cpu().numpy()
    assert np.isfinite(got).all()
    assert oracle.rel_frobenius(got, c_oracle.gemm(x, raw, name, n, k, operand="bf16")) < 1e-3


@pytest.mark.gpu
@pytest.mark.parametrize("name,m,n,k", [("q4_k", 1, 512, 1024), ("q6_k", 1, 300, 512), ("q8_0", 3, 256, 512), ("q4_0", 9, 64, 256)])
def test_f32_signature_artifact_runs_like_the_provider_would(tmp_path, name, m, n, k):
    """``kernel_kernel(const float* x, const uint8_t* w, float* out)`` over flat buffers, the signature the
    reference's own kernels for this path present (no declared outputs: the caller passes all three)."""
    import torch

    from oracle import c_oracle
    from oracle import gguf_oracle as oracle
    from tbin_runner import TbinKernel

    dev = torch.device("cuda", 0)
    torch.zeros(1, device=dev)
    path = str(tmp_path / "f32.tbin")
    manifest = tbin.build_gemv_f32_tbin(path, name, m, n, k)
    assert manifest["outputs"] == []
    kern = TbinKernel(path)
    raw = oracle.make_weights(name, n, k, seed=5)
    x = oracle.make_activations(m, k, seed=6, dtype="f32")
    bufs = {"x": torch.from_numpy(x).to(dev).reshape(-1), "w": torch.from_numpy(raw).to(dev),
            "out": torch.full((m * n,), float("nan"), device=dev)}
    keep = kern.launch(torch.cuda.current_stream().cuda_stream, **bufs)
    torch.cuda.synchronize()
    del keep
    got = bufs["out"].cpu().numpy().reshape(m, n)
    assert np.isfinite(got).all()
    assert oracle.rel_frobenius(got, c_oracle.gemv(x, raw, name, n, k)) < 1e-3
