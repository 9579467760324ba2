"""The GGUF container reader, against files written by the third-party ``gguf`` package (the format's own
Python writer): directory, metadata, alignment and the raw bytes must come back unchanged, and the blocks
read from the file must dequantise (oracle) to what ``gguf.quants.dequantize`` gives for the same bytes."""

import numpy as np
import pytest

from oracle import gguf_oracle as oracle
from tensor_b200.gguf_file import GgufError, GgufFile

gguf = pytest.importorskip("gguf")

TYPES = {"q4_0": gguf.GGMLQuantizationType.Q4_0, "q8_0": gguf.GGMLQuantizationType.Q8_0,
         "q4_k": gguf.GGMLQuantizationType.Q4_K, "q6_k": gguf.GGMLQuantizationType.Q6_K}


def _write(path, tensors, alignment=None):
    w = gguf.GGUFWriter(path, "llama")
    w.add_uint32("llama.block_count", 2)
    w.add_string("general.name", "fixture")
    if alignment:
        w.add_custom_alignment(alignment)  # writes general.alignment and pads the data with it
    for name, array, raw_dtype in tensors:
        w.add_tensor(name, array, raw_dtype=raw_dtype)
    w.write_header_to_file()
    w.write_kv_data_to_file()
    w.write_tensors_to_file()
    w.close()


@pytest.mark.parametrize("alignment", [None, 64])
def test_reader_round_trip(tmp_path, alignment):
    path = str(tmp_path / "model.gguf")
    shapes = {"q4_0": (24, 256), "q8_0": (8, 512), "q4_k": (40, 1024), "q6_k": (16, 512)}
    raws = {}
    tensors = []
    for i, (name, (n, k)) in enumerate(shapes.items()):
        raw = oracle.make_weights(name, n, k, seed=i)
        raws[name] = raw
        fmt = oracle.get_format(name)
        tensors.append((f"blk.0.{name}.weight", raw.reshape(n, k // fmt.weights * fmt.nbytes), TYPES[name]))
    norm = np.linspace(0.5, 1.5, 256, dtype=np.float32)
    tensors.append(("blk.0.attn_norm.weight", norm, None))
    _write(path, tensors, alignment)
    with GgufFile(path) as f:
        assert f.version == 3 and f.alignment == (alignment or 32)
        assert f.metadata["general.architecture"] == "llama" and f.metadata["llama.block_count"] == 2
        assert f.metadata["general.name"] == "fixture"
        assert set(f.projections()) == {f"blk.0.{name}.weight" for name in shapes}
        for name, (n, k) in shapes.items():
            t = f.tensors[f"blk.0.{name}.weight"]
            assert t.shape == (n, k) and t.format.name == name
            assert np.array_equal(t.data, raws[name])
            want = gguf.quants.dequantize(raws[name].reshape(n, -1), TYPES[name])
            assert np.array_equal(oracle.dequantize(np.array(t.data), name, n, k), want)
        assert np.array_equal(f.tensors["blk.0.attn_norm.weight"].as_numpy(), norm)
        with pytest.raises(GgufError):
            f.tensors["blk.0.attn_norm.weight"].format


def test_reader_rejects_damaged_files(tmp_path):
    path = str(tmp_path / "bad.gguf")
    with open(path, "wb") as f:
        f.write(b"GGML" + b"\0" * 64)
    with pytest.raises(GgufError):
        GgufFile(path)
    good = str(tmp_path / "good.gguf")
    _write(good, [("w", oracle.make_weights("q4_k", 4, 256, seed=1).reshape(4, 144), TYPES["q4_k"])])
    data = open(good, "rb").read()
    with open(path, "wb") as f:
        f.write(data[:-100])  # tensor data cut short
    with pytest.raises(GgufError):
        GgufFile(path)
    with open(path, "wb") as f:
        f.write(data[:20])  # header cut short
    with pytest.raises(GgufError):
        GgufFile(path)


@pytest.mark.gpu
def test_projection_straight_from_a_file(tmp_path):
    import torch

    import tensor_b200 as tb
    from oracle import c_oracle

    n, k, m = 512, 1024, 2
    raw = oracle.make_weights("q4_k", n, k, seed=3)
    path = str(tmp_path / "model.gguf")
    _write(path, [("blk.0.ffn_down.weight", raw.reshape(n, -1), TYPES["q4_k"])])
    with GgufFile(path) as f:
        t = f.projections()["blk.0.ffn_down.weight"]
        dev = torch.device("cuda", 0)
        w = t.to_device(dev)
        rows, depth = t.shape
        x = oracle.make_activations(m, depth, seed=4, dtype="bf16")
        out = tb.gguf(m, rows, depth, t.format)(torch.from_numpy(x).to(dev).to(torch.bfloat16), w)
    assert oracle.rel_frobenius(out.cpu().numpy(), c_oracle.gemv(x, raw, "q4_k", n, k)) < 1e-3
