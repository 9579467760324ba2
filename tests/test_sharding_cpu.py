"""N-sharding of a GGUF weight across ranks, checked on CPU with two gloo ranks: every rank runs the
oracle GEMV on its own rows, the outputs are all-gathered with the same routine the GPU path uses,
and the result must equal the unsharded product bit for bit (each output column is produced by
exactly one rank with the same K order)."""

import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import gguf_oracle as oracle
from tensor_b200.projection import all_gather_columns, shard_rows, shard_weight_bytes


def test_shard_rows_and_bytes():
    assert shard_rows(18944, 3, 8) == (7104, 9472)
    assert shard_rows(16, 0, 1) == (0, 16)
    with pytest.raises(ValueError):
        shard_rows(10, 0, 3)
    with pytest.raises(ValueError):
        shard_rows(16, 2, 2)
    n, k = 32, 512
    raw = torch.from_numpy(oracle.make_weights("q6_k", n, k, seed=1))
    parts = [shard_weight_bytes(raw, "q6_k", n, k, r, 4) for r in range(4)]
    assert all(p.numel() == n // 4 * 2 * 210 for p in parts)
    assert torch.equal(torch.cat(parts), raw)
    for r, p in enumerate(parts):  # a shard is a valid weight of n/4 rows: same decode as the full rows
        full = oracle.dequantize(raw.numpy(), "q6_k", n, k)
        part = oracle.dequantize(p.numpy(), "q6_k", n // 4, k)
        assert np.array_equal(part, full[r * 8:(r + 1) * 8])
    with pytest.raises(ValueError):
        shard_weight_bytes(raw[:-1], "q6_k", n, k, 0, 4)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank_main(rank, world, port, fmt, m, n, k, result_path):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        raw = torch.from_numpy(oracle.make_weights(fmt, n, k, seed=5))
        x = oracle.make_activations(m, k, seed=6, dtype="bf16")
        mine = shard_weight_bytes(raw, fmt, n, k, rank, world).numpy()
        n_local = n // world
        out_local = torch.from_numpy(oracle.gemv_ref(x, mine, fmt, n_local, k))
        gathered = torch.empty((world, m, n_local), dtype=torch.float32)
        out = torch.empty((m, n), dtype=torch.float32)
        all_gather_columns(out_local, gathered, out)
        # column block r of the assembled output is exactly what rank r computed on its rows
        want = torch.from_numpy(oracle.gemv_ref(x, raw.numpy(), fmt, n, k))
        blocks_ok = torch.equal(out[:, rank * n_local:(rank + 1) * n_local], out_local)
        # the assembled output equals the unsharded product (same decode, same K order per column)
        close = bool(np.allclose(out.numpy(), want.numpy(), rtol=1e-5, atol=1e-5))
        every = [None] * world
        dist.all_gather_object(every, (blocks_ok, close, out.numpy().tobytes()))
        if rank == 0:
            same_everywhere = all(e[2] == every[0][2] for e in every)
            np.save(result_path, np.array([all(e[0] for e in every), all(e[1] for e in every), same_everywhere]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("fmt,m", [("q4_k", 1), ("q6_k", 4), ("q8_0", 16)])
def test_two_rank_gloo_sharded_gemv(tmp_path, fmt, m):
    world, n, k = 2, 48, 512
    path = str(tmp_path / "result.npy")
    mp.spawn(_rank_main, args=(world, _free_port(), fmt, m, n, k, path), nprocs=world, join=True)
    blocks_ok, close, same = np.load(path)
    assert blocks_ok and close and same
