"""Schedules: legality without a GPU, the profile file, and (on a GPU) a measured search behind the
correctness gate.  Mirrors how the reference tests its schedule spaces and search
(tests/compiler/test_search.py, tests/compiler/test_cuda_schedules.py in the reference checkout)."""

import numpy as np
import pytest

import tensor_b200 as tb
from tensor_b200 import schedule


def test_spaces_and_legality_need_no_gpu():
    assert set(schedule.projection_space("decode", 1)["gemv"]) == {"k_splits", "ctas_per_sm", "convert_ahead"}
    assert schedule.projection_space("decode", 1)["gemv"]["convert_ahead"] == (2,)
    assert schedule.projection_space("prefill")["gemm"]["gemm_shape"] == (11, 12, 22)
    with pytest.raises(ValueError):
        schedule.projection_space("training")
    shape = ("q4_k", 1, 18944, 3584)
    assert schedule.legal("gemv", *shape, {})
    assert schedule.legal("gemv", *shape, {"k_splits": 2, "ctas_per_sm": 2})
    assert not schedule.legal("gemv", *shape, {"k_splits": 15})            # 14 super-blocks: an empty K range
    assert not schedule.legal("gemv", *shape, {"k_splits": 2}, scratch_bytes=0)  # a split needs scratch
    assert not schedule.legal("gemv", *shape, {"ctas_per_sm": 3})
    assert not schedule.legal("gemv", "q4_k", 4, 18944, 3584, {"convert_ahead": 1}, scratch_bytes=0)
    assert not schedule.legal("gemv", "q6_k", 1, 4096, 4096, {})           # the mma.sync pipeline is Q4_K only
    assert schedule.legal("gemm", "q6_k", 512, 12288, 4096, {"gemm_shape": 22})
    assert not schedule.legal("gemm", "q6_k", 512, 12288, 4096, {"gemm_shape": 33})
    configs = list(schedule.candidates("gemv", "q4_k", 4, 3584, 18944))
    assert configs[0] == {} and all(schedule.legal("gemv", "q4_k", 4, 3584, 18944, c) for c in configs)
    assert {"k_splits": 8, "ctas_per_sm": 1, "convert_ahead": 1} in configs


def test_recorded_schedule_becomes_the_default_plan():
    shape = ("q4_k", 1, 3584, 16384)
    schedule.clear()
    derived = tb.gemv_plan(*shape)
    try:
        schedule.record("gemv", *shape, {"k_splits": 4, "ctas_per_sm": 1})
        pinned = tb.gemv_plan(*shape)
        assert pinned["k_splits"] == 4 and pinned["ctas_per_sm"] == 1
        assert tb.gemv_plan("q4_k", 1, 3584, 16384 + 256) != pinned  # only that exact shape
    finally:
        schedule.clear()
    assert tb.gemv_plan(*shape) == derived


def test_derived_plan_counts_the_latency_of_a_split():
    """Batch 1 at K = 4096: a K split balances the SMs on paper but its extra phase costs about 2 us, more than
    the whole unsplit launch takes (measured 4.4 against 11.6 us at 3072 rows): the derived plan must not split.
    Where K is long and the rows are few, it still does."""
    schedule.clear()
    try:
        for n in (1024, 1536, 2048, 3072, 4096, 6144):
            assert tb.gemv_plan("q4_k", 1, n, 4096)["k_splits"] == 1, n
        assert tb.gemv_plan("q4_k", 1, 3584, 18944)["k_splits"] > 1
        assert tb.gemv_plan("q4_k", 16, 3584, 18944)["k_splits"] > 1
    finally:
        from tensor_b200 import _native

        _native._apply_shipped_schedules()
    assert tb.gemv_plan("q4_k", 1, 3584, 18944)["k_splits"] == 3  # the shipped schedule for the benchmark's down projection


def test_profile_round_trip(tmp_path):
    profile = schedule.Profile()
    profile.add({"op": "gemv", "format": "q4_k", "m": 1, "n": 3584, "k": 18944, "best": {"k_splits": 8, "ctas_per_sm": 2},
                 "us": 14.0, "default_us": 15.0, "rows": []})
    profile.add({"op": "gemv", "format": "q4_k", "m": 1, "n": 3584, "k": 18944, "best": {"k_splits": 7, "ctas_per_sm": 2},
                 "us": 13.5, "default_us": 15.0, "rows": []})  # replaces the first
    path = str(tmp_path / "profile.json")
    profile.save(path)
    schedule.clear()
    loaded = schedule.Profile.load(path)
    assert len(loaded.entries) == 1 and loaded.entries[0]["best"]["k_splits"] == 7
    try:
        assert loaded.apply() == 1
        assert tb.gemv_plan("q4_k", 1, 3584, 18944)["k_splits"] == 7
    finally:
        schedule.clear()
        from tensor_b200 import _native

        _native._apply_shipped_schedules()  # what loading the library had recorded


@pytest.mark.gpu
@pytest.mark.parametrize("op,name,m,n,k", [("gemv", "q4_k", 4, 1024, 8192), ("gemm", "q4_k", 300, 512, 1024)])
def test_measured_search_behind_the_parity_gate(op, name, m, n, k):
    import torch

    from oracle import c_oracle
    from oracle import gguf_oracle as oracle

    result = schedule.search(op, name, m, n, k, repeats=3, l2_bytes=8 << 20)
    timed = [r for r in result["rows"] if "us" in r]
    assert len(timed) >= 2 and result["us"] <= result["default_us"] + 1e-9
    assert all(r["error"] <= 1e-3 for r in timed)
    # the winner, recorded, is what the ordinary entry point runs; its result matches the oracle
    try:
        schedule.record(op, name, m, n, k, result["best"])
        dev = torch.device("cuda", 0)
        raw = oracle.make_weights(name, n, k, seed=1)
        x = oracle.make_activations(m, k, seed=2, dtype="bf16")
        xd, wd = torch.from_numpy(x).to(dev).to(torch.bfloat16), torch.from_numpy(raw).to(dev)
        out = torch.full((m, n), float("nan"), device=dev)
        tb.gguf(m, n, k, name, op=op).launch(xd, wd, out)
        want = c_oracle.gemv(x, raw, name, n, k) if op == "gemv" else c_oracle.gemm(x, raw, name, n, k, operand="bf16")
        assert oracle.rel_frobenius(out.cpu().numpy(), want) < 1e-3
    finally:
        schedule.clear()
    assert tb.device_status() == 0
