"""Host-side logic of bench.py that needs no GPU: the work it divides by, the workload description
both arms must share, the scaled traffic figure, the row samples of the parity check."""

import importlib.util
import os

import pytest

from conftest import ROOT

spec = importlib.util.spec_from_file_location("tpa_bench", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)


def test_algorithmic_flops_of_the_five_configurations():
    """F = 4 B h d P with P = T (T + 1) / 2 causal, T^2 otherwise (two contractions, 2 FLOP per MAC)."""
    want = {"c0": 2.689597e8, "c1": 5.498900e11, "c2": 8.796361e12, "c3": 1.407386e14, "c4": 1.374390e11}
    for name, f in want.items():
        dt, b, t, h, d, rq, rk, causal = bench.WORKLOADS[name]
        assert bench.flops(b, t, h, d, causal) == pytest.approx(f, rel=1e-6), name


def test_both_arms_describe_the_workload_identically():
    for world in (1, 2, 8):
        name = "c2" if world == 1 else "c3"
        a = bench.config_for(name, world, "reference_local")
        b = bench.config_for(name, world, "reference_local")
        assert a == b and a["workload"] == name and set(a) == {"workload", "shape", "parallelism", "l2"}
        assert ("ring" in a["parallelism"]) == (world > 1)


def test_traffic_scales_with_sequence_length_and_only_for_the_captured_shape():
    assert bench.ncu_traffic("c2", 8192) == bench.NCU_T8192_BYTES
    assert bench.ncu_traffic("c2", 32768) == 4 * bench.NCU_T8192_BYTES
    assert bench.ncu_traffic("c2@T16384", 16384) == 2 * bench.NCU_T8192_BYTES
    assert bench.ncu_traffic("c1", 4096) is None and bench.ncu_traffic("c3", 131072) is None


def test_parity_rows_cover_both_ends_and_are_reproducible():
    rows = bench._sample_rows(32768, 64, 7)
    assert rows.tolist() == sorted(set(rows.tolist())) and len(rows) >= 64
    assert {0, 1, 2, 3, 32764, 32765, 32766, 32767} <= set(rows.tolist())
    assert bench._sample_rows(32768, 64, 7).tolist() == rows.tolist()
    assert bench._bounds("bf16") == (2e-2, 5e-3) and bench._bounds("f32") == (1e-5, 1e-5)


def test_host_threads_are_shared_among_ranks():
    import torch

    before = torch.get_num_threads()
    try:
        all_ = bench.host_threads()
        assert bench.host_threads(share=max(1, all_)) == 1
        assert bench.host_threads(share=2) == max(1, all_ // 2)
    finally:
        torch.set_num_threads(before)
