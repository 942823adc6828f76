"""The benchmark's synthetic batch is a function of the global row index alone: whatever the number of
ranks, the ranks' slices put together are the same 65536 rows (so the throughput lines of 1, 2, 4 and 8
GPUs train on identical data and their final loss and parameter checksums can be compared)."""
import importlib.util
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    return module


def test_rank_slices_are_the_rows_of_one_global_batch():
    bench = load_bench()
    total = 8192
    whole_x, whole_t = bench.synthetic_rows(0, total)
    assert whole_x.shape == (total, bench.DIMS[0]) and whole_x.dtype == np.float32 and whole_t.dtype == np.int32
    assert 0.0 <= whole_x.min() and whole_x.max() < 1.0 and set(np.unique(whole_t)) <= set(range(bench.DIMS[-1]))
    for world in (2, 4, 8):
        rows = total // world
        parts = [bench.synthetic_rows(rank * rows, rows) for rank in range(world)]
        assert np.array_equal(np.concatenate([p[0] for p in parts]), whole_x)
        assert np.array_equal(np.concatenate([p[1] for p in parts]), whole_t)
    # another seed is another batch (the inference record uses its own)
    assert not np.array_equal(bench.synthetic_rows(0, 1024, seed=4321)[0], whole_x[:1024])


def test_traffic_interpolation_hits_both_captures():
    bench = load_bench()
    for rows, value in bench.NCU_GEMM_TRAFFIC.items():
        assert abs(bench.interpolate_rows(bench.NCU_GEMM_TRAFFIC, rows) - value) <= 1e-6 * value
    middle = bench.interpolate_rows(bench.NCU_GEMM_TRAFFIC, 32768)
    assert min(bench.NCU_GEMM_TRAFFIC.values()) < middle < max(bench.NCU_GEMM_TRAFFIC.values())
