"""Host-side logic that needs no GPU: chunking of the host-buffer pipeline, the benchmark's workload description and
its DRAM-traffic scaling, the per-iteration tables' size limit."""
import argparse
import importlib.util
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("cnl_bench", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_chunk_ranges_cover_the_batch_in_order():
    from customnetworklayers_b200.host_pipeline import _chunks
    assert _chunks(8, 4) == [(0, 4), (4, 8)]
    assert _chunks(5, 2) == [(0, 2), (2, 4), (4, 5)]
    assert _chunks(8, [1, 3]) == [(0, 1), (1, 4), (4, 7), (7, 8)]          # the last size repeats
    assert _chunks(3, 8) == [(0, 3)]
    for bad in (0, [], [2, 0]):
        with pytest.raises(ValueError):
            _chunks(4, bad)


def test_both_bench_arms_describe_the_same_workload():
    b = _bench()
    for world in (1, 2, 4, 8):
        args = argparse.Namespace(workload="cfg1", scaling=None)
        cfg = b.workload_config(args, world)
        assert b.resolve_scaling(args) == "strong"
        assert cfg["global_batch"] == 8 and cfg["parallelism"] == f"dp{world}"
        assert "batch 8" in cfg["workload"] and "2x384x1280" in cfg["workload"] and "100 iterations" in cfg["workload"]
        weak = b.workload_config(argparse.Namespace(workload="cfg1", scaling="weak"), world)
        assert weak["global_batch"] == 8 * world


def test_traffic_figure_scales_with_images_and_iterations():
    b = _bench()
    t8 = b.ncu_traffic_per_launch(8, 2, 384, 1280, 99, 100)
    t1 = b.ncu_traffic_per_launch(1, 2, 384, 1280, 99, 100)
    assert abs(t8["reverse"] / t1["reverse"] - 8.0) < 1e-9 and abs(t8["forward"] / t1["forward"] - 8.0) < 1e-9
    # one time block (four iterations) of the batch of 8: what the capture showed
    blk = b.ncu_traffic_per_launch(8, 2, 384, 1280, 4, 4)
    assert 500e6 < blk["reverse"] < 600e6 and 300e6 < blk["forward"] < 360e6
    assert b.ncu_traffic_per_launch(8, 2, 100, 100, 4, 4) is None
    fwd_b, rev_b = b.algorithmic_bytes_per_pixel_iter(2)
    assert (fwd_b, rev_b) == (60, 108)
