"""Host-side pieces of bench.py that need no GPU: the algorithmic byte count the roofline is computed from, the
configuration keys both arms print, the partition of a timed region into graph replays."""
import importlib.util
import math
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_algorithmic_bytes_of_the_headline_layer(bench):
    c = math.ceil(bench.K_IN / 256) // 8 * 8
    assert (bench.K_IN, bench.N_OUT, bench.BITS, bench.GROUP, c) == (4096, 11008, 4, 128, 16)
    # qweight 2040 x 11008, scales 32 x 11008 fp16, cherries 16 x 11008 fp16 + 16 indices, x and y of one row
    assert bench.algorithmic_bytes(4096, 11008, 4, 128, 1, 16) == 2040 * 11008 + 32 * 11008 * 2 + 16 * 11008 * 2 + 32 + 8192 + 22016
    assert bench.algorithmic_bytes(4096, 11008, 4, 128, 1, 16) == 23_543_328
    assert bench.algorithmic_bytes(28672, 8192, 3, 128, 1, 112) == 93_315_296


def test_both_arms_name_the_same_workload(bench):
    cfg = bench.workload_config(path="x")
    assert {"workload", "bits", "group", "K", "N", "batch"} <= set(cfg)
    assert cfg["workload"] == bench.WORKLOAD and cfg["batch"] == 1 and cfg["path"] == "x"


def test_region_partition_covers_exactly_the_requested_steps(bench):
    class FakeGraph:
        def __init__(self):
            self.n = 0

    launches = []

    class FakeRegion(bench.Region):
        def _capture(self, launch, idx):
            g = FakeGraph()
            g.n = len(list(idx))
            return g

    for steps, ncopies in [(20, 17), (20, 34), (20000, 17), (5, 5), (1, 17)]:
        r = FakeRegion(None, None, lambda i: launches.append(i), steps, ncopies)
        total = r.rounds * (r.g_round.n if r.g_round else 0) + (r.g_rem.n if r.g_rem else 0)
        assert total == steps, (steps, ncopies)
        assert "CUDA graphs only" in r.what


def test_median_and_thread_count(bench):
    assert bench.median([3.0, 1.0, 2.0]) == 2.0
    assert 1 <= bench.host_threads() <= 32
