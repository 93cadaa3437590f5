"""CPU: the bench's workloads and sweep grid are the ones the reference and its sweep define."""
import importlib.util
import os

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _bench():
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    m = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(m)
    return m


def test_full_sweep_grid_is_the_reference_grid():
    g = _bench().SWEEP_GRIDS["full"]           # bench.py:32-35 of the reference
    assert sorted(g["B"]) == [1, 2, 4, 8, 16, 32, 64, 128, 256, 512]
    assert sorted(g["V"]) == [256, 32768, 50304, 65536, 100256, 131072, 151936, 262144]
    assert g["p"] == [0.1, 0.3, 0.7, 0.9, 1] and g["k"] == [-1, 1, 10, 100, 1000, 10000]
    assert len(g["B"]) * len(g["V"]) * len(g["p"]) * len(g["k"]) * 5 == 12000


def test_workloads_have_the_headline_shapes():
    b = _bench()
    shapes = {n: (b.workload(n)["B"], b.workload(n)["T"], b.workload(n)["V"]) for n in ("C1", "C2", "C3", "C4", "C5")}
    assert shapes == {"C1": (4, 1, 131072), "C2": (1, 1, 262144), "C3": (64, 1, 151936), "C4": (256, 1, 65536),
                      "C5": (32, 4, 1048576)}
    assert b.workload("C4")["rep"] and not b.workload("C2")["rep"]
