"""GPU: a cut through the reference's own parameter sweep (B x V x top_p x top_k x its five logit distributions,
bench.py:32-72 of the reference), 5 calls per point, ids compared with the reference's CUDA kernel on the same
logits and states.  Every id must be identical."""
import argparse
import importlib.util
import os

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_small_sweep_ids_identical_to_reference_kernel(ref, tmp_path):
    spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    line = bench.run_sweep(argparse.Namespace(sweep="small", sweep_out=str(tmp_path / "sweep.json")))
    g = bench.SWEEP_GRIDS["small"]
    assert line["combinations"] == len(g["B"]) * len(g["V"]) * len(g["p"]) * len(g["k"]) * 5
    assert line["ids_differ"] == 0
