"""GPU: the entry point that allocates nothing (rs_sample_static_scratch) against rs_sample.

Meant for hosts that cannot call cudaMalloc when they sample (all HBM already owned by their own
arena, or a decode loop that may not enter a synchronising allocator): its scratch rows sit in a fixed
array inside the library.  The test makes two calls in a row -- the second one finds the first one's
leftovers in that shared array -- and expects exactly the ids, RNG states and penalties of the
workspace-based entry point (integer results: the tolerance is equality).  Collected last on purpose.
"""
import pytest
import torch

from helpers import make_logits

pytestmark = pytest.mark.gpu


def _static(abi, lg, st, temp, k, p, pen=None):
    B, V = lg.shape
    out = torch.empty(B, dtype=torch.int32, device="cuda")
    rc = abi.L.rs_sample_static_scratch(lg.data_ptr(), B, 1, V, pen.data_ptr() if pen is not None else None,
                                        st.data_ptr(), out.data_ptr(), temp, k, p, 0.1, 0.1, 0.95, abi.stream())
    assert rc == 0, abi.abi.status_string(rc) + " " + abi.L.rs_last_cuda_error().decode()
    return out


@pytest.mark.parametrize("kind,B,V,temp,k,p,rep", [
    ("normal3", 3, 1048576, 1.0, -1, 0.95, False),     # rows that need global scratch in rs_sample too
    ("peaked", 16, 151936, 0.8, 50, 0.9, True),        # rs_sample keeps these on chip: cross-variant check
    ("uniform", 8, 32768, 1.0, -1, 0.5, False),
])
def test_two_calls_in_a_row_match_rs_sample(abi, kind, B, V, temp, k, p, rep):
    lg = make_logits(kind, B, V, 5, torch).cuda()
    st_a, st_b = abi.setup_rand(21, B), abi.setup_rand(21, B)
    pen_a = torch.zeros(B, V, device="cuda") if rep else None
    pen_b = torch.zeros(B, V, device="cuda") if rep else None
    for call in range(2):
        want = abi.sample(lg, st_a, temp, k, p, penalties=pen_a, presence=0.1, repetition=0.1, decay=0.95)
        got = _static(abi, lg, st_b, temp, k, p, pen_b)
        torch.cuda.synchronize()
        assert torch.equal(got, want), call
        assert torch.equal(st_a, st_b)
        if rep:
            assert torch.equal(pen_a, pen_b)


def test_sizes_beyond_the_fixed_array_are_rejected(abi):
    B, V = 5, 1048576                                   # 5 Mi floats > 4 Mi
    lg = torch.zeros(1, 4, device="cuda")
    out = torch.empty(B, dtype=torch.int32, device="cuda")
    st = abi.setup_rand(0, B)
    rc = abi.L.rs_sample_static_scratch(lg.data_ptr(), B, 1, V, None, st.data_ptr(), out.data_ptr(), 1.0, -1, 0.5,
                                        0.0, 0.0, 0.0, abi.stream())
    assert rc == abi.abi.RS_ERR_LIMIT
    assert "beyond" in abi.abi.status_string(rc)
