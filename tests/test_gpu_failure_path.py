"""GPU: the failure path, exercised without faulting, trapping or hanging anything.

Every on-chip wait of the kernels is bounded; when one gives up the kernel writes RS_ERR_TIMEOUT to the status
word (and its host mirror) and returns normally.  The self-test entry makes exactly that happen in isolation: one
CTA waits a few polls on a barrier that nothing will ever complete, with no copy or remote store in flight.
The context must stay usable afterwards.  (The reference checks nothing after a launch, sampling.cu:500-515.)
"""
import pytest
import torch

from helpers import make_logits

pytestmark = pytest.mark.gpu


def test_bounded_wait_runs_out_and_reports_through_the_status_word(abi):
    L, codes = abi.L, abi.abi
    ws = torch.zeros(L.rs_workspace_bytes(4, 32768), dtype=torch.uint8, device="cuda")
    assert L.rs_device_status(ws.data_ptr(), abi.stream()) == 0
    assert L.rs_selftest_bounded_wait(ws.data_ptr(), 4, abi.stream()) == 0
    assert L.rs_device_status(ws.data_ptr(), abi.stream()) == codes.RS_ERR_TIMEOUT
    assert "gave up" in codes.status_string(codes.RS_ERR_TIMEOUT)
    assert L.rs_clear_status(ws.data_ptr(), abi.stream()) == 0
    assert L.rs_device_status(ws.data_ptr(), abi.stream()) == 0
    # the context is intact: a sampling call on the same workspace runs and leaves the word clear
    B, V = 4, 32768
    lg = make_logits("normal3", B, V, 1, torch).cuda()
    out = torch.empty(B, dtype=torch.int32, device="cuda")
    st = abi.setup_rand(1, B)
    rc = L.rs_sample(lg.data_ptr(), B, 1, V, None, st.data_ptr(), out.data_ptr(), 0.8, 50, 0.9, 0.0, 0.0, 0.0, ws.data_ptr(),
                     ws.numel(), abi.stream())
    assert rc == 0
    assert torch.equal(out, abi.sample(lg, abi.setup_rand(1, B), 0.8, 50, 0.9))
    assert L.rs_device_status(ws.data_ptr(), abi.stream()) == 0
    # refusals of the self-test itself
    assert L.rs_selftest_bounded_wait(None, 4, abi.stream()) == codes.RS_ERR_POINTER
    assert L.rs_selftest_bounded_wait(ws.data_ptr(), 0, abi.stream()) == codes.RS_ERR_LIMIT
    assert L.rs_selftest_bounded_wait(ws.data_ptr(), 1 << 20, abi.stream()) == codes.RS_ERR_LIMIT
    import rapid_sampling_b200 as rs
    rs.device_status()       # the torch binding's host mirror saw the time-out too: consume it here


def test_poll_limit_is_settable(abi):
    prev = abi.L.rs_set_wait_polls(1 << 20)
    assert abi.L.rs_set_wait_polls(0) == 1 << 20          # 0 only queries
    assert abi.L.rs_set_wait_polls(prev) == 1 << 20
    assert abi.L.rs_set_wait_polls(0) == prev


def test_torch_binding_raises_a_device_status_on_the_next_call():
    import rapid_sampling_b200 as rs
    ext = rs._load_ext()
    B, V = 4, 32768
    lg = make_logits("normal3", B, V, 2, torch).cuda()
    st = rs.setup_rand(3, B)
    want = rs.batch_sampling_temperature_topk_topp(lg, st, 0.8, 50, 0.9).clone()
    assert rs.device_status() == 0
    ext.selftest_bounded_wait(4)
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="gave up"):
        rs.batch_sampling_temperature_topk_topp(lg, st, 0.8, 50, 0.9)
    # raised once; the status is consumed and sampling goes on
    again = rs.batch_sampling_temperature_topk_topp(lg, rs.setup_rand(3, B), 0.8, 50, 0.9)
    assert torch.equal(again, want)
    assert rs.device_status() == 0


def test_static_scratch_status_word_is_readable(abi):
    B, V = 4, 32768
    lg = make_logits("normal3", B, V, 3, torch).cuda()
    out = torch.empty(B, dtype=torch.int32, device="cuda")
    st = abi.setup_rand(2, B)
    rc = abi.L.rs_sample_static_scratch(lg.data_ptr(), B, 1, V, None, st.data_ptr(), out.data_ptr(), 0.8, 50, 0.9, 0.0, 0.0, 0.0,
                                        abi.stream())
    assert rc == 0
    assert abi.L.rs_device_status(None, abi.stream()) == 0
    assert torch.equal(out, abi.sample(lg, abi.setup_rand(2, B), 0.8, 50, 0.9))
    # an absurd batch cannot wrap the size check
    assert abi.L.rs_sample_static_scratch(lg.data_ptr(), 1 << 44, 1, 1 << 20, None, st.data_ptr(), out.data_ptr(), 0.8, 50, 0.9,
                                          0.0, 0.0, 0.0, abi.stream()) == abi.abi.RS_ERR_LIMIT
