"""GPU: the PyTorch extension is a drop-in for the reference module (sampling.cpp:5-9): same names,
positional order, dtypes, in-place mutation and ValueError conditions."""
import pytest
import torch

from helpers import make_logits

pytestmark = pytest.mark.gpu


def test_example_workload_matches_reference(ref):
    """example.py: B=4, V=131072, U[0,1) logits from torch seed 0, temperature 1, top_k -1, top_p 0.5."""
    import rapid_sampling_b200 as rs
    torch.manual_seed(0)
    logits = torch.rand(4, 131072).to(0)
    ours = rs.batch_sampling_temperature_topk_topp(logits, rs.setup_rand(0, 4), 1.0, -1, 0.5)
    theirs = ref.batch_sampling_temperature_topk_topp(logits, ref.setup_rand(0, 4), 1.0, -1, 0.5)
    assert ours.dtype == torch.int32 and ours.shape == (4,) and ours.is_cuda     # sampling.cu:1024
    assert torch.equal(ours, theirs)


def test_repetition_call_positional_and_keyword(ref):
    import rapid_sampling_b200 as rs
    B, V = 8, 65536
    lg = make_logits("normal3", B, V, 3, torch).cuda()
    pen_a, pen_b, pen_r = (torch.zeros(B, V, device="cuda") for _ in range(3))
    st_a, st_b, st_r = rs.setup_rand(5, B), rs.setup_rand(5, B), ref.setup_rand(5, B)
    a = rs.batch_sampling_repetition_temperature_topk_topp(lg, pen_a, st_a, 0.1, 0.1, 0.95, 0.8, 50, 0.9)
    b = rs._load_ext().batch_sampling_repetition_temperature_topk_topp(
        lg, pen_b, st_b, presence_penalty=0.1, repetition_penalty=0.1, penalty_decay=0.95, temperature=0.8, top_k=50,
        top_p=0.9)
    r = ref.batch_sampling_repetition_temperature_topk_topp(lg, pen_r, st_r, 0.1, 0.1, 0.95, 0.8, 50, 0.9)
    assert torch.equal(a, r) and torch.equal(b, r)
    assert torch.equal(pen_a, pen_r) and torch.equal(pen_b, pen_r) and torch.equal(st_a, st_r)


def test_states_are_interchangeable_with_the_reference(ref):
    """A state made by either library continues the same stream in the other (64-byte cuRAND layout)."""
    import rapid_sampling_b200 as rs
    lg = make_logits("normal3", 4, 32768, 8, torch).cuda()
    st_x, st_y = ref.setup_rand(11, 4), rs.setup_rand(11, 4)
    a1 = rs.batch_sampling_temperature_topk_topp(lg, st_x, 0.9, 30, 0.9)       # ours on the reference's state
    b1 = ref.batch_sampling_temperature_topk_topp(lg, st_y, 0.9, 30, 0.9)      # reference on ours
    a2 = ref.batch_sampling_temperature_topk_topp(lg, st_x, 0.9, 30, 0.9)
    b2 = rs.batch_sampling_temperature_topk_topp(lg, st_y, 0.9, 30, 0.9)
    assert torch.equal(a1, b1) and torch.equal(a2, b2) and torch.equal(st_x, st_y)


def test_checkpoint_resume_of_states_and_penalties():
    import rapid_sampling_b200 as rs
    B, V = 4, 16384
    lg = make_logits("normal3", B, V, 12, torch).cuda()

    def run(n, st, pen):
        return [rs.batch_sampling_repetition_temperature_topk_topp(lg, pen, st, 0.2, 0.3, 0.9, 0.8, 20, 0.9).cpu() for _ in range(n)]
    st, pen = rs.setup_rand(1, B), torch.zeros(B, V, device="cuda")
    full = run(6, st, pen)
    st2, pen2 = rs.setup_rand(1, B), torch.zeros(B, V, device="cuda")
    first = run(3, st2, pen2)
    saved = (st2.cpu().clone(), pen2.cpu().clone())          # what torch.save would keep
    rest = run(3, saved[0].cuda(), saved[1].cuda())
    assert all(torch.equal(x, y) for x, y in zip(full, first + rest))


def test_error_conditions_raise_value_error():
    import rapid_sampling_b200 as rs
    st = rs.setup_rand(0, 2)
    ok = torch.zeros(2, 1024, device="cuda")
    with pytest.raises(ValueError, match="float32"):
        rs.batch_sampling_temperature_topk_topp(ok.half(), st, 1.0, -1, 0.5)
    with pytest.raises(ValueError, match="Vocabulary size"):
        rs.batch_sampling_temperature_topk_topp(torch.zeros(2, 1022, device="cuda"), st, 1.0, -1, 0.5)
    with pytest.raises(ValueError, match="Temperature"):
        rs.batch_sampling_temperature_topk_topp(ok, st, 0.0, -1, 0.5)
    with pytest.raises(ValueError, match="Temperature"):
        rs.batch_sampling_temperature_topk_topp(ok, st, 2000.0, -1, 0.5)
    with pytest.raises(ValueError):
        rs.batch_sampling_temperature_topk_topp(torch.zeros(4, 1024, device="cuda"), st, 1.0, -1, 0.5)   # states too small
    with pytest.raises(ValueError):
        rs.setup_rand(0, 0)
    # out-of-range top_k / top_p are remapped, not errors (sampling.cu:1005-1010)
    out = rs.batch_sampling_temperature_topk_topp(ok, st, 1.0, 10 ** 9, 7.0)
    assert out.shape == (2,)


def test_call_is_capturable_in_a_cuda_graph():
    """A decode loop may record the call once and replay it: no allocation, synchronisation or host read-back
    happens inside the call once its workspace for the stream exists (the reference allocates per call,
    sampling.cu:488, :498).  Replays advance states and penalties exactly like eager calls."""
    import rapid_sampling_b200 as rs
    for B, V, rep in [(8, 32768, True), (160, 32768, False), (2, 262144, False)]:
        lg = make_logits("normal3", B, V, 21, torch).cuda()
        st_e, st_g = rs.setup_rand(9, B), rs.setup_rand(9, B)
        pen_e, pen_g = torch.zeros(B, V, device="cuda"), torch.zeros(B, V, device="cuda")

        def call(st, pen):
            if rep:
                return rs.batch_sampling_repetition_temperature_topk_topp(lg, pen, st, 0.1, 0.2, 0.9, 0.8, 40, 0.9)
            return rs.batch_sampling_temperature_topk_topp(lg, st, 0.8, 40, 0.9)
        eager = [call(st_e, pen_e).clone() for _ in range(3)]
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):      # first call on the capture stream: creates its workspace
            call(rs.setup_rand(1, B), torch.zeros(B, V, device="cuda"))
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            out = call(st_g, pen_g)
        for want in eager:
            graph.replay()
            torch.cuda.synchronize()
            assert torch.equal(out, want)
        assert torch.equal(st_g, st_e) and torch.equal(pen_g, pen_e)
