"""GPU: per-row temperature / top_k / top_p.  Row b of a batched call must equal a ONE-ROW call of the reference's
CUDA kernel with row b's values (same ids, RNG states and penalties, bit for bit); the extra outputs are checked
against the float64 statement of the semantics."""
import numpy as np
import pytest
import torch

from helpers import make_logits

pytestmark = pytest.mark.gpu

# per-row settings cycled over the batch: (temperature, top_k, top_p); values are float32-exact or rounded first
SETTINGS = [(1.0, -1, 0.3), (0.8, 50, 0.9), (1.0, -1, 1.0), (1.3, 1, 1.0), (0.7, 400, 0.5), (1.0, 10, 0.0), (2.0, 0, 0.95),
            (0.5, 200000, 1.5), (1.0, 5, -1.0)]


def row_settings(B):
    t = torch.tensor([SETTINGS[b % len(SETTINGS)][0] for b in range(B)], dtype=torch.float32)
    k = torch.tensor([SETTINGS[b % len(SETTINGS)][1] for b in range(B)], dtype=torch.int32)
    p = torch.tensor([SETTINGS[b % len(SETTINGS)][2] for b in range(B)], dtype=torch.float32)
    return t, k, p


@pytest.mark.parametrize("B,V,kind,rep", [(9, 32768, "normal3", False), (9, 65536, "peaked", True), (200, 32768, "normal3", False),
                                          (170, 16384, "uniform", True), (3, 524288, "normal3", False),
                                          (300, 65536, "peaked", True), (130, 65536, "normal3", True), (330, 50300, "normal3", False)])
def test_rows_equal_one_row_reference_calls(ref, B, V, kind, rep):
    import rapid_sampling_b200 as rs
    lg = make_logits(kind, B, V, 31, torch).cuda()
    t, k, p = row_settings(B)
    st_o, st_r = rs.setup_rand(12, B), ref.setup_rand(12, B)
    pen_o = torch.zeros(B, V, device="cuda") if rep else None
    pen_r = torch.zeros(B, V, device="cuda") if rep else None
    for call in range(2):
        got = rs.batch_sampling_rows(lg, st_o, t.cuda(), k.cuda(), p.cuda(), penalties=pen_o, presence_penalty=0.1,
                                     repetition_penalty=0.2, penalty_decay=0.9)
        want = torch.empty(B, dtype=torch.int32, device="cuda")
        for b in range(B):
            s_b = st_r[b * 64:(b + 1) * 64]
            if rep:
                want[b] = ref.batch_sampling_repetition_temperature_topk_topp(lg[b:b + 1], pen_r[b:b + 1], s_b, 0.1, 0.2, 0.9,
                                                                              float(t[b]), int(k[b]), float(p[b]))[0]
            else:
                want[b] = ref.batch_sampling_temperature_topk_topp(lg[b:b + 1], s_b, float(t[b]), int(k[b]), float(p[b]))[0]
        assert torch.equal(got, want), (call, (got != want).nonzero().flatten().tolist())
        assert torch.equal(st_o, st_r)
        if rep:
            assert torch.equal(pen_o, pen_r)


@pytest.mark.parametrize("B", [12, 160])     # the larger batch runs one CTA per row
def test_rows_bf16_logits_and_neutral_defaults(ref, B):
    import rapid_sampling_b200 as rs
    V = 65536
    lg = make_logits("normal3", B, V, 5, torch).cuda().bfloat16()
    t, k, p = row_settings(B)
    st_o, st_r = rs.setup_rand(3, B), ref.setup_rand(3, B)
    got = rs.batch_sampling_rows(lg, st_o, t.cuda(), k.cuda(), p.cuda())
    lf = lg.float()
    for b in range(B):
        want = ref.batch_sampling_temperature_topk_topp(lf[b:b + 1], st_r[b * 64:(b + 1) * 64], float(t[b]), int(k[b]), float(p[b]))
        assert int(got[b]) == int(want[0])
    # no tensors at all: temperature 1, no top_k, no top_p
    st_a, st_b = rs.setup_rand(4, B), rs.setup_rand(4, B)
    a = rs.batch_sampling_rows(lf, st_a)
    b_ = rs.batch_sampling_temperature_topk_topp(lf, st_b, 1.0, -1, 1.0)
    assert torch.equal(a, b_) and torch.equal(st_a, st_b)


@pytest.mark.parametrize("B", [9, 153])      # the larger batch runs one CTA per row
def test_rows_probability_and_kept_mass(B):
    import rapid_sampling_b200 as rs
    from oracle import cpu_ref
    V = 32768
    lg = make_logits("normal3", B, V, 77, torch)
    t, k, p = row_settings(B)
    ids, prob, kept = rs.batch_sampling_rows(lg.cuda(), rs.setup_rand(1, B), t.cuda(), k.cuda(), p.cuda(), return_prob=True)
    ids, prob, kept = ids.cpu(), prob.cpu().double(), kept.cpu().double()
    for b in range(B):
        d = cpu_ref.distribution(lg[b:b + 1], float(t[b]), int(k[b]), float(p[b]))
        assert abs(float(prob[b]) - float(d["probs"][0, ids[b]])) <= 1e-5 * float(d["probs"][0, ids[b]]) + 1e-12
        want_mass = float(d["weights"][0].sum()) if "weights" in d else None
        if want_mass is not None:
            assert abs(float(kept[b]) - want_mass) <= 2e-5 * max(want_mass, 1e-6), (b, float(kept[b]), want_mass)
        assert 0.0 < float(kept[b]) <= 1.0 + 1e-5


def test_rows_bad_temperature_sets_status_and_spares_other_rows(abi):
    import ctypes as C
    torch.cuda.synchronize()
    B, V = 4, 8192
    lg = make_logits("normal3", B, V, 2, torch).cuda()
    t = torch.tensor([1.0, 0.0, float("nan"), 0.9], device="cuda")
    L = abi.L
    ws = torch.zeros(L.rs_rows_workspace_bytes(B, V), dtype=torch.uint8, device="cuda")
    out = torch.empty(B, dtype=torch.int32, device="cuda")
    st = abi.setup_rand(6, B)
    rc = L.rs_sample_rows(lg.data_ptr(), abi.abi.RS_DTYPE_F32, B, 1, V, None, st.data_ptr(), out.data_ptr(), t.data_ptr(), None, None,
                          0.0, 0.0, 0.0, None, None, ws.data_ptr(), ws.numel(), abi.stream())
    assert rc == 0
    assert L.rs_device_status(ws.data_ptr(), abi.stream()) == abi.abi.RS_ERR_TEMPERATURE
    import rapid_sampling_b200 as rs
    rs.device_status()       # the torch binding's host mirror (if registered) saw it too: consume it here
    # rows 0 and 3 as one-row calls with their own values; rows 1 and 2 ran at temperature 1
    st2 = abi.setup_rand(6, B)
    for b, temp in enumerate([1.0, 1.0, 1.0, float(np.float32(0.9))]):
        one = abi.sample(lg[b:b + 1], st2[b * 64:(b + 1) * 64], temp, -1, 1.0)
        assert int(one[0]) == int(out[b])
    # too small a workspace is refused
    assert L.rs_sample_rows(lg.data_ptr(), 0, B, 1, V, None, st.data_ptr(), out.data_ptr(), t.data_ptr(), None, None, 0.0, 0.0, 0.0,
                            None, None, ws.data_ptr(), 256, abi.stream()) == abi.abi.RS_ERR_WORKSPACE


@pytest.mark.parametrize("B", [12, 300])     # the larger batch runs one CTA per row
def test_rows_probability_is_taken_before_the_penalty_update(B):
    """With penalties, the reported probability of the sampled id must come from the penalties as they were BEFORE
    the call (the same values the softmax ran on), on every call of a chain."""
    import rapid_sampling_b200 as rs
    from oracle import cpu_ref
    V = 32768
    lg = make_logits("peaked", B, V, 13, torch)
    t, k, p = row_settings(B)
    pen = torch.zeros(B, V, device="cuda")
    st = rs.setup_rand(5, B)
    for call in range(4):
        before = pen.cpu().clone()
        ids, prob, kept = rs.batch_sampling_rows(lg.cuda(), st, t.cuda(), k.cuda(), p.cuda(), penalties=pen, presence_penalty=0.5,
                                                 repetition_penalty=0.7, penalty_decay=0.9, return_prob=True)
        ids, prob = ids.cpu(), prob.cpu().double()
        for b in range(B):
            d = cpu_ref.distribution(lg[b:b + 1], float(t[b]), int(k[b]), float(p[b]), penalties=before[b:b + 1])
            want = float(d["probs"][0, ids[b]])
            assert abs(float(prob[b]) - want) <= 1e-5 * want + 1e-12, (call, b, float(prob[b]), want)
