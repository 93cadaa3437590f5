"""GPU parity tests, all through the C ABI.

Bar: sampled ids, RNG states and penalty tensors are BIT-IDENTICAL to the reference's own CUDA
extension (oracle/_ref, compiled unmodified) on the same seeded inputs and the same RNG states;
given the kernel's own fp32 probabilities the order-faithful C oracle reproduces threshold,
compensation factor, lane pick and id bit for bit; the kept set equals the float64 closed form
except at fp32-level ties; sampled frequencies pass a chi-square test over 10^6 draws.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from helpers import kept_set_flips_ok, make_logits
from oracle import c_oracle as co
from oracle import cpu_ref

pytestmark = pytest.mark.gpu

# (kind, B, V, temperature, top_k, top_p, seed)
MATRIX = [
    ("uniform", 4, 131072, 1.0, -1, 0.5, 0),       # example.py workload
    ("normal3", 1, 262144, 1.0, -1, 0.3, 1),       # headline shape
    ("peaked", 64, 151936, 0.8, 50, 0.9, 2),       # batched decode, ragged lanes
    ("normal3", 4, 1048576, 1.0, -1, 0.95, 4),     # largest V: global scratch-row variant
    ("uniform4", 3, 262144, 1.0, -1, 0.3, 5),      # the setting of the one published number
    ("uniform", 4, 4, 1.0, -1, 0.5, 6),            # smallest V
    ("equal", 4, 256, 1.0, -1, 0.5, 7),            # all ties: search never starts
    ("equal", 4, 8192, 0.7, 100, 0.25, 8),
    ("coarse", 16, 4096, 0.9, 7, 0.6, 9),          # heavy ties at the boundary, fractional comp
    ("coarse", 8, 50304, 1.0, -1, 0.7, 10),
    ("special", 8, 50304, 1.3, 100, 0.9, 11),      # NaN / +-Inf entries
    ("uniform", 8, 100256, 1.0, -1, 1.0, 12),      # no filter at all
    ("uniform", 8, 100256, 1.0, 1, 0.0, 13),       # top_p == 0 -> greedy
    ("normal3", 8, 65536, 0.001, -1, 0.9, 14),     # extreme temperatures
    ("normal3", 8, 65536, 1000.0, 1000, 0.9, 15),
    ("normal3", 8, 32768, 1.0, 10, 1.0, 16),       # temperature 1 with top-k: general kernel
    ("normal3", 8, 32768, 1.0, -1, 0.999999, 17),
    ("peaked", 300, 8192, 0.8, 50, 0.9, 18),       # more rows than fit at once
    ("normal3", 2, 524288, 0.9, 200, 0.95, 19),    # needs the 16-CTA cluster to stay on chip
    ("uniform", 100, 32768, 1.0, -1, 0.9, 20),     # flat rows, streaming variant: the lowered bound takes in the whole row
    ("uniform4", 90, 16384, 1.0, -1, 0.1, 21),     # long candidate lists that shrink as the bracket rises
    ("coarse", 80, 32768, 1.0, -1, 0.7, 22),       # the same with heavy ties
    ("normal3", 130, 65536, 1.0, -1, 0.9, 23),     # one CTA per row: the kept set (~4 % of the row) overflows the lanes' shared-memory lists
    ("normal3", 20, 151936, 1.0, -1, 0.7, 24),     # the same with a ragged last stripe
    ("uniform4", 160, 32768, 1.0, -1, 0.3, 25),    # ... and lists that spill widely
]


def _ref_call(ref, lg, st, temp, k, p, pen=None):
    if pen is None:
        return ref.batch_sampling_temperature_topk_topp(lg, st, temp, k, p)
    return ref.batch_sampling_repetition_temperature_topk_topp(lg, pen, st, 0.1, 0.1, 0.95, temp, k, p)


def test_setup_rand_bytes_equal_reference_and_oracle(abi, ref):
    for seed, B in [(0, 4), (1234567890123, 8), (2 ** 63 + 5, 300), (-1 & (2 ** 64 - 1), 2)]:
        ours = abi.setup_rand(seed, B)
        theirs = ref.setup_rand(seed - 2 ** 64 if seed >= 2 ** 63 else seed, B)
        assert torch.equal(ours, theirs)
        assert np.array_equal(ours.cpu().numpy(), co.setup_rand(seed, B))
    shard = abi.setup_rand(77, 5, first_row=10)
    assert np.array_equal(shard.cpu().numpy(), co.setup_rand(77, 15)[10 * 64:])


@pytest.mark.parametrize("kind,B,V,temp,k,p,seed", MATRIX)
def test_ids_and_states_bit_identical_to_reference_kernel(abi, ref, kind, B, V, temp, k, p, seed):
    abi.set_cluster(0)
    lg = make_logits(kind, B, V, seed, torch).cuda()
    try:
        for mode in (0, 1, 2, 3, 4, 5, 6):         # automatic / whole-row search only / streaming / on-chip / one CTA per row / 4 and 0 with the exact search only
            abi.set_path(mode)
            s_ref, s_our = ref.setup_rand(seed, B), abi.setup_rand(seed, B)
            for call in range(3):                  # consecutive calls advance the states
                want = _ref_call(ref, lg, s_ref, temp, k, p)
                got = abi.sample(lg, s_our, temp, k, p)
                assert torch.equal(got, want), (mode, call, (got != want).nonzero()[:5])
                assert torch.equal(s_our, s_ref)
    finally:
        abi.set_path(0)
    assert abi.device_status() == 0


def test_both_search_strategies_are_exercised(abi):
    """Peaked / top-k rows must resolve on the candidate list; flat rows (kept set = a third of the row)
    cannot and must fall back to the whole-row search.  Same ids either way."""
    cases = [("peaked", 16, 151936, 0.8, 50, 0.9, 0), ("normal3", 16, 65536, 0.8, 50, 0.9, 0),
             ("normal3", 4, 262144, 1.0, -1, 0.3, 0), ("uniform", 4, 131072, 1.0, -1, 0.5, 1),
             ("uniform", 4, 32768, 1.0, -1, 1.0, 1), ("equal", 4, 8192, 0.7, 100, 0.25, 1)]
    for kind, B, V, temp, k, p, want_path in cases:
        lg = make_logits(kind, B, V, 3, torch).cuda()
        out_a, _, tr = abi.sample(lg, abi.setup_rand(3, B), temp, k, p, debug=True)
        assert all(t.path == want_path for t in tr), (kind, [t.path for t in tr])
        if want_path == 0:
            assert all(0 < t.ncand < V // 8 for t in tr), (kind, [t.ncand for t in tr])
        try:
            abi.set_path(1)
            out_b, _, tr_b = abi.sample(lg, abi.setup_rand(3, B), temp, k, p, debug=True)
        finally:
            abi.set_path(0)
        assert torch.equal(out_a, out_b)
        for x, y in zip(tr, tr_b):
            assert y.path == 1 and x.left == y.left and x.rounds == y.rounds and x.idxt == y.idxt
            assert x.sum_p == y.sum_p and x.comp == y.comp and x.seqk == y.seqk and x.sgtk == y.sgtk


def test_row_cta_integer_search_and_its_hand_over_to_exact_sums(abi, ref):
    """The one-CTA-per-row kernel first runs the search in one warp on exact integer masses and keeps the result only
    if no mass came within the fp32 rounding of the reference's sums of top_p.  Ordinary rows must be settled that
    way; with top_p set to the very mass of a prefix of the sorted row the integer search must stand back and the
    block-wide search on fp32 sums must give the reference's ids, trace for trace."""
    B, V = 6, 32768
    lg = make_logits("peaked", B, V, 3, torch).cuda()
    outcome = lambda t: (t.t_ns[0] >> 16) & 0xf
    try:
        abi.set_path(4)
        _, probs, tr = abi.sample(lg, abi.setup_rand(3, B), 0.8, 50, 0.9, debug=True)
        assert all(outcome(t) == 1 and t.path == 0 for t in tr), [(outcome(t), t.path) for t in tr]
        top = torch.sort(probs[0], descending=True).values[:3].cpu()
        stood_back = 0
        for top_p in (float(top[0]), float(top[0] + top[1]), float((top[0] + top[1]) + top[2])):
            res = {}
            for mode in (4, 5):
                abi.set_path(mode)
                s_ref, s_our = ref.setup_rand(5, B), abi.setup_rand(5, B)
                want = ref.batch_sampling_temperature_topk_topp(lg, s_ref, 0.8, 50, top_p)
                got, _, tr = abi.sample(lg, s_our, 0.8, 50, top_p, debug=True)
                assert torch.equal(got, want) and torch.equal(s_our, s_ref), (top_p, mode)
                res[mode] = [(t.left, t.rounds, t.sum_p, t.comp, t.seqk, t.sgtk, t.idxt) for t in tr]
                if mode == 4:
                    stood_back += int(outcome(tr[0]) == 0 and tr[0].path == 0)
            assert res[4] == res[5], top_p
        assert stood_back >= 2
    finally:
        abi.set_path(0)


def test_back_to_back_calls_under_dependent_launch_equal_the_reference_chain(abi, ref):
    """Small grids are launched with programmatic stream serialization: call n+1 may be set up while call n runs and
    must not touch states or penalties before call n is complete.  A chain of 60 calls, each depending on the states
    and penalties the previous one wrote, queued without any host synchronisation, must end bit-equal to the reference's
    chain -- with the early launch on, and with ordinary launches."""
    B, V = 3, 65536
    lgs = [make_logits("normal3", B, V, 40 + i, torch).cuda() for i in range(4)]
    L = abi.L
    prev = L.rs_set_dependent_launch(-1)
    try:
        for on in (1, 0):
            L.rs_set_dependent_launch(on)
            pen_ref, pen_our = torch.zeros(B, V, device="cuda"), torch.zeros(B, V, device="cuda")
            s_ref, s_our = ref.setup_rand(9, B), abi.setup_rand(9, B)
            want, got = [], []
            for i in range(60):
                want.append(ref.batch_sampling_repetition_temperature_topk_topp(lgs[i % 4], pen_ref, s_ref, 0.1, 0.1, 0.95, 0.8, 50, 0.9))
            for i in range(60):
                got.append(abi.sample(lgs[i % 4], s_our, 0.8, 50, 0.9, penalties=pen_our, presence=0.1, repetition=0.1, decay=0.95))
            torch.cuda.synchronize()
            assert torch.equal(torch.stack(got), torch.stack(want)), on
            assert torch.equal(pen_our, pen_ref) and torch.equal(s_our, s_ref), on
    finally:
        L.rs_set_dependent_launch(prev)


@pytest.mark.parametrize("cluster", [1, 2, 4, 8, 16])
def test_every_cluster_width_gives_the_same_ids(abi, ref, cluster):
    try:
        for kind, V, temp, k, p in [("uniform", 32768, 1.0, -1, 0.5), ("normal3", 32768, 0.7, 40, 0.8),
                                    ("coarse", 20480, 0.9, 7, 0.6), ("peaked", 36868, 0.8, 50, 0.9)]:
            B = 24
            lg = make_logits(kind, B, V, 31, torch).cuda()
            s_ref, s_our = ref.setup_rand(3, B), abi.setup_rand(3, B)
            pen_ref, pen_our = torch.zeros(B, V, device="cuda"), torch.zeros(B, V, device="cuda")
            abi.set_cluster(cluster)
            for _ in range(2):
                assert torch.equal(abi.sample(lg, s_our, temp, k, p), _ref_call(ref, lg, s_ref, temp, k, p))
                got = abi.sample(lg, s_our, temp, k, p, penalties=pen_our, presence=0.1, repetition=0.1, decay=0.95)
                assert torch.equal(got, _ref_call(ref, lg, s_ref, temp, k, p, pen_ref))
            assert torch.equal(pen_our, pen_ref) and torch.equal(s_our, s_ref)
    finally:
        abi.set_cluster(0)


def test_global_scratch_variant_matches_on_chip_variant(abi, ref):
    """Forcing a cluster width whose shared memory cannot hold the row selects the scratch-row variant."""
    B, V = 6, 262144
    lg = make_logits("normal3", B, V, 41, torch).cuda()
    s_a, s_b = abi.setup_rand(9, B), abi.setup_rand(9, B)
    a = abi.sample(lg, s_a, 0.9, 100, 0.9)
    try:
        abi.set_cluster(1)           # 1 MiB row cannot fit one CTA: needs the B*V scratch
        need = 256 + B * V * 4
        ws = torch.zeros(need, dtype=torch.uint8, device="cuda")
        out = torch.empty(B, dtype=torch.int32, device="cuda")
        rc = abi.L.rs_sample(lg.data_ptr(), B, 1, V, None, s_b.data_ptr(), out.data_ptr(), 0.9, 100, 0.9, 0.0, 0.0, 0.0,
                             ws.data_ptr(), 256, abi.stream())
        assert rc == abi.abi.RS_ERR_WORKSPACE
        rc = abi.L.rs_sample(lg.data_ptr(), B, 1, V, None, s_b.data_ptr(), out.data_ptr(), 0.9, 100, 0.9, 0.0, 0.0, 0.0,
                             ws.data_ptr(), need, abi.stream())
        assert rc == 0
    finally:
        abi.set_cluster(0)
    assert torch.equal(a, out) and torch.equal(s_a, s_b)


def test_btv_reads_only_the_last_position(abi):
    B, T, V = 5, 4, 65536
    lg = make_logits("normal3", B * T, V, 51, torch).reshape(B, T, V).cuda()
    s3, s2 = abi.setup_rand(4, B), abi.setup_rand(4, B)
    a = abi.sample(lg, s3, 0.8, 50, 0.9)
    b = abi.sample(lg[:, -1, :].contiguous(), s2, 0.8, 50, 0.9)
    assert torch.equal(a, b) and torch.equal(s3, s2)
    v1 = abi.sample(lg[0, -1].contiguous(), abi.setup_rand(4, 1), 0.8, 50, 0.9)      # (V,) input
    assert v1.shape == (1,) and int(v1[0]) == int(a[0])


def test_repetition_chain_128_steps_bit_identical(abi, ref):
    """The repetition workload at reduced batch: 128 chained calls, logits regenerated per step,
    penalties fed back.  Ids must match at every step, so the final penalty tensors are equal bit for bit
    (the stated tolerance is 1e-6 relative; equality is stronger)."""
    B, V = 32, 65536
    pen_ref, pen_our = torch.zeros(B, V, device="cuda"), torch.zeros(B, V, device="cuda")
    s_ref, s_our = ref.setup_rand(3, B), abi.setup_rand(3, B)
    for step in range(128):
        lg = (torch.randn(B, V, generator=torch.Generator().manual_seed(3 + step)) * 2.5).cuda()
        want = _ref_call(ref, lg, s_ref, 0.8, 50, 0.9, pen_ref)
        got = abi.sample(lg, s_our, 0.8, 50, 0.9, penalties=pen_our, presence=0.1, repetition=0.1, decay=0.95)
        assert torch.equal(got, want), step
    assert torch.equal(pen_our, pen_ref) and torch.equal(s_our, s_ref)
    assert int((pen_our != 0).sum()) > B


def test_penalties_with_masks_and_existing_values(abi, ref):
    """-inf / +inf penalties act as masks (sampling.cu:177); non-zero entries take the repetition branch."""
    B, V = 16, 32768
    lg = make_logits("normal3", B, V, 61, torch).cuda()
    base = torch.zeros(B, V)
    g = torch.Generator().manual_seed(5)
    base[:, torch.randperm(V, generator=g)[:2000]] = float("inf")       # masked out
    base[:, torch.randperm(V, generator=g)[:50]] = float("-inf")        # forced candidates
    base[:, torch.randperm(V, generator=g)[:500]] = 0.3
    pen_ref, pen_our = base.clone().cuda(), base.clone().cuda()
    s_ref, s_our = ref.setup_rand(6, B), abi.setup_rand(6, B)
    for _ in range(4):
        want = _ref_call(ref, lg, s_ref, 0.9, 40, 0.95, pen_ref)
        got = abi.sample(lg, s_our, 0.9, 40, 0.95, penalties=pen_our, presence=0.1, repetition=0.1, decay=0.95)
        assert torch.equal(got, want)
    assert torch.equal(pen_our.view(torch.int32), pen_ref.view(torch.int32))


def test_long_candidate_lists_are_searched_in_place(abi):
    """Flat rows in the streaming variant: the lowered bound admits (nearly) the whole row to the candidate buffer, which is
    then searched like a slab, shrinking as the bracket rises.  Same trace as the whole-row search."""
    B, V = 100, 32768
    lg = make_logits("uniform", B, V, 3, torch).cuda()
    out_a, _, tr = abi.sample(lg, abi.setup_rand(3, B), 1.0, -1, 0.9, debug=True)
    assert all(t.path == 0 and t.ncand > 4096 for t in tr), [(t.path, t.ncand) for t in tr][:4]
    try:
        abi.set_path(1)
        out_b, _, tr_b = abi.sample(lg, abi.setup_rand(3, B), 1.0, -1, 0.9, debug=True)
    finally:
        abi.set_path(0)
    assert torch.equal(out_a, out_b)
    for x, y in zip(tr, tr_b):
        assert y.path == 1 and x.left == y.left and x.rounds == y.rounds and x.idxt == y.idxt
        assert x.sum_p == y.sum_p and x.comp == y.comp and x.seqk == y.seqk and x.sgtk == y.sgtk


@pytest.mark.parametrize("kind,B,V,temp,k,p,seed", [m for m in MATRIX if m[2] <= 262144 and m[1] <= 64])
def test_oracle_reproduces_kernel_bit_for_bit_given_its_probabilities(abi, kind, B, V, temp, k, p, seed):
    """Everything after the softmax is IEEE fp32 add/mul/div/compare in a fixed order, so the CPU oracle,
    fed the kernel's own probabilities and the same RNG state, must land on the same bits."""
    lg = make_logits(kind, B, V, seed, torch)
    st = abi.setup_rand(seed, B)
    st_cpu = st.cpu().numpy().copy()
    out, probs, tr = abi.sample(lg.cuda(), st, temp, k, p, debug=True)
    knd, scale, kk, pp = co.normalise(V, B, 1, temp, k, p)
    probs = probs.cpu().numpy()
    for b in range(min(B, 8)):
        tok, o, _ = co.sample_row(lg[b].numpy(), st_cpu[64 * b:64 * b + 64], knd, scale, kk, pp, probs_in=probs[b])
        g = tr[b]
        assert tok == int(out[b]) == g.token
        for f in ("left", "seqk", "sgtk", "rounds", "idxt", "early_exit"):
            assert getattr(o, f) == getattr(g, f), f
        for f in ("threshold", "comp", "sgtp", "sum_p", "randp", "sum_o", "rand2", "pmin", "pmax"):
            a, c = np.float32(getattr(o, f)), np.float32(getattr(g, f))
            assert a.view(np.uint32) == c.view(np.uint32), (f, a, c)
        assert list(o.rnd) == list(g.rnd)
        # softmax stage: only exp2f differs (hardware approximation vs libm), a few ulp
        own_tok, own, own_probs = co.sample_row(lg[b].numpy(), st_cpu[64 * b:64 * b + 64].copy(), knd, scale, kk, pp,
                                                want_probs=True)
        assert own.maxu == g.maxu
        assert abs(own.denom - g.denom) <= 2e-6 * g.denom
        big = probs[b] > 1e-30
        assert np.all(np.abs(own_probs[big] - probs[b][big]) <= 4e-6 * probs[b][big])
    assert np.array_equal(st.cpu().numpy()[:64], st_cpu[:64])       # oracle advanced its copy the same way


@pytest.mark.parametrize("kind,B,V,temp,k,p,seed", [m for m in MATRIX if m[2] <= 262144 and m[1] <= 64 and m[0] != "special"])
def test_kept_set_matches_float64_reference(abi, kind, B, V, temp, k, p, seed):
    lg = make_logits(kind, B, V, seed, torch)
    out, probs, tr = abi.sample(lg.cuda(), abi.setup_rand(seed, B), temp, k, p, debug=True)
    d = cpu_ref.distribution(lg, temp, k, p)
    probs = probs.cpu().numpy()
    for b in range(min(B, 8)):
        kept32 = probs[b] >= np.float32(tr[b].threshold)
        # tolerance: a token may flip only at the boundary -- float64 cumulative mass within 1e-6 relative
        # of top_p, or a probability that ties with the boundary probability within 4e-6 (fp32 rounding of p)
        ok, nflips = kept_set_flips_ok(kept32, d, b)
        assert ok, (b, nflips)
        assert kept32[int(out[b])]


def test_chi_square_one_million_draws(abi):
    """1000 identical rows x 1000 calls = 10^6 draws against the float64 sampling weights
    (cells with expectation < 5 merged; reject below p = 1e-4)."""
    from scipy import stats
    V, R, CALLS = 8192, 1000, 1000
    row = make_logits("normal3", 1, V, 71, torch)
    lg = row.expand(R, V).contiguous().cuda()
    for temp, k, p in [(0.9, 64, 0.9), (1.0, -1, 0.5)]:
        st = abi.setup_rand(123, R)
        hist = torch.zeros(V, dtype=torch.int64, device="cuda")
        for _ in range(CALLS):
            hist += torch.bincount(abi.sample(lg, st, temp, k, p).long(), minlength=V)
        hist = hist.cpu().numpy().astype(np.float64)
        w = cpu_ref.distribution(row, temp, k, p)["weights"][0].numpy()
        exp = w / w.sum() * R * CALLS
        assert hist[exp == 0].sum() == 0
        order = np.argsort(-exp)
        e, o = exp[order], hist[order]
        cells_e, cells_o, ae, ao = [], [], 0.0, 0.0
        for ei, oi in zip(e, o):
            if ei == 0:
                break
            ae += ei
            ao += oi
            if ae >= 5:
                cells_e.append(ae); cells_o.append(ao); ae = ao = 0.0
        if ae > 0:
            cells_e[-1] += ae; cells_o[-1] += ao
        ce, cobs = np.array(cells_e), np.array(cells_o)
        chi2 = ((cobs - ce) ** 2 / ce).sum()
        pval = stats.chi2.sf(chi2, len(ce) - 1)
        assert pval > 1e-4, (temp, k, p, chi2, len(ce), pval)


def test_status_word_stays_clear_and_launches_are_counted(abi):
    n0 = abi.L.rs_kernel_launch_count()
    lg = make_logits("uniform", 2, 4096, 0, torch).cuda()
    abi.sample(lg, abi.setup_rand(0, 2), 1.0, -1, 0.5)
    assert abi.L.rs_kernel_launch_count() == n0 + 2          # setup_rand + sampler
    assert abi.device_status(2, 4096) == 0


def test_host_buffer_entry_point(abi):
    B, T, V = 6, 3, 32768
    lg = make_logits("normal3", B * T, V, 81, torch).reshape(B, T, V).pin_memory()
    s_a, s_b = abi.setup_rand(2, B), abi.setup_rand(2, B)
    want = abi.sample(lg.cuda(), s_a, 0.8, 50, 0.9).cpu()
    staging = torch.empty(B, V, device="cuda")
    out_dev = torch.empty(B, dtype=torch.int32, device="cuda")
    out_host = torch.empty(B, dtype=torch.int32).pin_memory()
    ws = abi.workspace(B, V)
    rc = abi.L.rs_sample_host(lg.data_ptr(), B, T, V, None, s_b.data_ptr(), out_host.data_ptr(), 0.8, 50, 0.9, 0.0, 0.0, 0.0,
                              staging.data_ptr(), out_dev.data_ptr(), ws.data_ptr(), ws.numel(), abi.stream())
    assert rc == 0
    assert torch.equal(out_host, want)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_sixteen_bit_logits_equal_reference_on_widened_logits(abi, ref, dtype):
    """fp16 / bf16 logits are read directly and widened exactly: ids, states and penalties must equal the
    reference kernel run on ``logits.float()`` (the reference itself rejects 16-bit input, sampling.cu:976)."""
    try:
        for kind, B, V, temp, k, p, rep in [("peaked", 16, 151936, 0.8, 50, 0.9, False), ("normal3", 4, 262144, 1.0, -1, 0.3, False),
                                            ("uniform", 4, 32768, 1.0, -1, 0.5, False), ("normal3", 32, 65536, 0.8, 50, 0.9, True),
                                            ("special", 4, 50304, 1.3, 100, 0.9, False), ("normal3", 200, 32768, 0.8, 50, 0.9, True),
                                            ("uniform", 160, 16380, 1.0, -1, 0.6, False)]:
            lg16 = make_logits(kind, B, V, 23, torch).to(dtype).cuda()
            lg32 = lg16.float()
            for mode in (0, 2, 3, 4, 5, 6):
                abi.set_path(mode)
                s_ref, s_our = ref.setup_rand(2, B), abi.setup_rand(2, B)
                pen_ref = torch.zeros(B, V, device="cuda") if rep else None
                pen_our = torch.zeros(B, V, device="cuda") if rep else None
                for _ in range(2):
                    want = _ref_call(ref, lg32, s_ref, temp, k, p, pen_ref)
                    got = abi.sample(lg16, s_our, temp, k, p, penalties=pen_our, presence=0.1, repetition=0.1, decay=0.95)
                    assert torch.equal(got, want), (kind, mode)
                assert torch.equal(s_our, s_ref)
                if rep:
                    assert torch.equal(pen_our, pen_ref)
    finally:
        abi.set_path(0)


def test_sixteen_bit_logits_through_the_torch_api(ref):
    import rapid_sampling_b200 as rs
    lg = make_logits("peaked", 8, 65536, 3, torch).to(torch.bfloat16).cuda()
    a = rs.batch_sampling_temperature_topk_topp_any(lg, rs.setup_rand(4, 8), 0.8, 50, 0.9)
    b = ref.batch_sampling_temperature_topk_topp(lg.float(), ref.setup_rand(4, 8), 0.8, 50, 0.9)
    assert torch.equal(a, b)
    with pytest.raises(ValueError, match="float32"):      # the reference-named call stays fp32-only
        rs.batch_sampling_temperature_topk_topp(lg, rs.setup_rand(4, 8), 0.8, 50, 0.9)
