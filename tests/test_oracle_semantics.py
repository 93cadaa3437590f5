"""CPU: the fp32 order-faithful C oracle against the float64 closed form, on small seeded cases,
plus the properties the reference relies on (monotone scan, argument remaps)."""
import numpy as np
import pytest
import torch

from helpers import kept_set_flips_ok, make_logits
from oracle import c_oracle as co
from oracle import cpu_ref

CASES = [
    ("uniform", 2, 4096, 1.0, -1, 0.5),
    ("uniform", 2, 8192, 1.0, -1, 1.0),
    ("normal3", 2, 8192, 1.0, -1, 0.3),
    ("normal3", 2, 8192, 0.8, 50, 0.9),
    ("peaked", 2, 4096, 0.8, 10, 0.95),
    ("coarse", 2, 4096, 0.9, 7, 0.6),
    ("coarse", 2, 1024, 1.0, -1, 0.7),
    ("equal", 2, 256, 1.0, -1, 0.5),
    ("equal", 1, 64, 2.0, 5, 1.0),
    ("special", 2, 4096, 1.3, 100, 0.9),
    ("uniform", 2, 4, 1.0, -1, 0.5),
    ("normal3", 2, 32768, 1.0, -1, 0.999999),
    ("uniform", 2, 2052, 1.0, 1, 0.0),      # greedy remap; ragged lanes (V/4 not a multiple of 1024 lanes)
]


@pytest.mark.parametrize("kind,B,V,temp,k,p", CASES)
def test_kept_set_and_weights_match_float64(kind, B, V, temp, k, p):
    lg = make_logits(kind, B, V, 11, torch)
    d = cpu_ref.distribution(lg, temp, k, p)
    knd, scale, kk, pp_ = co.normalise(V, B, 1, temp, k, p)
    st = co.setup_rand(5, B)
    for b in range(B):
        tok, tr, probs = co.sample_row(lg[b].numpy(), st[64 * b:64 * b + 64], knd, scale, kk, pp_, want_probs=True)
        kept32 = probs >= np.float32(tr.threshold)
        ok, nflips = kept_set_flips_ok(kept32, d, b)     # flips only at the mass / tie boundary
        assert ok, (kind, b, nflips)
        flips = [0] * nflips
        assert kept32[tok]
        # weights: full above the threshold, scaled by comp at it
        w32 = np.where(probs > tr.threshold, probs, np.where(probs == tr.threshold, probs * tr.comp, 0)).astype(np.float64)
        w64 = d["weights"][b].numpy()
        if len(flips) == 0:
            assert abs(w32.sum() - w64.sum()) <= 1e-5 * max(w64.sum(), 1e-30)
        assert 0.0 <= tr.comp <= 1.0


def test_brute_force_tiny_rows():
    """V = 8: enumerate the semantics by hand (sort, cumsum) for every row."""
    g = torch.Generator().manual_seed(3)
    lg = torch.randn(64, 8, generator=g)
    for b in range(64):
        for (k, p) in [(-1, 0.6), (3, 1.0), (2, 0.9)]:
            knd, scale, kk, pp_ = co.normalise(8, 1, 1, 1.0, k, p)
            st = co.setup_rand(b, 1)
            tok, tr, probs = co.sample_row(lg[b].numpy(), st, knd, scale, kk, pp_, want_probs=True)
            pr = np.exp(lg[b].double().numpy())
            pr /= pr.sum()
            order = np.argsort(-pr, kind="stable")
            cum = np.cumsum(pr[order])
            n_p = 8 if p >= 1 else int(np.searchsorted(cum, p, side="left")) + 1
            n = min(n_p, kk)
            expect = set(order[:n].tolist())
            got = set(np.nonzero(probs >= tr.threshold)[0].tolist())
            # fp32 rounding can move the boundary only when the cumulative mass is within 1e-6 of top_p
            if got != expect:
                assert p < 1 and min(abs(cum - p)) < 1e-6
            assert tok in got


def test_descending_scan_is_monotone_and_ascending_is_not():
    """The property behind sampling.cu:48-58 / monotonicity.py: Hillis-Steele with descending offsets
    never decreases on non-negative fp32 input; ascending offsets do."""
    rng = np.random.default_rng(0)
    bad_asc = 0
    for _ in range(300):
        x = rng.integers(0, 0x70000000, 2048, dtype=np.int64).astype(np.uint32).view(np.float32)
        d = co.scan_n(x, ascending=False)
        a = co.scan_n(x, ascending=True)
        assert np.all(d[1:] >= d[:-1])
        bad_asc += int(np.any(a[1:] < a[:-1]))
    assert bad_asc > 0


def test_block_scan_monotone_and_total():
    rng = np.random.default_rng(1)
    for _ in range(200):
        x = (rng.random(1024, dtype=np.float32) ** 8).astype(np.float32)
        out, total = co.block_scan(x)
        assert np.all(out[1:] >= out[:-1])
        assert out[-1] == total
        assert abs(float(total) - float(x.astype(np.float64).sum())) < 1e-3


def test_argument_remaps_and_errors():
    LOG2E = 1.4426950408889634
    assert co.normalise(1024, 1, 1, 1.0, -1, 0.5) == (co.KIND_TOPP, pytest.approx(np.float32(LOG2E)), 1024, 0.5)
    assert co.normalise(1024, 1, 1, 1.0, 5000, 0.5)[0] == co.KIND_TOPP          # top_k > V -> V
    assert co.normalise(1024, 1, 1, 0.5, -1, 0.5)[0] == co.KIND_GENERAL
    assert co.normalise(1024, 1, 1, 1.0, 10, 0.5)[0] == co.KIND_GENERAL
    assert co.normalise(1024, 1, 1, 1.0, -1, 0.5, with_penalties=True)[0] == co.KIND_REPETITION
    k = co.normalise(1024, 1, 1, 1.0, -1, 0.0)                                  # top_p == 0 -> greedy
    assert (k[2], k[3]) == (1, 1.0)
    assert co.normalise(1024, 1, 1, 1.0, -1, 1.5)[3] == 1.0
    assert co.normalise(1024, 1, 1, 1.0, -1, -0.1)[3] == 1.0
    for bad_v in (0, 6, 1048580):
        with pytest.raises(ValueError):
            co.normalise(bad_v, 1, 1, 1.0, -1, 0.5)
    for bad_t in (0.0005, 1001.0, float("nan")):
        with pytest.raises(ValueError):
            co.normalise(1024, 1, 1, bad_t, -1, 0.5)
    with pytest.raises(ValueError):
        co.normalise(1024, 0, 1, 1.0, -1, 0.5)


def test_greedy_picks_argmax():
    lg = make_logits("normal3", 8, 4096, 2, torch)
    st = co.setup_rand(1, 8)
    out = co.sample(lg.numpy(), st, 1.0, -1, 0.0)
    assert np.array_equal(out, lg.argmax(dim=-1).numpy().astype(np.int32))


def test_penalty_update_rule():
    """sampling.cu:427-437: every entry decays; the sampled id gets presence (if it was 0) or repetition."""
    V = 1024
    lg = make_logits("normal3", 4, V, 9, torch).numpy()
    pen = np.zeros((4, V), dtype=np.float32)
    pen[:, 5] = 0.25
    st = co.setup_rand(2, 4)
    before = pen.copy()
    out = co.sample(lg, st, 0.8, 50, 0.9, penalties=pen, presence=0.3, repetition=0.7, decay=0.5)
    for b in range(4):
        exp = before[b] * np.float32(0.5)
        t = out[b]
        exp[t] = np.float32(np.float32(before[b, t]) * np.float32(0.5) + np.float32(0.3 if before[b, t] == 0 else 0.7))
        assert np.allclose(pen[b], exp, rtol=1e-6, atol=0)


def test_last_position_of_btv_is_used():
    lg = make_logits("normal3", 3 * 4, 2048, 4, torch).reshape(3, 4, 2048)
    st1, st2 = co.setup_rand(8, 3), co.setup_rand(8, 3)
    a = co.sample(lg.numpy(), st1, 0.9, 20, 0.9)
    b = co.sample(lg[:, -1, :].contiguous().numpy(), st2, 0.9, 20, 0.9)
    assert np.array_equal(a, b) and np.array_equal(st1, st2)
