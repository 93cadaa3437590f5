"""GPU: the benchmark configurations exactly as they are stated (batch, vocabulary, distribution, seeds, call count),
on the kernel variant the launch planner picks for them by itself -- the same path the benchmark times.

Bar: ids, RNG states and penalty tensors bit-identical to the reference's own CUDA extension (oracle/_ref);
for the vocab-parallel mode (no reference counterpart): identical ids on every rank, inside the float64 kept set.
The reference is only ever given 2-D logits: for (B, T, V) input it indexes its (B, V) scratch with the 3-D
offset (sampling.cu:488 against :206) and would write out of bounds.
"""
import numpy as np
import pytest
import torch

from helpers import make_logits

pytestmark = pytest.mark.gpu


def boosted_btv(B, T, V, seed):
    """(B, T, V) N(0,1) logits with 1 % of the ids of every row boosted by +8 (the same ids at every position)."""
    g = torch.Generator(device="cuda").manual_seed(seed)
    x = torch.randn(B, T, V, generator=g, device="cuda")
    idx = torch.randint(0, V, (B, V // 100), generator=g, device="cuda")
    boost = torch.zeros(B, V, device="cuda").scatter_(1, idx, 8.0)
    return x + boost.unsqueeze(1)


def test_repetition_workload_as_stated_256_rows_128_steps(abi, ref):
    """B=256, V=65536, N(0, 2.5^2) logits regenerated from seed 3+step, penalties from zero, 128 chained calls.
    Every step's ids must match (the penalties of step n+1 depend on every id of step n), and the final
    penalties and states must be equal bit for bit (stated tolerance: 1e-6 relative)."""
    B, V = 256, 65536
    pen_ref, pen_our = torch.zeros(B, V, device="cuda"), torch.zeros(B, V, device="cuda")
    s_ref, s_our = ref.setup_rand(3, B), abi.setup_rand(3, B)
    for step in range(128):
        g = torch.Generator(device="cuda").manual_seed(3 + step)
        lg = torch.randn(B, V, generator=g, device="cuda") * 2.5
        want = ref.batch_sampling_repetition_temperature_topk_topp(lg, pen_ref, s_ref, 0.1, 0.1, 0.95, 0.8, 50, 0.9)
        got = abi.sample(lg, s_our, 0.8, 50, 0.9, penalties=pen_our, presence=0.1, repetition=0.1, decay=0.95)
        assert torch.equal(got, want), (step, (got != want).nonzero().flatten()[:5].tolist())
    assert torch.equal(pen_our.view(torch.int32), pen_ref.view(torch.int32))
    assert torch.equal(s_our, s_ref)
    assert int((pen_our != 0).sum()) > B
    assert abi.device_status(B, V) == 0


def test_large_vocab_workload_as_stated_btv(abi, ref):
    """(B, T, V) = (32, 4, 1048576), 1 % boosted, top_p 0.95: ours reads position T-1 of the 3-D tensor in place,
    the reference gets the contiguous last slice."""
    B, T, V = 32, 4, 1048576
    lg = boosted_btv(B, T, V, 4)
    last = lg[:, -1, :].contiguous()
    s_ref, s_our = ref.setup_rand(4, B), abi.setup_rand(4, B)
    for call in range(3):
        want = ref.batch_sampling_temperature_topk_topp(last, s_ref, 1.0, -1, 0.95)
        got = abi.sample(lg, s_our, 1.0, -1, 0.95)
        assert torch.equal(got, want), (call, (got != want).nonzero().flatten()[:5].tolist())
        assert torch.equal(s_our, s_ref)
    assert abi.device_status(B, V) == 0


@pytest.mark.parametrize("N", [1, 8])
def test_large_vocab_workload_vocab_parallel(abi, N):
    """The same rows split over N ranks (emulated on one GPU: every rank's stage kernels run back to back and the
    collectives are done by hand on their workspace regions).  Every rank must name the same ids, and each id
    must lie in the float64 kept set (or tie with its boundary within fp32 rounding)."""
    from test_gpu_vocab_parallel import emulated_sample
    from oracle import cpu_ref
    from rapid_sampling_b200.vocab_parallel import VocabParallelSampler
    B, T, V = 32, 4, 1048576
    lg = boosted_btv(B, T, V, 4)
    samplers = [VocabParallelSampler(B, V, r, N, T=T) for r in range(N)]
    shards = [lg[:, :, s.col0:s.col0 + s.V_local].contiguous() for s in samplers]
    states = [abi.setup_rand(4, B) for _ in range(N)]
    last = lg[:, -1, :].cpu()
    del lg
    d = cpu_ref.distribution(last, 1.0, -1, 0.95)
    for call in range(2):
        ids = emulated_sample(samplers, shards, states, 1.0, -1, 0.95)
        torch.cuda.synchronize()
        assert emulated_sample.last == "fast"
        for r in range(1, N):
            assert torch.equal(ids[r], ids[0]) and torch.equal(states[r], states[0])
        got = ids[0].cpu().numpy()
        for b in range(B):
            assert 0 <= got[b] < V
            pb, vb = float(d["probs"][b][got[b]]), float(d["v"][b])
            assert bool(d["kept"][b][got[b]]) or abs(pb - vb) <= 1e-5 * vb, (call, b)


def test_batch_shards_reproduce_the_unsharded_ids(abi):
    """Rank r of N takes rows [r*B/N, (r+1)*B/N) with RNG subsequences counted from its first GLOBAL row
    (rs_setup_rand(first_row)): the shards' ids, states and penalties concatenate to the unsharded call's."""
    B, V, N = 24, 65536, 3
    lg = make_logits("normal3", B, V, 91, torch).cuda()
    pen_all = torch.zeros(B, V, device="cuda")
    st_all = abi.setup_rand(17, B)
    per = B // N
    pens = [torch.zeros(per, V, device="cuda") for _ in range(N)]
    sts = [abi.setup_rand(17, per, first_row=r * per) for r in range(N)]
    for call in range(3):
        want = abi.sample(lg, st_all, 0.8, 50, 0.9, penalties=pen_all, presence=0.1, repetition=0.1, decay=0.95)
        got = torch.cat([abi.sample(lg[r * per:(r + 1) * per], sts[r], 0.8, 50, 0.9, penalties=pens[r], presence=0.1,
                                    repetition=0.1, decay=0.95) for r in range(N)])
        assert torch.equal(got, want), call
    assert torch.equal(torch.cat(sts), st_all)
    assert torch.equal(torch.cat(pens), pen_all)
