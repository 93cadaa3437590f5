"""GPU: the vocab-parallel kernels (rs_vp_stage through the C ABI).  N ranks are emulated on one GPU by running
every rank's stage back to back and reducing their workspace regions by hand -- the same numbers NCCL would
deliver -- so the multi-rank arithmetic is checked without several GPUs.  With >= 2 GPUs visible the real NCCL
path is exercised as well."""
import numpy as np
import pytest
import torch

from helpers import kept_set_flips_ok, make_logits
from oracle import cpu_ref

pytestmark = pytest.mark.gpu


def emulated_sample(samplers, shards, states, temp, k, p, pens=None, fast=True):
    """Drives N single-process 'ranks' through the stage sequence of VocabParallelSampler.sample."""
    from rapid_sampling_b200 import abi
    N = len(samplers)
    for r, s in enumerate(samplers):
        s.compute.bind(s, shards[r], states[r], None if pens is None else pens[r], temp, k, p, 0.1, 0.2, 0.5)
    if fast:
        def fstep(name, region=None, op=None, rnd=0):
            for s in samplers:
                s.compute.stage(name, rnd)
            if region is not None:
                stack = torch.stack([region(s) for s in samplers])
                red = stack.max(dim=0).values if op == "max" else stack.sum(dim=0)
                for s in samplers:
                    region(s).copy_(red)
        fstep("f_max", lambda s: s.f_stat1, "max")
        fstep("f_sum", lambda s: s.f_stat2, "sum")
        fstep("f_extract")
        fstep("f_compact")
        for s in samplers:          # the all-gather
            s.f_gath_block.copy_(torch.cat([x.f_send_block for x in samplers]))
        fstep("f_finish")
        before = [st.clone() for st in states]
        fstep("f_advance")            # applied by the device only if every row was settled
        if pens is not None:
            fstep("penalty", rnd=1)
        torch.cuda.synchronize()
        if all(int(s.f_all_valid.item()) == 1 for s in samplers):
            assert all(int(s.f_valid.min()) == 1 for s in samplers)
            emulated_sample.last = "fast"
            return [s.f_ids - 1 for s in samplers]
        assert all(int(s.f_all_valid.item()) == 0 and int(s.f_valid.min()) == 0 for s in samplers)   # same verdict on every rank
        assert all(torch.equal(a, b) for a, b in zip(before, states))   # nothing was advanced
    emulated_sample.last = "staged"

    def step(name, rnd, region, op):
        for s in samplers:
            s.compute.stage(name, rnd)
        if region is not None:
            stack = torch.stack([region(s) for s in samplers])
            red = stack.max(dim=0).values if op == "max" else stack.sum(dim=0)
            for s in samplers:
                region(s).copy_(red)
    step("max", 0, lambda s: s.gmax, "max")
    step("sum", 0, lambda s: s.gsum, "sum")
    for r in range(abi.VP_ROUNDS):
        step("round", r, lambda s, r=r: s.tallies[r], "sum")
    step("tally", 0, lambda s: s.gtally, "sum")
    step("weight", 0, lambda s: s.weights, "sum")
    step("pick", 0, lambda s: s.ids, "max")
    if pens is not None:
        step("penalty", 0, None, None)
    return [s.ids - 1 for s in samplers]


@pytest.mark.parametrize("N", [1, 2, 8])
def test_emulated_ranks_agree_and_match_float64_kept_set(abi, N):
    from rapid_sampling_b200.vocab_parallel import VocabParallelSampler
    B, V = 8, 32768
    full = make_logits("peaked", B, V, 4, torch)
    samplers = [VocabParallelSampler(B, V, r, N) for r in range(N)]
    shards = [full[:, s.col0:s.col0 + s.V_local].contiguous().cuda() for s in samplers]
    states = [abi.setup_rand(9, B) for _ in range(N)]
    pens = [torch.zeros(B, s.V_local, device="cuda") for s in samplers]
    pen64 = torch.zeros(B, V)
    used = []
    for temp, k, p in [(0.8, 50, 0.9), (1.0, -1, 0.5), (1.0, -1, 1.0), (0.7, 1, 0.0)]:
        ids = emulated_sample(samplers, shards, states, temp, k, p, pens)
        used.append(emulated_sample.last)
        torch.cuda.synchronize()
        for r in range(1, N):
            assert torch.equal(ids[r], ids[0])
            assert torch.equal(states[r], states[0])
        d = cpu_ref.distribution(full, temp, k, p, penalties=pen64)
        got = ids[0].cpu().numpy()
        for b in range(B):
            assert 0 <= got[b] < V
            # the sampled id lies in the float64 kept set, or ties with its boundary within fp32 rounding
            assert bool(d["kept"][b][got[b]]) or abs(float(d["probs"][b][got[b]]) - float(d["v"][b])) <= 1e-5 * float(d["v"][b])
        hit = torch.zeros(B, V)
        for b in range(B):
            hit[b, got[b]] = 0.1 if pen64[b, got[b]] == 0 else 0.2
        pen64 = pen64 * 0.5 + hit
        cat = torch.cat([x.cpu() for x in pens], dim=1)
        assert torch.allclose(cat, pen64, rtol=1e-6, atol=0)
    assert used[0] == "fast" and used[2] == "staged"      # peaked top-k rows settle on candidates; 'keep everything' cannot


def test_threshold_matches_single_gpu_kernel(abi):
    """Same kept set as the single-GPU sampler (whose threshold is bit-identical to the reference's)."""
    from rapid_sampling_b200.vocab_parallel import VocabParallelSampler
    B, V, N = 4, 65536, 4
    full = make_logits("normal3", B, V, 6, torch)
    _, probs, tr = abi.sample(full.cuda(), abi.setup_rand(1, B), 0.9, -1, 0.8, debug=True)
    samplers = [VocabParallelSampler(B, V, r, N) for r in range(N)]
    shards = [full[:, s.col0:s.col0 + s.V_local].contiguous().cuda() for s in samplers]
    emulated_sample(samplers, shards, [abi.setup_rand(1, B) for _ in range(N)], 0.9, -1, 0.8, fast=False)
    torch.cuda.synchronize()
    d = cpu_ref.distribution(full, 0.9, -1, 0.8)
    s0 = samplers[0]
    g = s0.gtally.cpu().numpy().reshape(B, 4)
    for b in range(B):
        kept_single = int((probs[b] >= tr[b].threshold).sum())
        kept_vp = int(g[b, 0] + g[b, 2])
        assert abs(kept_single - kept_vp) <= 2           # summation order may move the boundary by a token
        assert abs(kept_vp - int(d["kept"][b].sum())) <= 2


def test_chi_square_vocab_parallel(abi):
    """10^6 draws through 4 emulated ranks against the float64 sampling weights."""
    from scipy import stats
    from rapid_sampling_b200.vocab_parallel import VocabParallelSampler
    V, R, CALLS, N = 8192, 1000, 1000, 4
    row = make_logits("normal3", 1, V, 71, torch)
    full = row.expand(R, V).contiguous()
    samplers = [VocabParallelSampler(R, V, r, N) for r in range(N)]
    shards = [full[:, s.col0:s.col0 + s.V_local].contiguous().cuda() for s in samplers]
    states = [abi.setup_rand(5, R) for _ in range(N)]
    hist = torch.zeros(V, dtype=torch.int64, device="cuda")
    for _ in range(CALLS):
        ids = emulated_sample(samplers, shards, states, 0.9, 64, 0.9)
        hist += torch.bincount(ids[0].long(), minlength=V)
    hist = hist.cpu().numpy().astype(np.float64)
    w = cpu_ref.distribution(row, 0.9, 64, 0.9)["weights"][0].numpy()
    exp = w / w.sum() * R * CALLS
    assert hist[exp == 0].sum() <= 2          # a boundary tie may admit a token the float64 set excludes
    order = np.argsort(-exp)
    e, o = exp[order], hist[order]
    ce, cobs, ae, ao = [], [], 0.0, 0.0
    for ei, oi in zip(e, o):
        if ei == 0:
            break
        ae += ei; ao += oi
        if ae >= 5:
            ce.append(ae); cobs.append(ao); ae = ao = 0.0
    if ae > 0:
        ce[-1] += ae; cobs[-1] += ao
    ce, cobs = np.array(ce), np.array(cobs)
    chi2 = ((cobs - ce) ** 2 / ce).sum()
    assert stats.chi2.sf(chi2, len(ce) - 1) > 1e-4, chi2


def _nccl_worker(rank, world, port, q):
    import os, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root); sys.path.insert(0, os.path.join(root, "tests"))
    import torch.distributed as dist
    from helpers import Abi, make_logits as ml
    from rapid_sampling_b200.vocab_parallel import VocabParallelSampler
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world,
                            device_id=torch.device("cuda", rank))
    B, V = 8, 65536
    full = ml("peaked", B, V, 4, torch)
    s = VocabParallelSampler(B, V, rank, world)
    shard = full[:, s.col0:s.col0 + s.V_local].contiguous().cuda()
    st = Abi().setup_rand(9, B)
    out = [s.sample(shard, st, 0.8, 50, 0.9).cpu().numpy() for _ in range(3)]
    # the same three calls with the stages recorded into a CUDA graph (first call eager, second records, third replays)
    sg = VocabParallelSampler(B, V, rank, world, graph=True)
    stg = Abi().setup_rand(9, B)
    outg = [sg.sample(shard, stg, 0.8, 50, 0.9).cpu().numpy() for _ in range(3)]
    ok = bool(torch.equal(st, stg)) and sg.last_protocol == "fast"
    sg.release_graphs()       # NCCL cannot shut the communicator down while a graph that captured its collectives lives
    q.put((rank, (out, s.last_protocol, outg, ok)))
    dist.barrier()
    dist.destroy_process_group()


def test_nccl_two_gpus_match_emulation(abi):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import socket
    import torch.multiprocessing as mp
    from rapid_sampling_b200.vocab_parallel import VocabParallelSampler
    sk = socket.socket(); sk.bind(("127.0.0.1", 0)); port = sk.getsockname()[1]; sk.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_nccl_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=300) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    B, V = 8, 65536
    full = make_logits("peaked", B, V, 4, torch)
    samplers = [VocabParallelSampler(B, V, r, 2) for r in range(2)]
    shards = [full[:, s.col0:s.col0 + s.V_local].contiguous().cuda() for s in samplers]
    states = [abi.setup_rand(9, B) for _ in range(2)]
    for call in range(3):
        want = emulated_sample(samplers, shards, states, 0.8, 50, 0.9)[0].cpu().numpy()
        assert np.array_equal(res[0][0][call], want) and np.array_equal(res[1][0][call], want)
        assert np.array_equal(res[0][2][call], want) and np.array_equal(res[1][2][call], want)   # graph replays
    assert res[0][1] == res[1][1] == "fast" and res[0][3] and res[1][3]


def test_graph_replay_matches_eager_single_rank(abi):
    """The stages of the fast protocol recorded into a CUDA graph (first call eager, second records, later ones replay):
    same ids, states and penalties as eager calls, including the device-side gate on the state advance."""
    from rapid_sampling_b200.vocab_parallel import VocabParallelSampler
    B, V = 8, 65536
    shard = make_logits("peaked", B, V, 4, torch).cuda()
    eager, graph = VocabParallelSampler(B, V, 0, 1), VocabParallelSampler(B, V, 0, 1, graph=True)
    st_e, st_g = abi.setup_rand(9, B), abi.setup_rand(9, B)
    pen_e, pen_g = torch.zeros(B, V, device="cuda"), torch.zeros(B, V, device="cuda")
    for call in range(4):
        a = eager.sample(shard, st_e, 0.8, 50, 0.9, penalties=pen_e, presence_penalty=0.1, repetition_penalty=0.2,
                         penalty_decay=0.5).clone()
        b = graph.sample(shard, st_g, 0.8, 50, 0.9, penalties=pen_g, presence_penalty=0.1, repetition_penalty=0.2,
                         penalty_decay=0.5).clone()
        assert eager.last_protocol == graph.last_protocol == "fast"
        assert torch.equal(a, b), call
        assert torch.equal(st_e, st_g) and torch.equal(pen_e, pen_g)
    graph.release_graphs()


def test_two_runs_give_identical_bits(abi):
    """The mode must give the same result every run: the octave histogram that steers the candidate bound is summed in
    integers, so neither it nor anything derived from it depends on the order in which shared-memory atomics land."""
    from rapid_sampling_b200.vocab_parallel import VocabParallelSampler
    B, V, N = 16, 262144, 4
    full = make_logits("normal3", B, V, 8, torch)
    runs = []
    for _ in range(2):
        samplers = [VocabParallelSampler(B, V, r, N) for r in range(N)]
        shards = [full[:, s.col0:s.col0 + s.V_local].contiguous().cuda() for s in samplers]
        states = [abi.setup_rand(3, B) for _ in range(N)]
        out = []
        for call in range(3):
            ids = emulated_sample(samplers, shards, states, 1.0, -1, 0.9)
            torch.cuda.synchronize()
            out.append((ids[0].clone(), samplers[0].f_stat2.clone(), samplers[0].f_gath_cnt.clone()))
        runs.append(out)
    for a, b in zip(*runs):
        assert torch.equal(a[0], b[0])
        assert torch.equal(a[1].view(torch.int32), b[1].view(torch.int32))       # reduced histograms, bit for bit
        assert torch.equal(a[2].view(torch.int32), b[2].view(torch.int32))       # candidate counts per rank


def test_deferred_check_single_rank(abi):
    """defer_check=True: sample() returns without waiting for the device's verdict; validate() reads it and repeats a
    call that could not be settled (top_k = -1, top_p = 1 keeps the whole row: no candidate bound exists)."""
    from rapid_sampling_b200.vocab_parallel import VocabParallelSampler
    B, V = 8, 65536
    shard = make_logits("peaked", B, V, 4, torch).cuda()
    sync, lazy = VocabParallelSampler(B, V, 0, 1), VocabParallelSampler(B, V, 0, 1, defer_check=True)
    st_s, st_l = abi.setup_rand(9, B), abi.setup_rand(9, B)
    for temp, k, p, proto in [(0.8, 50, 0.9, "fast"), (1.0, -1, 1.0, "staged"), (0.8, 50, 0.9, "fast")]:
        want = sync.sample(shard, st_s, temp, k, p).clone()
        got = lazy.sample(shard, st_l, temp, k, p).clone()
        fixed = lazy.validate()
        assert (fixed is not None) == (proto == "staged")
        if fixed is not None:
            got = fixed.clone()
        assert sync.last_protocol == proto
        assert torch.equal(got, want) and torch.equal(st_s, st_l)


def test_lm_head_tile_hook_matches_the_max_pass(abi):
    """The row maxima of the first stage fed tile by tile (as an lm_head epilogue would hand its output over), in a
    shuffled order and with uneven tile widths, on 2 emulated ranks: same ids, states and penalties as the normal call."""
    from rapid_sampling_b200.vocab_parallel import VocabParallelSampler
    B, V, N = 8, 65536, 2
    full = make_logits("peaked", B, V, 4, torch)
    ref_s = [VocabParallelSampler(B, V, r, N) for r in range(N)]
    hook_s = [VocabParallelSampler(B, V, r, N) for r in range(N)]
    shards = [full[:, s.col0:s.col0 + s.V_local].contiguous().cuda() for s in ref_s]
    st_ref = [abi.setup_rand(9, B) for _ in range(N)]
    st_hook = [abi.setup_rand(9, B) for _ in range(N)]
    pen_ref = [torch.zeros(B, s.V_local, device="cuda") for s in ref_s]
    pen_hook = [torch.zeros(B, s.V_local, device="cuda") for s in ref_s]
    g = torch.Generator().manual_seed(1)
    for call in range(3):
        want = emulated_sample(ref_s, shards, st_ref, 0.8, 50, 0.9, pen_ref)
        # hook path: stage 1 from tiles, the remaining stages as in emulated_sample
        for r, s in enumerate(hook_s):
            s.begin_tiles(shards[r], st_hook[r], 0.8, 50, 0.9, penalties=pen_hook[r], presence_penalty=0.1,
                          repetition_penalty=0.2, penalty_decay=0.5)
            edges = sorted(set([0, s.V_local] + [int(x) * 4 for x in torch.randint(1, s.V_local // 4, (9,), generator=g)]))
            tiles = list(zip(edges[:-1], edges[1:]))
            for i in torch.randperm(len(tiles), generator=g).tolist():
                a, b_ = tiles[i]
                s.push_tile(shards[r][:, a:b_], a)
        # emulate the all-reduce MAX and run the remaining stages
        stack = torch.stack([s.f_stat1 for s in hook_s]).max(dim=0).values
        for s in hook_s:
            s.f_stat1.copy_(stack)
        for name in ("f_sum",):
            for s in hook_s:
                s.compute.stage(name)
        red = torch.stack([s.f_stat2 for s in hook_s]).sum(dim=0)
        for s in hook_s:
            s.f_stat2.copy_(red)
        for s in hook_s:
            s.compute.stage("f_extract")
        for s in hook_s:
            s.f_gath_block.copy_(torch.cat([x.f_send_block for x in hook_s]))
        for name, rnd in (("f_finish", 0), ("f_advance", 0), ("penalty", 1)):
            for s in hook_s:
                s.compute.stage(name, rnd)
        torch.cuda.synchronize()
        for r in range(N):
            assert int(hook_s[r].f_all_valid.item()) == 1
            assert torch.equal(hook_s[r].f_ids - 1, want[r]), (call, r)
            assert torch.equal(st_hook[r], st_ref[r]) and torch.equal(pen_hook[r], pen_ref[r])


def test_lm_head_tile_hook_through_the_driver(abi):
    """Single rank, through VocabParallelSampler.sample(max_from_tiles=True)."""
    from rapid_sampling_b200.vocab_parallel import VocabParallelSampler
    B, V = 8, 65536
    shard = make_logits("peaked", B, V, 4, torch).cuda()
    a, h = VocabParallelSampler(B, V, 0, 1), VocabParallelSampler(B, V, 0, 1)
    st_a, st_h = abi.setup_rand(9, B), abi.setup_rand(9, B)
    for call in range(3):
        want = a.sample(shard, st_a, 0.8, 50, 0.9).clone()
        h.begin_tiles(shard, st_h, 0.8, 50, 0.9)
        for c0 in (32768, 0, 49152, 16384):
            h.push_tile(shard[:, c0:c0 + 16384], c0)
        got = h.sample(shard, st_h, 0.8, 50, 0.9, max_from_tiles=True).clone()
        assert h.last_protocol == "fast"
        assert torch.equal(got, want) and torch.equal(st_a, st_h)
