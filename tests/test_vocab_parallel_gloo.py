"""CPU, world_size 2 over gloo: the vocab-parallel DRIVER (sequence of stages and collectives, bracket updates,
owner election, id exchange) with a numpy model standing in for the per-shard kernels."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

# the last one keeps the whole row: no candidate bound exists, so the 3-collective protocol must hand over to the staged one
CONFIGS = [(0.8, 50, 0.9), (1.0, -1, 0.3), (1.0, 5, 1.0), (1.3, -1, 1.0)]


def _worker(rank, world, port, q, fast=False, defer=False):
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    sys.path.insert(0, root)
    sys.path.insert(0, os.path.join(root, "tests"))
    from helpers import make_logits
    from oracle import c_oracle as co
    from oracle.vp_model import NumpyCompute, NumpyFastCompute
    from rapid_sampling_b200.vocab_parallel import VocabParallelSampler
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    B, V = 6, 4096
    full = make_logits("normal3", B, V, 5, torch)
    s = VocabParallelSampler(B, V, rank, world, device="cpu", compute=NumpyFastCompute() if fast else NumpyCompute(),
                             fast=fast, defer_check=defer)
    shard = full[:, s.col0:s.col0 + s.V_local].contiguous()
    states = torch.from_numpy(co.setup_rand(17, B))
    pen = torch.zeros(B, s.V_local)
    outs = []
    for temp, k, p in CONFIGS:
        ids = s.sample(shard, states, temp, k, p, penalties=pen, presence_penalty=0.1, repetition_penalty=0.2,
                       penalty_decay=0.5).clone()
        if defer:      # no verdict was awaited inside sample(): ask now; a repeat with the staged protocol replaces the ids
            fixed = s.validate()
            if fixed is not None:
                ids = fixed.clone()
        if s.last_protocol == "fast":
            thr = np.array([s.compute._thr[b] for b in range(B)], dtype=np.float32)
        else:
            thr = s.compute._bracket(8)[0].view(np.float32).copy()
        outs.append((ids.numpy(), thr, s.last_protocol))
    q.put((rank, outs, states.numpy().copy(), pen.numpy().copy()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("fast,defer", [(False, False), (True, False), (True, True)])
def test_two_rank_vocab_parallel_driver(fast, defer):
    from helpers import kept_set_flips_ok, make_logits
    from oracle import c_oracle as co
    from oracle import cpu_ref
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q, fast, defer)) for r in range(2)]
    for p in procs:
        p.start()
    res = dict()
    for _ in range(2):
        rank, outs, st, pen = q.get(timeout=180)
        res[rank] = (outs, st, pen)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    B, V = 6, 4096
    full = make_logits("normal3", B, V, 5, torch)
    # both ranks agree on ids and thresholds; states advanced identically (one draw per call and row)
    want_states = co.setup_rand(17, B)
    for b in range(B):
        for _ in range(len(CONFIGS)):
            co.draw4(want_states, b)
    assert np.array_equal(res[0][1], want_states) and np.array_equal(res[1][1], want_states)
    pen_full = torch.zeros(B, V)
    for i, (temp, k, p) in enumerate(CONFIGS):
        ids0, thr0, proto0 = res[0][0][i]
        ids1, thr1, proto1 = res[1][0][i]
        assert proto0 == proto1 == ("fast" if fast and i < 3 else "staged")
        assert np.array_equal(ids0, ids1) and np.array_equal(thr0.view(np.uint32), thr1.view(np.uint32))
        d = cpu_ref.distribution(full, temp, k, p, penalties=pen_full)
        for b in range(B):
            kept32 = d["probs"][b].numpy().astype(np.float32) >= thr0[b]
            ok, n = kept_set_flips_ok(kept32, d, b, mass_tol=2e-6, tie_tol=1e-5)
            assert ok, (i, b, n)
            assert d["kept"][b][ids0[b]] or kept32[ids0[b]]
        # float64 statement of the penalty update with the ids that were sampled
        hit = torch.zeros(B, V)
        for b in range(B):
            hit[b, ids0[b]] = 0.1 if pen_full[b, ids0[b]] == 0 else 0.2
        pen_full = pen_full * 0.5 + hit
    got = np.concatenate([res[0][2], res[1][2]], axis=1)
    assert np.allclose(got, pen_full.numpy(), rtol=1e-6, atol=0)
