"""CPU, world_size 2 over gloo: batch sharding is a pure partition -- each rank samples its own rows
with states seeded by GLOBAL row index, and the gathered ids equal the unsharded run (checked with
the CPU oracle standing in for the kernel; the GPU version of this check is
test_batch_shards_reproduce_the_unsharded_ids in test_gpu_baseline_configs.py)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from rapid_sampling_b200.sharding import row_range, vocab_range


def test_row_range_is_a_partition():
    for B in (1, 2, 7, 64, 255, 256):
        for world in (1, 2, 3, 4, 8):
            covered = []
            for r in range(world):
                a, b = row_range(B, r, world)
                assert 0 <= a <= b <= B
                covered += list(range(a, b))
            assert covered == list(range(B))
            sizes = [row_range(B, r, world)[1] - row_range(B, r, world)[0] for r in range(world)]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        row_range(4, 2, 2)


def test_vocab_range():
    assert vocab_range(1048576, 3, 8) == (393216, 524288)
    with pytest.raises(ValueError):
        vocab_range(1000, 0, 3)
    with pytest.raises(ValueError):
        vocab_range(24, 0, 4)      # 6 columns per shard: not a multiple of 4


def _worker(rank, world, port, B, V, q):
    import sys
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    from helpers import make_logits
    from oracle import c_oracle as co
    dist.init_process_group("gloo", init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
    lg = make_logits("normal3", B, V, 21, torch)
    a, b = row_range(B, rank, world)
    st = co.setup_rand(99, b - a, row0=a)
    pen = np.zeros((b - a, V), dtype=np.float32)
    ids = None
    for _ in range(3):
        ids = co.sample(lg[a:b].numpy(), st, 0.8, 50, 0.9, penalties=pen, presence=0.1, repetition=0.1, decay=0.95, nthreads=1)
    # gather (control plane only; the data path has no collective)
    sizes = [row_range(B, r, world)[1] - row_range(B, r, world)[0] for r in range(world)]
    parts = [torch.zeros(s, dtype=torch.int32) for s in sizes]
    if len(set(sizes)) == 1:
        dist.all_gather(parts, torch.from_numpy(ids))
    else:
        pad = max(sizes)
        padded = [torch.zeros(pad, dtype=torch.int32) for _ in range(world)]
        mine = torch.zeros(pad, dtype=torch.int32)
        mine[:len(ids)] = torch.from_numpy(ids)
        dist.all_gather(padded, mine)
        parts = [p[:s] for p, s in zip(padded, sizes)]
    if rank == 0:
        q.put(torch.cat(parts).numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("B", [8, 7])
def test_two_rank_batch_shard_equals_unsharded(B):
    from helpers import make_logits
    from oracle import c_oracle as co
    V = 2048
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, B, V, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = q.get(timeout=120)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    lg = make_logits("normal3", B, V, 21, torch)
    st = co.setup_rand(99, B)
    pen = np.zeros((B, V), dtype=np.float32)
    for _ in range(3):
        want = co.sample(lg.numpy(), st, 0.8, 50, 0.9, penalties=pen, presence=0.1, repetition=0.1, decay=0.95)
    assert np.array_equal(got, want)
