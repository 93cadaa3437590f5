"""Generates tests/golden/ref_vectors.npz by running the REFERENCE's own CUDA extension
(oracle/_ref, built by oracle/build_ref.py from the unmodified reference sources) on a B200.

    python tests/golden/make_golden.py --out <dir>

What is stored (all small):
  rng_*      state bytes straight from the reference's setup_rand, and after n sampling calls
  case_*     for each seeded case: the reference's sampled ids for 2 consecutive calls, a checksum of
             the regenerated logits, and which rows the C oracle (libm exp2f) reproduces from logits
  small_*    for small rows additionally the logits, the fp32 probabilities the kernels searched on
             (dumped by this repository's kernel, after checking that its ids equal the reference's)
             and the per-row trace, so that the CPU tests can pin the oracle's post-softmax
             arithmetic bit for bit
  chain_*    16 chained repetition-penalty calls: ids per step and the final penalties
The CPU test-suite (tests/test_oracle_golden.py) replays these without a GPU.
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

from helpers import Abi, make_logits  # noqa: E402
from oracle import build_ref, c_oracle as co  # noqa: E402

CASES = [  # name, kind, B, V, temperature, top_k, top_p, seed
    ("example", "uniform", 4, 131072, 1.0, -1, 0.5, 0),
    ("headline", "normal3", 1, 262144, 1.0, -1, 0.3, 1),
    ("decode", "peaked", 8, 151936, 0.8, 50, 0.9, 2),
    ("ties", "coarse", 8, 4096, 0.9, 7, 0.6, 9),
    ("equal", "equal", 4, 256, 1.0, -1, 0.5, 7),
    ("special", "special", 4, 50304, 1.3, 100, 0.9, 11),
    ("nofilter", "uniform", 4, 100256, 1.0, -1, 1.0, 12),
    ("greedy", "uniform", 4, 100256, 1.0, 1, 0.0, 13),
    ("hot", "normal3", 4, 65536, 1000.0, 1000, 0.9, 15),
    ("tiny", "uniform", 4, 4, 1.0, -1, 0.5, 6),
]
SMALL = [
    ("s_topp", "uniform", 4, 2048, 1.0, -1, 0.5, 101),
    ("s_topk", "normal3", 4, 4096, 0.8, 50, 0.9, 102),
    ("s_ties", "coarse", 4, 1024, 0.9, 7, 0.6, 103),
    ("s_ragged", "peaked", 4, 2052, 0.7, 20, 0.95, 104),
]


def checksum(x):
    b = x.contiguous().view(torch.int32).to(torch.int64)
    return np.array([int(b.sum()), int((b * torch.arange(1, b.numel() + 1).view_as(b) % 1000003).sum())], dtype=np.int64)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    os.makedirs(a.out, exist_ok=True)
    ref = build_ref.load_ref()
    assert ref is not None, "oracle/_ref is not built"
    abi = Abi()
    g = {}
    for i, (seed, B) in enumerate([(0, 4), (1234567890123, 3), (-7, 2)]):
        st = ref.setup_rand(seed, B)
        g["rng_%d_seed" % i] = np.array([seed], dtype=np.int64)
        g["rng_%d_init" % i] = st.cpu().numpy()
        lg = make_logits("uniform", B, 1024, 0, torch).cuda()
        for _ in range(3):
            ref.batch_sampling_temperature_topk_topp(lg, st, 1.0, -1, 0.5)
        g["rng_%d_after3" % i] = st.cpu().numpy()
    for name, kind, B, V, temp, k, p, seed in CASES + SMALL:
        lg = make_logits(kind, B, V, seed, torch)
        st_ref, st_our = ref.setup_rand(seed, B), abi.setup_rand(seed, B)
        st_cpu = st_ref.cpu().numpy().copy()
        ids = []
        for call in range(2):
            r = ref.batch_sampling_temperature_topk_topp(lg.cuda(), st_ref, temp, k, p)
            if call == 0:
                o, probs, tr = abi.sample(lg.cuda(), st_our, temp, k, p, debug=True)
            else:
                o = abi.sample(lg.cuda(), st_our, temp, k, p)
            assert torch.equal(o, r), name
            ids.append(r.cpu().numpy())
        ids = np.stack(ids)
        oracle_ids = np.stack([co.sample(lg.numpy(), st_cpu, temp, k, p) for _ in range(2)])
        pre = ("small_" if name.startswith("s_") else "case_") + name
        g[pre + "_params"] = np.array([B, V, k, seed], dtype=np.int64)
        g[pre + "_fparams"] = np.array([temp, p], dtype=np.float64)
        g[pre + "_kind"] = np.array(kind)
        g[pre + "_ids"] = ids
        g[pre + "_logits_checksum"] = checksum(lg)
        g[pre + "_oracle_match"] = (oracle_ids == ids)
        if name.startswith("s_"):
            g[pre + "_logits"] = lg.numpy()
            g[pre + "_probs"] = probs.cpu().numpy()
            g[pre + "_trace"] = np.frombuffer(bytes(tr), dtype=np.uint8).copy()
        print(name, "ids", ids[0][:4], "oracle-from-logits match", float((oracle_ids == ids).mean()), flush=True)
    # chained repetition calls
    B, V = 8, 4096
    pen = torch.zeros(B, V, device="cuda")
    st = ref.setup_rand(3, B)
    steps = []
    for step in range(16):
        lg = (torch.randn(B, V, generator=torch.Generator().manual_seed(3 + step)) * 2.5).cuda()
        steps.append(ref.batch_sampling_repetition_temperature_topk_topp(lg, pen, st, 0.1, 0.1, 0.95, 0.8, 50, 0.9).cpu().numpy())
    g["chain_ids"] = np.stack(steps)
    g["chain_penalties"] = pen.cpu().numpy()
    g["chain_states"] = st.cpu().numpy()
    g["torch_version"] = np.array(torch.__version__)
    np.savez_compressed(os.path.join(a.out, "ref_vectors.npz"), **g)
    print("wrote", os.path.join(a.out, "ref_vectors.npz"))


if __name__ == "__main__":
    main()
