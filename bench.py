#!/usr/bin/env python
"""Benchmark of the sampling hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config C1..C5] [--impl ours|reference|reference-cuda]

A step is ONE sampling call over one batch of synthetic logits.  Default workload (N=1): the
headline shape B=1, V=262144, N(0,3^2) logits, temperature 1, top_k -1, top_p 0.3.  Prints one JSON
line: `value` = rows/s over all GPUs with inputs resident in HBM (each step reads a different row set
from a pool larger than L2), `median_us` = median per-call latency, `e2e` = the same metric through
the torch-facing API with pinned HOST logits (H2D + call + D2H of ids inside the timed region),
`roofline` for the sampler kernel against the measured HBM copy bandwidth, `cpu_baseline` = the
CPU port of the reference timed on the host.

Under torchrun each rank takes the same per-GPU batch (weak scaling); rows are independent, so there
is no collective on the data path -- only the barrier and the max-over-ranks of the timings.
`--impl reference` times the CPU restatement of the reference (the reference has no CPU code of its
own) on rank 0; `--impl reference-cuda` times the reference's own CUDA extension (oracle/_ref) on the
same workload, for the latency comparison against the original kernel.  `--sweep small|full` runs a parameter
sweep in the shape of the reference's own (B x V x top_p x top_k x five distributions) and writes a table.
"""
import argparse
import json
import os
import statistics
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

L2_BYTES = 126 * 1000 * 1000
MIN_LATENCY_CALLS = 1000      # the headline latency is a median over at least this many calls, whatever --steps says
MIN_E2E_STEPS = 200
EXTRA_CALLS = 200             # calls per side for the other workloads reported beside the headline
# Per-launch DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of the sampler kernel, copied from the ncu
# capture named beside it; a workload without a capture of the current kernel has no entry.
PROFILED_TRAFFIC = {"C1": (2.214e6, "profiles/sampler_kernel_C1_C2_C5_cluster.md"),
                    "C2": (1.168e6, "profiles/sampler_kernel_C1_C2_C5_cluster.md"),
                    "C3": (39.02e6, "profiles/sampler_kernel_C3_load_paths.md"),
                    "C4": (219.4e6, "profiles/rowcta_kernel_C4_C3.md"),
                    "C5": (526.6e6, "profiles/sampler_kernel_C1_C2_C5_cluster.md")}


def workload(name):
    """BASELINE configs. Returns dict(B, T, V, temperature, top_k, top_p, rep, dist, seed)."""
    W = {
        "C1": dict(B=4, T=1, V=131072, temperature=1.0, top_k=-1, top_p=0.5, rep=False, dist="uniform", seed=0,
                   desc="example.py: B=4 V=131072 U[0,1) T=1 top_k=-1 top_p=0.5"),
        "C2": dict(B=1, T=1, V=262144, temperature=1.0, top_k=-1, top_p=0.3, rep=False, dist="normal3", seed=1,
                   desc="headline: B=1 V=262144 N(0,3^2) T=1 top_k=-1 top_p=0.3"),
        "C3": dict(B=64, T=1, V=151936, temperature=0.8, top_k=50, top_p=0.9, rep=False, dist="peaked", seed=2,
                   desc="batched decode: B=64 V=151936 N(0,2^2)+10 on 32 ids T=0.8 top_k=50 top_p=0.9"),
        "C4": dict(B=256, T=1, V=65536, temperature=0.8, top_k=50, top_p=0.9, rep=True, dist="normal2.5", seed=3,
                   desc="repetition: B=256 V=65536 N(0,2.5^2) penalties presence=.1 repetition=.1 decay=.95 T=0.8 top_k=50 top_p=0.9"),
        "C5": dict(B=32, T=4, V=1048576, temperature=1.0, top_k=-1, top_p=0.95, rep=False, dist="boosted", seed=4,
                   desc="large vocab: (B,T,V)=(32,4,1048576) N(0,1)+8 on 1% ids T=1 top_k=-1 top_p=0.95"),
    }
    return W[name]


def gen_logits(w, seed, device, torch):
    """One synthetic logits tensor of the workload's shape and distribution, generated on `device`."""
    g = torch.Generator(device=device).manual_seed(seed)
    B, T, V = w["B"], w["T"], w["V"]
    shape = (B, V) if T == 1 else (B, T, V)
    d = w["dist"]
    if d == "uniform":
        return torch.rand(shape, generator=g, device=device)
    x = torch.randn(shape, generator=g, device=device)
    if d == "normal3":
        return x * 3
    if d == "normal2.5":
        return x * 2.5
    if d == "peaked":
        x = x * 2
        idx = torch.rand(B, V, generator=g, device=device).argsort(dim=-1)[:, :32]
        return x.scatter_add_(1, idx, torch.full((B, 32), 10.0, device=device))
    if d == "boosted":
        n = V // 100
        idx = torch.randint(0, V, (B, n), generator=g, device=device)
        boost = torch.zeros(B, V, device=device).scatter_(1, idx, 8.0)
        return x + (boost if T == 1 else boost.unsqueeze(1))
    raise ValueError(d)


class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed regions run (read-only)."""

    def __init__(self, index):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._t = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _run(self):
        nv = self.nv
        names = {"hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
                 "hw_power_brake_slowdown": 0x80}
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for n, bit in names.items():
                    if r & bit:
                        self.reasons.add(n)
            except Exception:
                pass
            time.sleep(0.01)

    def start(self):
        if self.nv:
            self._t = threading.Thread(target=self._run, daemon=True)
            self._t.start()

    def stop(self):
        self._stop.set()
        if self._t:
            self._t.join()
        med = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(self.samples)}


def cpu_port_baseline(w, budget_s=12.0, max_calls=4096):
    """Times the CPU restatement of the reference (oracle/sampler_oracle.c) on this host: whole calls of the
    workload's shape, rows spread over the host cores, until the budget is used."""
    import numpy as np
    import torch
    from oracle import c_oracle as co
    B, V = w["B"], w["V"]
    lg = gen_logits(dict(w, T=1), w["seed"], "cpu", torch).numpy()
    pen = np.zeros((B, V), dtype=np.float32) if w["rep"] else None
    st = co.setup_rand(w["seed"], B)
    cores = min(os.cpu_count() or 1, B)
    co.sample(lg, st, w["temperature"], w["top_k"], w["top_p"], penalties=pen, presence=0.1, repetition=0.1, decay=0.95,
              nthreads=cores)
    t0 = time.perf_counter()
    calls = 0
    while calls < max_calls and time.perf_counter() - t0 < budget_s:
        co.sample(lg, st, w["temperature"], w["top_k"], w["top_p"], penalties=pen, presence=0.1, repetition=0.1,
                  decay=0.95, nthreads=cores)
        calls += 1
    dt = time.perf_counter() - t0
    return {"value": B * calls / dt, "unit": "rows/s", "cores": cores, "kind": "port",
            "sample": "%d whole calls of the workload (%d rows x V=%d each), %.1f s" % (calls, B, V, dt),
            "ms_per_call": dt / calls * 1e3}


def cpu_torch_f64(w, budget_s=6.0, max_calls=16):
    """The same semantics as a float64 torch CPU path (sort + cumsum), for the record."""
    import torch
    from oracle import cpu_ref
    lg = gen_logits(dict(w, T=1), w["seed"], "cpu", torch)
    pen = torch.zeros(w["B"], w["V"]) if w["rep"] else None
    cpu_ref.sample(lg, w["temperature"], w["top_k"], w["top_p"], pen, 0.1, 0.1, 0.95)
    t0 = time.perf_counter()
    calls = 0
    while calls < max_calls and time.perf_counter() - t0 < budget_s:
        cpu_ref.sample(lg, w["temperature"], w["top_k"], w["top_p"], pen, 0.1, 0.1, 0.95)
        calls += 1
    dt = time.perf_counter() - t0
    return {"rows_per_s": w["B"] * calls / dt, "ms_per_call": dt / calls * 1e3, "threads": torch.get_num_threads(),
            "cpu_count": os.cpu_count()}


def hbm_peak():
    """Measured HBM copy bandwidth of this pool's B200s (GB/s) when the driver's file is present, else the fallback."""
    try:
        return float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def alg_bytes(w, esz=4):
    """Algorithmic bytes of one call: logits of the read position once, plus fp32 penalties read and written."""
    return ((8 if w["rep"] else 0) + esz) * w["V"] * w["B"]


def make_pool(w, dev, torch, rank=0, min_sets=2, max_sets=256):
    """Logits sets that together exceed L2, so that consecutive calls read their rows from HBM."""
    row_bytes = w["B"] * w["T"] * w["V"] * 4
    n = max(min_sets, min(max_sets, -(-int(1.6 * L2_BYTES) // row_bytes)))
    return [gen_logits(w, w["seed"] + 1000 * i + 7 * rank, dev, torch) for i in range(n)]


def sampler_call(ext, w, states, pen):
    if w["rep"]:
        return lambda lg: ext.batch_sampling_repetition_temperature_topk_topp(lg, pen, states, 0.1, 0.1, 0.95, w["temperature"],
                                                                              w["top_k"], w["top_p"])
    return lambda lg: ext.batch_sampling_temperature_topk_topp(lg, states, w["temperature"], w["top_k"], w["top_p"])


def graph_of_calls(call, pool, n, torch):
    """n calls recorded into one CUDA graph (after three calls on the capture stream, so that the stream's workspace
    exists); None if the capture fails."""
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            for i in range(3):
                call(pool[i % len(pool)])
        torch.cuda.current_stream().wait_stream(side)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        keep = []
        with torch.cuda.graph(g, stream=side):
            for i in range(n):
                keep.append(call(pool[i % len(pool)]))
        g.replay()
        torch.cuda.synchronize()
        g._keep = keep
        return g
    except Exception:   # noqa: BLE001
        return None


def time_calls(call, pool, n, torch, warm=5, graph=False):
    """(ms per call over n back-to-back calls -- one replay of a CUDA graph of the n calls if `graph` --, median us of
    per-call event pairs)."""
    for i in range(warm):
        call(pool[i % len(pool)])
    torch.cuda.synchronize()
    g = graph_of_calls(call, pool, n, torch) if graph else None
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if g is not None:
        g.replay()
    else:
        for i in range(n):
            call(pool[i % len(pool)])
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / n
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    for i in range(n):
        evs[i][0].record()
        call(pool[i % len(pool)])
        evs[i][1].record()
    torch.cuda.synchronize()
    lat = sorted(x.elapsed_time(y) * 1e3 for x, y in evs)
    return ms, lat[len(lat) // 2]


def reference_cuda_on(ref, w, pool, n, torch):
    """The reference's own CUDA kernel (oracle/_ref) on the same logits; 3-D workloads give it the last position only
    (it indexes its (B, V) scratch with the 3-D offset, sampling.cu:488 against :206)."""
    if w["T"] != 1:
        pool = [x[:, -1, :].contiguous() for x in pool]
        w = dict(w, T=1)
    pen = torch.zeros(w["B"], w["V"], device=pool[0].device) if w["rep"] else None
    st = ref.setup_rand(w["seed"], w["B"])
    ms, med = time_calls(sampler_call(ref, w, st, pen), pool, n, torch)
    return {"median_us": med, "ms_per_call": ms, "rows_per_s": w["B"] / (ms * 1e-3)}


def ids_equal_to_reference(ext, ref, w, pool, torch, calls=3):
    """Same states, same logits: the ids of `calls` consecutive calls must be identical to the reference kernel's."""
    from rapid_sampling_b200.sharding import setup_rand_rows
    dev = pool[0].device
    st_o, st_r = setup_rand_rows(w["seed"], 0, w["B"]), ref.setup_rand(w["seed"], w["B"])
    pen_o = torch.zeros(w["B"], w["V"], device=dev) if w["rep"] else None
    pen_r = torch.zeros(w["B"], w["V"], device=dev) if w["rep"] else None
    co, cr = sampler_call(ext, w, st_o, pen_o), sampler_call(ref, dict(w, T=1), st_r, pen_r)
    ok = True
    for i in range(calls):
        lg = pool[i % len(pool)]
        ok = ok and bool(torch.equal(co(lg), cr(lg if w["T"] == 1 else lg[:, -1, :].contiguous())))
    return ok and bool(torch.equal(st_o, st_r)) and (pen_o is None or bool(torch.equal(pen_o, pen_r)))


def other_workloads(ext, ref, dev, torch, names=("C1", "C3", "C4", "C5")):
    """The workloads that are not the headline, each timed over EXTRA_CALLS calls beside the reference's CUDA kernel
    on the same logits (one GPU).  Reported as extra keys of the headline's line, outside its timed region."""
    from rapid_sampling_b200.sharding import setup_rand_rows
    peak, _ = hbm_peak()
    out = {}
    for name in names:
        w = workload(name)
        pool = make_pool(w, dev, torch, max_sets=(2 if name == "C5" else 256))
        pen = torch.zeros(w["B"], w["V"], device=dev) if w["rep"] else None
        st = setup_rand_rows(w["seed"], 0, w["B"])
        ms, med = time_calls(sampler_call(ext, w, st, pen), pool, EXTRA_CALLS, torch, graph=True)
        row = {"median_us": med, "ms_per_call": ms, "rows_per_s": w["B"] / (ms * 1e-3), "calls": EXTRA_CALLS,
               "roofline_frac": alg_bytes(w) / (ms * 1e-3) / 1e9 / peak, "algorithmic_bytes": alg_bytes(w)}
        if ref is not None:
            r = reference_cuda_on(ref, w, pool, EXTRA_CALLS, torch)
            row.update(reference_cuda_median_us=r["median_us"], speedup_vs_reference_cuda=r["median_us"] / med,
                       ids_equal=ids_equal_to_reference(ext, ref, w, pool, torch))
        else:
            row["reference_cuda_median_us"] = None
        out[name] = row
        del pool, pen
        torch.cuda.empty_cache()
    return out


def multi_gpu_extras(ext, rank, world, dev, torch, dist, calls=100):
    """What only a multi-GPU run can show, measured after the headline on every rank (rank 0 reports): C3 and C4
    batch-sharded with the same per-GPU batch (weak) and with the batch divided over the ranks (strong), and C5
    vocab-parallel with the ids checked to be identical on all ranks."""
    from rapid_sampling_b200.sharding import row_range, setup_rand_rows
    from rapid_sampling_b200.vocab_parallel import VocabParallelSampler

    def max_over_ranks(x):
        t = torch.tensor([x], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0])
    out = {}
    for name in ("C3", "C4"):
        w = workload(name)
        for mode in ("weak", "strong"):
            if mode == "weak":
                wl, first = w, rank * w["B"]
            else:
                a0, a1 = row_range(w["B"], rank, world)
                wl, first = dict(w, B=a1 - a0), a0
            if wl["B"] == 0:
                continue
            pool = make_pool(wl, dev, torch, rank=rank)
            pen = torch.zeros(wl["B"], wl["V"], device=dev) if wl["rep"] else None
            st = setup_rand_rows(w["seed"], first, wl["B"])
            call = sampler_call(ext, wl, st, pen)
            for i in range(5):
                call(pool[i % len(pool)])
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            g = graph_of_calls(call, pool, calls, torch)     # the timed region holds the launches, not the host's loop
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            if g is not None:
                g.replay()
            else:
                for i in range(calls):
                    call(pool[i % len(pool)])
            e1.record()
            torch.cuda.synchronize()
            mine = e0.elapsed_time(e1) / calls
            ms = max_over_ranks(mine)
            fastest = -max_over_ranks(-mine)
            del g
            total_rows = w["B"] * world if mode == "weak" else w["B"]
            out["%s_%s" % (name, mode)] = {"rows_per_gpu": wl["B"], "total_rows": total_rows, "ms_per_call": ms,
                                           "ms_per_call_fastest_rank": fastest,
                                           "rows_per_s": total_rows / (ms * 1e-3), "collectives_on_data_path": 0}
            del pool, pen
            torch.cuda.empty_cache()
    # C5 vocab-parallel: V / world columns per rank, NCCL collectives between the stages
    w = workload("C5")
    B, T, V = w["B"], w["T"], w["V"]
    s = VocabParallelSampler(B, V, rank, world, T=T)
    pool = []
    for i in range(2):
        full = gen_logits(dict(w, T=1), w["seed"] + 1000 * i, dev, torch)          # the same rows on every rank (same seed)
        shard = full[:, s.col0:s.col0 + s.V_local]
        pool.append(shard.unsqueeze(1).expand(B, T, s.V_local).contiguous())
        del full
    st = setup_rand_rows(w["seed"], 0, B)
    ids = None
    for i in range(5):
        ids = s.sample(pool[i % 2], st, w["temperature"], w["top_k"], w["top_p"])
    chk = ids.to(torch.int64).sum().reshape(1)
    lo, hi = chk.clone(), chk.clone()
    dist.all_reduce(lo, op=dist.ReduceOp.MIN)
    dist.all_reduce(hi, op=dist.ReduceOp.MAX)

    def timed(n, check_every_call):
        s.defer_check = not check_every_call
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(n):
            s.sample(pool[i % 2], st, w["temperature"], w["top_k"], w["top_p"])
        e1.record()
        torch.cuda.synchronize()
        bad = s.validate() is not None
        return max_over_ranks(e0.elapsed_time(e1)) / n, bad
    ms_sync, _ = timed(calls, True)          # the host reads the device's validity flag after every call
    ms, redone = timed(calls, False)         # the flag is read when the ids are (here: after the last call)
    out["C5_vocab_parallel"] = {"columns_per_gpu": s.V_local, "ms_per_call": ms, "ms_per_call_host_check_every_call": ms_sync,
                                "rows_per_s": B / (ms * 1e-3), "protocol": s.last_protocol, "last_call_repeated": redone,
                                "ids_identical_on_all_ranks": bool(int(lo[0]) == int(hi[0])),
                                "collectives_per_call": "2 all-reduces + 1 all-gather (NCCL)"}
    s.release_graphs()
    return out


def bench_vocab_parallel(a, w, rank, local_rank, world, dev, base, K, Wm, torch, dist):
    """Strong scaling over the vocabulary: the batch is fixed, every rank streams V/N columns of every row and the
    cutoff search is reduced over NVLink (13 small NCCL collectives per call)."""
    from rapid_sampling_b200.sharding import setup_rand_rows
    from rapid_sampling_b200.vocab_parallel import VocabParallelSampler
    B, T, V = w["B"], w["T"], w["V"]
    s = VocabParallelSampler(B, V, rank, world, T=T, graph=a.vp_graph)
    pool_n = 2 if V * B * T * 4 // world > 256 * 2 ** 20 else 4
    pool = []
    for i in range(pool_n):   # the same full tensor on every rank (same seed), sliced: shards of one logical row set
        full = gen_logits(dict(w, T=1), w["seed"] + 1000 * i, dev, torch)
        shard = full[:, s.col0:s.col0 + s.V_local]
        pool.append((shard.unsqueeze(1).expand(B, T, s.V_local).contiguous() if T > 1 else shard.contiguous()))
        del full
    states = setup_rand_rows(w["seed"], 0, B)
    pen = torch.zeros(B, s.V_local, device=dev) if w["rep"] else None

    def call(lg):
        return s.sample(lg, states, w["temperature"], w["top_k"], w["top_p"], penalties=pen, presence_penalty=0.1,
                        repetition_penalty=0.1, penalty_decay=0.95)
    for i in range(max(Wm, 2 * pool_n + 1) if a.vp_graph else Wm):   # a graph per buffer: one eager call, one recording
        call(pool[i % pool_n])
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = ClockSampler(local_rank)
    clocks.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for i in range(K):
        call(pool[i % pool_n])
    e1.record()
    torch.cuda.synchronize()
    total_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t[0])
    clk = clocks.stop()
    if rank == 0:
        ms = total_ms / K
        alg = 4 * V * B            # logits of the read position, once, over all shards
        peak = 6650.0
        try:
            peak = float(json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"])
        except Exception:
            pass
        ach = alg / (ms * 1e-3) / 1e9
        line = dict(base, impl="ours", scaling="strong", value=B * K / (total_ms * 1e-3), ms_per_step=ms, median_us=ms * 1e3,
                    clocks=clk, gpu_launches=K * (6 if s.last_protocol == "fast" else 19), protocol=s.last_protocol + ("+graph" if a.vp_graph else ""),
                    roofline={"bound": "hbm", "kernel": "vpf_* stage kernels (fast protocol: 3 passes over the shard, 3 collectives)", "achieved": ach,
                              "peak": peak * world, "unit": "GB/s", "frac": ach / (peak * world),
                              "algorithmic_bytes_per_launch": alg, "traffic": None,
                              "note": "latency-bound: collectives and one host check per call"})
        line["config"]["parallelism"] = "vocab-parallel x%d (V/N = %d columns per GPU; NCCL: 2 all-reduces + 1 all-gather per call)" % (world, V // world)
        print(json.dumps(line), flush=True)
    s.release_graphs()      # recorded graphs must be gone before NCCL shuts its communicator down
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


SWEEP_GRIDS = {
    # the reference's own grid (bench.py:32-35): 12000 combinations
    "full": dict(B=[512, 256, 128, 64, 32, 16, 8, 4, 2, 1], V=[262144, 151936, 131072, 100256, 65536, 50304, 32768, 256],
                 p=[0.1, 0.3, 0.7, 0.9, 1], k=[-1, 1, 10, 100, 1000, 10000]),
    # a cut through it that finishes in about a minute
    "small": dict(B=[128, 16, 1], V=[262144, 151936, 32768, 256], p=[0.1, 0.9, 1], k=[-1, 1, 100, 10000]),
}


def sweep_logits(kind, B, V, dev, torch):
    """The five synthetic distributions of the reference's sweep (bench.py:66-72)."""
    if kind == 0:
        return torch.zeros(B, V, dtype=torch.float32, device=dev)
    if kind == 1:
        return torch.rand(B, V, dtype=torch.float32, device=dev)
    if kind == 2:
        return torch.randn(B, V, dtype=torch.float32, device=dev) / 2
    if kind == 3:
        return torch.randn(B, V, dtype=torch.float32, device=dev) * 3
    return torch.rand(B, V, dtype=torch.float32, device=dev) * 4


def run_sweep(a):
    """Breadth run in the shape of the reference's sweep: B x V x top_p x top_k x 5 distributions, 5 repetitions each,
    per-call wall time with a synchronise on both sides (the reference's method, bench.py:73-92), median.  Where the
    reference's CUDA kernel is available it is timed on the same logits and its ids are compared with ours."""
    import torch
    import rapid_sampling_b200 as rs
    from oracle import build_ref
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    ext = rs._load_ext()
    ref = build_ref.load_ref()
    g = SWEEP_GRIDS[a.sweep]
    torch.manual_seed(0)
    rows, mismatched = [], 0

    def timed(f):
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        out = f()
        torch.cuda.synchronize()
        return out, (time.perf_counter() - t0) * 1e6
    for V in g["V"]:
        for B in g["B"]:
            for p in g["p"]:
                for k in g["k"]:
                    for kind in range(5):
                        st_o = ext.setup_rand(0, B)
                        st_r = ref.setup_rand(0, B) if ref is not None else None
                        t_o, t_r, bad = [], [], 0
                        for _ in range(5):
                            lg = sweep_logits(kind, B, V, dev, torch)
                            out_o, dt = timed(lambda: ext.batch_sampling_temperature_topk_topp(lg, st_o, 1.0, k, float(p)))
                            t_o.append(dt)
                            if ref is not None:
                                out_r, dt = timed(lambda: ref.batch_sampling_temperature_topk_topp(lg, st_r, 1.0, k, float(p)))
                                t_r.append(dt)
                                bad += int((out_o != out_r).sum().item())
                        mismatched += bad
                        rows.append({"B": B, "V": V, "top_p": p, "top_k": k, "logit_type": kind,
                                     "ours_us": float(np.median(t_o)),
                                     "reference_cuda_us": float(np.median(t_r)) if t_r else None, "ids_differ": bad})
    with open(a.sweep_out, "w") as f:
        json.dump(rows, f)
    line = {"sweep": a.sweep, "combinations": len(rows), "repetitions": 5, "ours_median_us": float(np.median([r["ours_us"] for r in rows])),
            "results_file": a.sweep_out}
    if ref is not None:
        ratio = np.array([r["reference_cuda_us"] / r["ours_us"] for r in rows])
        line.update(reference_cuda_median_us=float(np.median([r["reference_cuda_us"] for r in rows])),
                    speedup_geomean=float(np.exp(np.log(ratio).mean())), speedup_min=float(ratio.min()),
                    speedup_max=float(ratio.max()), ids_differ=mismatched)
    print(json.dumps(line))
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--config", default="C2", choices=["C1", "C2", "C3", "C4", "C5"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "reference-cuda"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--eager", action="store_true", help="time the plain Python launch loop instead of one replay of a CUDA graph of the K calls")
    ap.add_argument("--ordinary-launch", action="store_true",
                    help="launch the sampler kernels without programmatic stream serialization (rs_set_dependent_launch(0))")
    ap.add_argument("--path-mode", type=int, default=0, choices=[0, 1, 2, 3, 4, 5, 6],
                    help="force a kernel variant (rs_set_path_override): 1 whole-row search, 2 streaming cluster, 3 on-chip cluster, "
                         "4 one CTA per row; for profiling one variant on a workload the planner would give to another")
    ap.add_argument("--per-row", action="store_true", help="ours only: per-row temperature / top_k / top_p tensors (rs_sample_rows)")
    ap.add_argument("--no-extras", action="store_true",
                    help="only the headline workload: skip the reference-CUDA arm, the other workloads and the multi-GPU extras")
    ap.add_argument("--dtype", default="f32", choices=["f32", "f16", "bf16"], help="storage type of the logits (ours only)")
    ap.add_argument("--vp", action="store_true", help="vocab-parallel: every rank holds V/N columns of every row")
    ap.add_argument("--vp-graph", action="store_true", help="vocab-parallel: replay the stages from a CUDA graph per input buffer")
    ap.add_argument("--sweep", choices=sorted(SWEEP_GRIDS), help="run the reference-shaped parameter sweep instead (one GPU)")
    ap.add_argument("--sweep-out", default="sweep_results.json")
    a = ap.parse_args()
    if a.sweep:
        run_sweep(a)
        return
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    w = workload(a.config)
    K, Wm = max(a.steps, 1), max(a.warmup, 3)
    B, T, V = w["B"], w["T"], w["V"]
    base = {"metric": "rows_per_s", "unit": "rows/s", "n_gpus": world, "steps": K, "warmup": Wm,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": a.config + " " + w["desc"], "rows_per_gpu": B, "parallelism": "batch-sharded x%d" % world}}

    if a.impl == "reference":
        # CPU arm: the reference ships no CPU implementation, so this is the CPU restatement (oracle port).
        if rank != 0:
            return
        cb = cpu_port_baseline(w, budget_s=max(5.0, min(60.0, 0.05 * K)), max_calls=K)
        line = dict(base, impl="reference", value=cb["value"], ms_per_step=cb["ms_per_call"], n_gpus=world,
                    cpu_baseline=cb, gpu_launches=0,
                    e2e={"value": cb["value"], "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0})
        line["config"]["parallelism"] = "host cores (%d threads)" % cb["cores"]
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    if a.vp:
        return bench_vocab_parallel(a, w, rank, local_rank, world, dev, base, K, Wm, torch, dist)

    if a.impl == "ours":
        import rapid_sampling_b200 as rs
        from rapid_sampling_b200.sharding import setup_rand_rows
        ext = rs._load_ext()
        states = setup_rand_rows(w["seed"], rank * B, B)
        launches = ext.kernel_launch_count
    else:
        from oracle import build_ref
        ext = build_ref.load_ref()
        if ext is None:
            if rank == 0:
                print(json.dumps({"impl": "reference-cuda", "unavailable": "oracle/_ref was not built"}))
            return
        if T != 1:
            w = dict(w, T=1)   # the reference kernel writes out of bounds for 3-D input: feed it the last slice
            T = 1
        states = ext.setup_rand(w["seed"], B)
        launches = lambda: 0  # noqa: E731

    # input pool larger than L2 so that every step reads its logits from HBM
    esz = 4 if (a.impl != "ours" or a.dtype == "f32") else 2
    row_bytes = B * T * V * esz
    pool_n = max(2, min(256, -(-int(1.6 * L2_BYTES) // row_bytes)))
    if a.config == "C5":
        pool_n = 2
    tdt = {"f32": torch.float32, "f16": torch.float16, "bf16": torch.bfloat16}[a.dtype if a.impl == "ours" else "f32"]
    pool = [gen_logits(w, w["seed"] + 1000 * i + 7 * rank, dev, torch).to(tdt) for i in range(pool_n)]
    pen = torch.zeros(B, V, device=dev) if w["rep"] else None

    lowp = (a.impl == "ours" and a.dtype != "f32")
    f_plain = ext.batch_sampling_temperature_topk_topp_any if lowp else ext.batch_sampling_temperature_topk_topp
    f_rep = ext.batch_sampling_repetition_temperature_topk_topp_any if lowp else ext.batch_sampling_repetition_temperature_topk_topp

    if a.impl == "ours" and a.ordinary_launch:
        from rapid_sampling_b200 import abi
        abi.load().rs_set_dependent_launch(0)
        base["config"]["ordinary_launch"] = True
    if a.impl == "ours" and a.path_mode:
        from rapid_sampling_b200 import abi
        abi.load().rs_set_path_override(a.path_mode)
        base["config"]["path_mode"] = a.path_mode
    if a.impl == "ours" and a.per_row:
        t_row = torch.full((B,), w["temperature"], device=dev, dtype=torch.float32)
        k_row = torch.full((B,), w["top_k"], device=dev, dtype=torch.int32)
        p_row = torch.full((B,), w["top_p"], device=dev, dtype=torch.float32)
        base["config"]["per_row_parameters"] = True

    def call(lg):
        if a.impl == "ours" and a.per_row:
            return ext.batch_sampling_rows(lg, states, t_row, k_row, p_row, penalties=pen, presence_penalty=0.1,
                                           repetition_penalty=0.1, penalty_decay=0.95)
        if w["rep"]:
            return f_rep(lg, pen, states, 0.1, 0.1, 0.95, w["temperature"], w["top_k"], w["top_p"])
        return f_plain(lg, states, w["temperature"], w["top_k"], w["top_p"])

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    for i in range(Wm):
        call(pool[i % pool_n])
    sync_all()
    clocks = ClockSampler(local_rank)
    clocks.start()

    # ---- timed region: exactly K steps, device-timed, max over ranks -------------------------------
    # The K calls are recorded once into a CUDA graph and replayed: the timed region then holds the K sampler launches
    # and nothing of the host (with several ranks on one host the Python launch loops compete for its cores).
    # --eager, the reference kernel, or a failed capture time the plain loop instead.
    graph = None
    n0 = launches()
    if a.impl == "ours" and not a.eager:
        try:
            side = torch.cuda.Stream(device=dev)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for i in range(3):      # the stream's workspace exists before the capture starts
                    call(pool[i % pool_n])
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            n0 = launches()
            graph = torch.cuda.CUDAGraph()
            keep = []
            with torch.cuda.graph(graph, stream=side):
                for i in range(K):
                    keep.append(call(pool[i % pool_n]))
            captured = launches() - n0
            graph.replay()              # one untimed replay
            torch.cuda.synchronize()
        except Exception as exc:        # noqa: BLE001 -- any capture problem: time the plain loop
            graph = None
            base["config"]["graph_capture_failed"] = repr(exc)[:200]
            n0 = launches()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sync_all()
    e0.record()
    if graph is not None:
        graph.replay()
    else:
        for i in range(K):
            call(pool[i % pool_n])
    e1.record()
    torch.cuda.synchronize()
    gpu_launches = captured if graph is not None else launches() - n0
    base["config"]["launch"] = ("one replay of a CUDA graph holding the %d calls" % K) if graph is not None else "eager loop"
    total_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([total_ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t[0])

    # ---- per-call latency (median), events around every call --------------------------------------
    nlat = max(K, MIN_LATENCY_CALLS) if a.impl == "ours" else max(min(K, MIN_LATENCY_CALLS), 200)
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(nlat)]
    for i in range(nlat):
        evs[i][0].record()
        call(pool[i % pool_n])
        evs[i][1].record()
    torch.cuda.synchronize()
    lat = sorted(x.elapsed_time(y) * 1e3 for x, y in evs)
    median_us = lat[len(lat) // 2]
    # wall-clock per call with a sync, the reference bench's own method (bench.py:73-92)
    nw = max(min(K, 1000), 200)
    walls = []
    for i in range(nw):
        t0 = time.perf_counter()
        call(pool[i % pool_n])
        torch.cuda.synchronize()
        walls.append((time.perf_counter() - t0) * 1e6)
    wall_median_us = statistics.median(walls)

    # ---- end to end: pinned host logits -> device -> call -> ids back on the host ------------------
    host_n = max(2, min(8, pool_n))
    last = (lambda x: x) if T == 1 else (lambda x: x[:, -1, :].contiguous())   # only position T-1 is ever read
    host_pool = [last(pool[i]).cpu().pin_memory() for i in range(host_n)]
    e2e = None
    if host_pool is not None:
        stage = torch.empty(B, V, device=dev, dtype=tdt)
        ke = max(min(K, 1000), MIN_E2E_STEPS)

        def e2e_step(i):
            stage.copy_(host_pool[i % host_n], non_blocking=True)
            return call(stage).cpu()
        for i in range(3):
            e2e_step(i)
        sync_all()
        t0 = time.perf_counter()
        for i in range(ke):
            e2e_step(i)
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t[0])
        e2e = {"value": world * B * ke / dt, "unit": "rows/s", "h2d_bytes_per_step": B * V * esz, "d2h_bytes_per_step": 4 * B,
               "steps": ke, "ms_per_step": dt / ke * 1e3, "api": "torch: pinned tensor -> copy_ -> sampling call -> .cpu()"}
        if a.impl == "ours" and a.dtype == "f32" and not a.per_row:
            # the same step through the C ABI's host-buffer entry point: one call copies the pinned host logits in,
            # samples, copies the ids back and synchronises the stream
            import ctypes as C
            from rapid_sampling_b200 import abi as rs_abi
            L = rs_abi.load()
            wsb = max(int(L.rs_workspace_bytes(B, V)), 256 + 4 * B * V)
            ws = torch.zeros(wsb, dtype=torch.uint8, device=dev)
            out_dev = torch.empty(B, dtype=torch.int32, device=dev)
            out_host = torch.empty(B, dtype=torch.int32).pin_memory()
            stream_h = C.c_void_p(torch.cuda.current_stream().cuda_stream)
            pen_ptr = pen.data_ptr() if pen is not None else None

            def host_step(i):
                rc = L.rs_sample_host(host_pool[i % host_n].data_ptr(), B, 1, V, pen_ptr, states.data_ptr(), out_host.data_ptr(),
                                      float(w["temperature"]), int(w["top_k"]), float(w["top_p"]), 0.1, 0.1, 0.95,
                                      stage.data_ptr(), out_dev.data_ptr(), ws.data_ptr(), wsb, stream_h)
                if rc != 0:
                    raise RuntimeError("rs_sample_host: %s" % rs_abi.status_string(rc))
            for i in range(3):
                host_step(i)
            sync_all()
            t0 = time.perf_counter()
            for i in range(ke):
                host_step(i)
            dt_c = time.perf_counter() - t0
            if world > 1:
                t = torch.tensor([dt_c], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                dt_c = float(t[0])
            e2e = {"value": world * B * ke / dt_c, "unit": "rows/s", "h2d_bytes_per_step": B * V * 4, "d2h_bytes_per_step": 4 * B,
                   "steps": ke, "ms_per_step": dt_c / ke * 1e3,
                   "api": "rs_sample_host (C ABI): pinned host logits in, ids out on the host, stream synchronised, per call",
                   "torch_api": {"value": world * B * ke / dt, "ms_per_step": dt / ke * 1e3}}
    clk = clocks.stop()

    # ---- beside the headline, outside its timed region --------------------------------------------------
    extras = {}
    if a.impl == "ours" and not a.no_extras and a.dtype == "f32" and not a.path_mode and not a.per_row:
        del host_pool
        if world > 1:
            extras["multi_gpu"] = multi_gpu_extras(ext, rank, world, dev, torch, dist)
        elif rank == 0:
            from oracle import build_ref
            ref = build_ref.load_ref()
            if ref is not None:
                extras["reference_cuda"] = dict(reference_cuda_on(ref, w, pool, max(min(K, 1000), 200), torch),
                                                what="the reference's own CUDA kernel (compiled unmodified) on the same logits pool")
            else:
                extras["reference_cuda"] = {"unavailable": "oracle/_ref was not built (needs the reference sources at build time)"}
            del pool
            torch.cuda.empty_cache()
            extras["configs"] = other_workloads(ext, ref, dev, torch, names=[c for c in ("C1", "C2", "C3", "C4", "C5") if c != a.config])

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    ms_per_step = total_ms / K
    alg_bytes = ((8 if w["rep"] else 0) + esz) * V * B     # logits read once (+ fp32 penalties read + write)
    peak, peak_src = hbm_peak()
    achieved = alg_bytes / (ms_per_step * 1e-3) / 1e9
    base["dtype"] = "f32" if esz == 4 else a.dtype + " logits, fp32 arithmetic"
    line = dict(base, impl=a.impl, value=world * B * K / (total_ms * 1e-3), ms_per_step=ms_per_step,
                median_us=median_us, p10_us=lat[len(lat) // 10], p90_us=lat[(len(lat) * 9) // 10],
                wall_sync_median_us=wall_median_us, clocks=clk, e2e=e2e, gpu_launches=int(gpu_launches),
                roofline={"bound": "hbm", "kernel": "sampler_kernel", "achieved": achieved, "peak": peak, "unit": "GB/s",
                          "frac": achieved / peak, "peak_source": peak_src + " HBM copy bandwidth",
                          "algorithmic_bytes_per_launch": alg_bytes, "traffic": PROFILED_TRAFFIC.get(a.config, (None, None))[0],
                          "traffic_source": PROFILED_TRAFFIC.get(a.config, (None, None))[1]})
    line.update(extras)
    line["latency_calls"] = nlat
    line["config"]["l2"] = "inputs rotate through a pool of %d logits sets (%.0f MB > L2)" % (pool_n, pool_n * row_bytes / 1e6)
    if a.impl == "ours" and not a.no_cpu_baseline:
        line["cpu_baseline"] = cpu_port_baseline(w)
        line["cpu_torch_f64"] = cpu_torch_f64(w)
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
