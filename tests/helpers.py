"""Shared helpers of the test-suite: seeded synthetic logits and thin wrappers that call the
CUDA sampler through its C ABI (ctypes) with torch tensors as device memory."""
import ctypes as C
import math
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def make_logits(kind, B, V, seed, torch):
    """Seeded CPU-generated fp32 logits (B, V); the same bits everywhere."""
    g = torch.Generator().manual_seed(seed)
    if kind == "uniform":            # example.py:29
        x = torch.rand(B, V, generator=g)
    elif kind == "normal3":          # bench.py logit_type 3
        x = torch.randn(B, V, generator=g) * 3
    elif kind == "uniform4":         # bench.py logit_type 4
        x = torch.rand(B, V, generator=g) * 4
    elif kind == "equal":            # bench.py logit_type 0
        x = torch.zeros(B, V)
    elif kind == "peaked":           # a few boosted ids over N(0, 2^2)
        x = torch.randn(B, V, generator=g) * 2
        for b in range(B):
            idx = torch.randperm(V, generator=g)[:min(32, V)]
            x[b, idx] += 10
    elif kind == "coarse":           # many exact ties: values on a coarse grid
        x = torch.randint(0, 16, (B, V), generator=g).float() * 0.5
    elif kind == "special":          # Inf / NaN entries, sanitised by the kernels (sampling.cu:131-134)
        x = torch.randn(B, V, generator=g)
        n = max(1, V // 97)
        for b in range(B):
            idx = torch.randperm(V, generator=g)[:3 * n]
            x[b, idx[:n]] = float("nan")
            x[b, idx[n:2 * n]] = float("-inf")
            if V > 64:
                x[b, idx[2 * n]] = float("inf")
    else:
        raise ValueError(kind)
    return x.contiguous()


def shape_of(logits, penalties=None):
    V = logits.shape[-1]
    if penalties is not None:
        B = penalties.shape[0] if penalties.dim() == 2 else 1
    else:
        B = logits.shape[0] if logits.dim() >= 2 else 1
    T = logits.shape[1] if logits.dim() == 3 else 1
    return B, T, V


class Abi:
    """C-ABI caller. Every method raises on a non-zero status."""

    def __init__(self):
        import torch
        from rapid_sampling_b200 import abi
        self.torch = torch
        self.abi = abi
        self.L = abi.load()
        self._ws = {}

    def stream(self):
        return C.c_void_p(self.torch.cuda.current_stream().cuda_stream)

    def workspace(self, B, V):
        # always room for the scratch rows, so that every kernel variant can be forced (rs_set_path_override)
        n = max(self.L.rs_workspace_bytes(B, V), 256 + 4 * B * V)
        dev = self.torch.cuda.current_device()
        w = self._ws.get(dev)
        if w is None or w.numel() < n:
            w = self.torch.zeros(n, dtype=self.torch.uint8, device="cuda")
            self._ws[dev] = w
        return w

    def setup_rand(self, seed, B, first_row=0):
        st = self.torch.empty(B * 64, dtype=self.torch.int8, device="cuda")
        rc = self.L.rs_setup_rand(st.data_ptr(), seed & (2 ** 64 - 1), B, first_row, self.stream())
        assert rc == 0, self.abi.status_string(rc)
        return st

    def sample(self, logits, states, temperature, top_k, top_p, penalties=None, presence=0.0, repetition=0.0,
               decay=0.0, debug=False, check=True, want_probs=True):
        torch = self.torch
        B, T, V = shape_of(logits, penalties)
        out = torch.empty(max(B, 0), dtype=torch.int32, device="cuda")
        ws = self.workspace(max(B, 1), max(V, 4))
        pen = penalties.data_ptr() if penalties is not None else None
        if logits.dtype != torch.float32:     # 16-bit logits go through the typed entry point
            dt = {torch.float16: self.abi.RS_DTYPE_F16, torch.bfloat16: self.abi.RS_DTYPE_BF16}[logits.dtype]
            rc = self.L.rs_sample_typed(logits.data_ptr(), dt, B, T, V, pen, states.data_ptr(), out.data_ptr(), temperature,
                                        top_k, top_p, presence, repetition, decay, ws.data_ptr(), ws.numel(), self.stream(),
                                        None, None)
            assert rc == 0, self.abi.status_string(rc)
            return out
        if debug:
            probs = torch.empty(B, V, dtype=torch.float32, device="cuda") if want_probs else None
            trace = torch.zeros(B * C.sizeof(self.abi.Trace), dtype=torch.uint8, device="cuda")
            rc = self.L.rs_sample_debug(logits.data_ptr(), B, T, V, pen, states.data_ptr(), out.data_ptr(), temperature,
                                        top_k, top_p, presence, repetition, decay, ws.data_ptr(), ws.numel(),
                                        self.stream(), probs.data_ptr() if want_probs else None, trace.data_ptr())
        else:
            rc = self.L.rs_sample(logits.data_ptr(), B, T, V, pen, states.data_ptr(), out.data_ptr(), temperature, top_k,
                                  top_p, presence, repetition, decay, ws.data_ptr(), ws.numel(), self.stream())
        if check:
            assert rc == 0, self.abi.status_string(rc) + " " + self.L.rs_last_cuda_error().decode()
        elif rc != 0:
            return rc
        if debug:
            torch.cuda.synchronize()
            tr = (self.abi.Trace * B).from_buffer_copy(trace.cpu().numpy().tobytes())
            return out, probs, tr
        return out

    def device_status(self, B=1, V=4):
        return self.L.rs_device_status(self.workspace(B, V).data_ptr(), self.stream())

    def set_cluster(self, c):
        return self.L.rs_set_cluster_override(c)

    def set_path(self, mode):
        return self.L.rs_set_path_override(mode)


def kept_set_flips_ok(kept32, d, b, mass_tol=1e-6, tie_tol=4e-6):
    """True when every token whose membership differs between the fp32 kept set and the float64
    closed form `d` (oracle.cpu_ref.distribution) lies on the boundary: its float64 cumulative
    mass is within `mass_tol` relative of top_p, or its probability ties with the boundary
    probability within `tie_tol` relative (fp32 rounding of p). Returns (ok, n_flips)."""
    kept64 = d["kept"][b].numpy()
    flips = np.nonzero(kept32 ^ kept64)[0]
    if len(flips) == 0:
        return True, 0
    V = kept64.shape[0]
    order = d["order"][b].numpy()
    cum = d["cum_sorted"][b].numpy()
    rank = np.empty(V, dtype=np.int64)
    rank[order] = np.arange(V)
    p64, v64, top_p = d["probs"][b].numpy(), float(d["v"][b]), d["top_p"]
    r = rank[flips]
    near_mass = np.abs(cum[r] - top_p) <= mass_tol * top_p
    near_mass |= np.abs(cum[np.maximum(r - 1, 0)] - top_p) <= mass_tol * top_p
    near_tie = np.abs(p64[flips] - v64) <= tie_tol * v64
    return bool(np.all(near_mass | near_tie)), len(flips)
