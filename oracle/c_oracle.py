"""ctypes front end of ``sampler_oracle.c`` (the fp32 order-faithful CPU restatement).

TEST INFRASTRUCTURE ONLY.  Builds ``librs_oracle.so`` next to the source with gcc on first use.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
SO = os.path.join(HERE, "librs_oracle.so")
SRC = os.path.join(HERE, "sampler_oracle.c")

KIND_TOPP, KIND_GENERAL, KIND_REPETITION = 0, 1, 2


class Trace(C.Structure):
    _fields_ = [(n, C.c_float) for n in
                ("maxu", "denom", "pmin", "pmax", "threshold", "comp", "sgtp", "sum_p", "randp", "sum_o", "rand2")] + \
               [(n, C.c_uint32) for n in ("left", "seqk", "sgtk", "rounds", "idxt", "early_exit")] + \
               [("rnd", C.c_uint32 * 4), ("token", C.c_int32)]


def build(force=False):
    if force or not os.path.exists(SO) or os.path.getmtime(SO) < os.path.getmtime(SRC):
        subprocess.run(["gcc", "-O2", "-fPIC", "-shared", "-fopenmp", "-ffp-contract=off", "-fno-fast-math",
                        "-o", SO, SRC, "-lm"], check=True)
    return SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(build())
        fp = C.POINTER(C.c_float)
        L.rs_oracle_philox4x32_10.argtypes = [C.POINTER(C.c_uint32)] * 3
        L.rs_oracle_setup_rand.argtypes = [C.c_void_p, C.c_uint64, C.c_int64, C.c_int64]
        L.rs_oracle_draw4.argtypes = [C.c_void_p, C.POINTER(C.c_uint32)]
        L.rs_oracle_uniform.argtypes = [C.c_uint32]
        L.rs_oracle_uniform.restype = C.c_float
        L.rs_oracle_sample_row.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int,
                                           C.c_float, C.c_float, C.c_float, C.c_float, C.c_void_p, C.c_void_p,
                                           C.POINTER(Trace)]
        L.rs_oracle_sample_row.restype = C.c_int32
        L.rs_oracle_normalise.argtypes = [C.c_int64, C.c_int64, C.c_int64, C.c_double, C.c_int64, C.c_double, C.c_int,
                                          C.POINTER(C.c_int), fp, C.POINTER(C.c_int), fp]
        L.rs_oracle_sample.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,
                                       C.c_double, C.c_int64, C.c_double, C.c_double, C.c_double, C.c_double, C.c_int]
        L.rs_oracle_block_scan.argtypes = [C.c_void_p, C.c_void_p]
        L.rs_oracle_block_scan.restype = C.c_float
        L.rs_oracle_warp_scan_ascending.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        L.rs_oracle_warp_scan_descending.argtypes = [C.c_void_p, C.c_void_p, C.c_int]
        for f in ("rs_oracle_block_sum_tree", "rs_oracle_block_sum_seq"):
            getattr(L, f).argtypes = [C.c_void_p]
            getattr(L, f).restype = C.c_float
        L.rs_oracle_sf.argtypes = [C.c_float]
        L.rs_oracle_sf.restype = C.c_float
        _lib = L
    return _lib


def philox4x32_10(ctr, key):
    c = (C.c_uint32 * 4)(*ctr)
    k = (C.c_uint32 * 2)(*key)
    o = (C.c_uint32 * 4)()
    lib().rs_oracle_philox4x32_10(c, k, o)
    return tuple(int(x) for x in o)


def setup_rand(seed, B, row0=0):
    """int8[B*64] numpy array with the layout of the reference's state tensor (sampling.cu:140-144)."""
    st = np.zeros(B * 64, dtype=np.int8)
    lib().rs_oracle_setup_rand(st.ctypes.data, seed & (2**64 - 1), B, row0)
    return st


def draw4(states, row):
    r = (C.c_uint32 * 4)()
    lib().rs_oracle_draw4(states.ctypes.data + 64 * row, r)
    return tuple(int(x) for x in r)


def uniform(x):
    return float(np.float32(lib().rs_oracle_uniform(x)))


class ArgError(ValueError):
    pass


_ERR = {-1: "Vocabulary size must be multiple of 4, and no larger than 1048576",
        -2: "B and T must be positive", -3: "Temperature outside range"}


def normalise(V, B, T, temperature, top_k, top_p, with_penalties=False):
    kind, k = C.c_int(), C.c_int()
    scale, p = C.c_float(), C.c_float()
    rc = lib().rs_oracle_normalise(V, B, T, temperature, top_k, top_p, int(with_penalties), kind, scale, k, p)
    if rc:
        raise ArgError(_ERR[rc])
    return kind.value, scale.value, k.value, p.value


def sample_row(logits, state, kind, scale, top_k, top_p, penalties=None, presence=0.0, repetition=0.0, decay=0.0,
               probs_in=None, want_probs=False):
    """One row. ``state`` is a 64-byte int8 view that is advanced in place; penalties updated in place.
    Returns (token, Trace, probs or None)."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    V = logits.shape[0]
    tr = Trace()
    pout = np.empty(V, dtype=np.float32) if want_probs else None
    if probs_in is not None:
        probs_in = np.ascontiguousarray(probs_in, dtype=np.float32)
    assert state.dtype == np.int8 and state.size == 64 and state.flags["C_CONTIGUOUS"]
    if penalties is not None:
        assert penalties.dtype == np.float32 and penalties.flags["C_CONTIGUOUS"]
    tok = lib().rs_oracle_sample_row(logits.ctypes.data, None if penalties is None else penalties.ctypes.data,
                                     state.ctypes.data, V, kind, scale, top_k, top_p, presence, repetition, decay,
                                     None if probs_in is None else probs_in.ctypes.data,
                                     None if pout is None else pout.ctypes.data, C.byref(tr))
    return tok, tr, pout


def sample(logits, states, temperature, top_k, top_p, penalties=None, presence=0.0, repetition=0.0, decay=0.0,
           nthreads=None):
    """Whole call with the reference's host semantics. logits: (V,), (B,V) or (B,T,V) float32 numpy.
    Returns int32[B]; states / penalties updated in place."""
    logits = np.ascontiguousarray(logits, dtype=np.float32)
    V = logits.shape[-1]
    if penalties is not None:
        B = penalties.shape[0] if penalties.ndim == 2 else 1      # sampling.cu:459
    else:
        B = logits.shape[0] if logits.ndim >= 2 else 1            # sampling.cu:983
    T = logits.shape[1] if logits.ndim == 3 else 1
    out = np.empty(B, dtype=np.int32)
    rc = lib().rs_oracle_sample(logits.ctypes.data, None if penalties is None else penalties.ctypes.data,
                                states.ctypes.data, out.ctypes.data, B, T, V, temperature, top_k, top_p,
                                presence, repetition, decay, nthreads or os.cpu_count() or 1)
    if rc:
        raise ArgError(_ERR[rc])
    return out


def block_scan(x):
    x = np.ascontiguousarray(x, dtype=np.float32)
    assert x.size == 1024
    out = np.empty(1024, dtype=np.float32)
    total = lib().rs_oracle_block_scan(x.ctypes.data, out.ctypes.data)
    return out, np.float32(total)


def scan_n(x, ascending):
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty_like(x)
    f = lib().rs_oracle_warp_scan_ascending if ascending else lib().rs_oracle_warp_scan_descending
    f(x.ctypes.data, out.ctypes.data, x.size)
    return out
