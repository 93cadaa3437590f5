"""ctypes view of the C ABI declared in ``include/rapid_sampling_b200.h``.

This is the boundary a non-Python host would bind; the parity tests call the kernels through it.
Loading fails loudly when the CUDA library has not been built -- there is no CPU fallback.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "librapid_sampling_b200.so")

RS_OK = 0
RS_ERR_DTYPE, RS_ERR_VOCAB, RS_ERR_BATCH, RS_ERR_TEMPERATURE = -1, -2, -3, -4
RS_ERR_POINTER, RS_ERR_WORKSPACE, RS_ERR_CUDA, RS_ERR_TIMEOUT, RS_ERR_LIMIT = -5, -6, -7, -8, -9
RS_ERR_INTERNAL = -10
RS_STATE_BYTES = 64
RS_DTYPE_F32, RS_DTYPE_F16, RS_DTYPE_BF16 = 0, 1, 2
RS_STATIC_SCRATCH_FLOATS = 4194304

SYMBOLS = ["rs_setup_rand", "rs_workspace_bytes", "rs_sample", "rs_sample_debug", "rs_sample_host", "rs_sample_typed", "rs_sample_static_scratch", "rs_rows_workspace_bytes", "rs_sample_rows",
           "rs_device_status", "rs_clear_status", "rs_set_status_mirror", "rs_set_wait_polls", "rs_set_dependent_launch", "rs_selftest_bounded_wait", "rs_set_cluster_override", "rs_set_path_override", "rs_kernel_launch_count", "rs_vp_workspace_bytes", "rs_vp_layout", "rs_vp_fast_layout", "rs_vp_stage", "rs_vp_tile_begin", "rs_vp_tile_max", "rs_status_string",
           "rs_last_cuda_error", "rs_version"]


class Trace(C.Structure):
    _fields_ = [(n, C.c_float) for n in
                ("maxu", "denom", "pmin", "pmax", "threshold", "comp", "sgtp", "sum_p", "randp", "sum_o", "rand2")] + \
               [(n, C.c_uint32) for n in ("left", "seqk", "sgtk", "rounds", "idxt", "early_exit")] + \
               [("rnd", C.c_uint32 * 4), ("token", C.c_int32), ("path", C.c_uint32), ("ncand", C.c_uint32), ("t_ns", C.c_uint32 * 10)]


class VpCall(C.Structure):
    _fields_ = [("logits", C.c_void_p), ("penalties", C.c_void_p), ("states", C.c_void_p), ("workspace", C.c_void_p),
                ("stream", C.c_void_p), ("B", C.c_int64), ("T", C.c_int64), ("V_local", C.c_int64),
                ("V_global", C.c_int64), ("col0", C.c_int64), ("top_k", C.c_int64), ("temperature", C.c_double),
                ("top_p", C.c_double), ("presence_penalty", C.c_double), ("repetition_penalty", C.c_double),
                ("penalty_decay", C.c_double), ("rank", C.c_int32), ("world", C.c_int32)]


VP_MAX, VP_SUM, VP_ROUND, VP_TALLY, VP_WEIGHT, VP_PICK, VP_PENALTY = range(7)
VP_ROUNDS = 8
VPF_MAX, VPF_SUM, VPF_COMPACT, VPF_FINISH, VPF_ADVANCE, VPF_EXTRACT = 10, 11, 12, 13, 14, 15

_lib = None


def load():
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError("%s is missing: build it with `python -m rapid_sampling_b200._build` "
                          "(there is no CPU fallback)" % LIB_PATH)
    L = C.CDLL(LIB_PATH)
    vp, i64, dbl = C.c_void_p, C.c_int64, C.c_double
    L.rs_setup_rand.argtypes = [vp, C.c_uint64, i64, i64, vp]
    L.rs_workspace_bytes.argtypes = [i64, i64]
    L.rs_workspace_bytes.restype = C.c_size_t
    common = [vp, i64, i64, i64, vp, vp, vp, dbl, i64, dbl, dbl, dbl, dbl]
    L.rs_sample.argtypes = common + [vp, C.c_size_t, vp]
    L.rs_sample_debug.argtypes = common + [vp, C.c_size_t, vp, vp, vp]
    L.rs_sample_host.argtypes = common + [vp, vp, vp, C.c_size_t, vp]
    L.rs_sample_typed.argtypes = [vp, C.c_int32] + common[1:] + [vp, C.c_size_t, vp, vp, vp]
    L.rs_sample_static_scratch.argtypes = common + [vp]
    L.rs_rows_workspace_bytes.argtypes = [i64, i64]
    L.rs_rows_workspace_bytes.restype = C.c_size_t
    L.rs_sample_rows.argtypes = [vp, C.c_int32, i64, i64, i64, vp, vp, vp, vp, vp, vp, C.c_double, C.c_double, C.c_double,
                                 vp, vp, vp, C.c_size_t, vp]
    L.rs_vp_workspace_bytes.argtypes = [i64, C.c_int32]
    L.rs_vp_workspace_bytes.restype = C.c_size_t
    L.rs_vp_layout.argtypes = [i64, C.c_int32, C.POINTER(C.c_int64)]
    L.rs_vp_fast_layout.argtypes = [i64, i64, C.c_int32, C.POINTER(C.c_int64)]
    L.rs_vp_stage.argtypes = [C.POINTER(VpCall), C.c_int32, C.c_int32]
    L.rs_vp_tile_begin.argtypes = [C.POINTER(VpCall)]
    L.rs_vp_tile_max.argtypes = [C.POINTER(VpCall), vp, i64, i64, i64]
    L.rs_device_status.argtypes = [vp, vp]
    L.rs_clear_status.argtypes = [vp, vp]
    L.rs_set_status_mirror.argtypes = [vp]
    L.rs_set_wait_polls.argtypes = [C.c_uint32]
    L.rs_set_wait_polls.restype = C.c_uint32
    L.rs_selftest_bounded_wait.argtypes = [vp, C.c_uint32, vp]
    L.rs_set_dependent_launch.argtypes = [C.c_int]
    L.rs_set_cluster_override.argtypes = [C.c_int]
    L.rs_set_path_override.argtypes = [C.c_int]
    L.rs_kernel_launch_count.restype = C.c_uint64
    for f in ("rs_status_string", "rs_last_cuda_error", "rs_version"):
        getattr(L, f).restype = C.c_char_p
    L.rs_status_string.argtypes = [C.c_int]
    _lib = L
    return L


def status_string(rc):
    return load().rs_status_string(rc).decode()
