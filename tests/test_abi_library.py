"""CPU: the C-ABI library loads, exports every symbol the header declares, and rejects bad
arguments with the documented codes before touching the GPU."""
import ctypes as C
import os
import re

from helpers import ROOT


def declared_functions():
    src = open(os.path.join(ROOT, "include", "rapid_sampling_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(rs_[a-z0-9_]+)\s*\(", src)))


def test_library_exports_every_declared_symbol():
    from rapid_sampling_b200 import abi
    L = abi.load()
    names = declared_functions()
    assert len(names) >= 10
    for n in names:
        assert hasattr(L, n), n
    assert sorted(abi.SYMBOLS) == names
    assert b"sm_100a" in L.rs_version()


def test_argument_errors_need_no_gpu():
    """Same conditions as the reference's std::invalid_argument throws (sampling.cu:986, :992, :999)."""
    from rapid_sampling_b200 import abi
    L = abi.load()
    dummy = C.c_void_p(256)

    def call(B, T, V, temp):
        return L.rs_sample(dummy, B, T, V, None, dummy, dummy, temp, -1, 0.5, 0.0, 0.0, 0.0, dummy, 256, None)
    assert call(1, 1, 6, 1.0) == abi.RS_ERR_VOCAB
    assert call(1, 1, 0, 1.0) == abi.RS_ERR_VOCAB
    assert call(1, 1, 1048580, 1.0) == abi.RS_ERR_VOCAB
    assert call(0, 1, 1024, 1.0) == abi.RS_ERR_BATCH
    assert call(1, 0, 1024, 1.0) == abi.RS_ERR_BATCH
    assert call(1, 1, 1024, 0.0005) == abi.RS_ERR_TEMPERATURE
    assert call(1, 1, 1024, 1001.0) == abi.RS_ERR_TEMPERATURE
    assert call(1, 1, 1024, float("nan")) == abi.RS_ERR_TEMPERATURE
    assert L.rs_sample(None, 1, 1, 1024, None, dummy, dummy, 1.0, -1, 0.5, 0.0, 0.0, 0.0, dummy, 256, None) == abi.RS_ERR_POINTER
    assert L.rs_sample(C.c_void_p(260), 1, 1, 1024, None, dummy, dummy, 1.0, -1, 0.5, 0.0, 0.0, 0.0, dummy, 256, None) == abi.RS_ERR_POINTER
    assert L.rs_setup_rand(None, 0, 4, 0, None) == abi.RS_ERR_POINTER
    assert L.rs_setup_rand(dummy, 0, 0, 0, None) == abi.RS_ERR_BATCH
    assert L.rs_workspace_bytes(4, 131072) == 256                        # whole batch on chip: status word only
    assert L.rs_workspace_bytes(64, 151936) == 256 + 64 * 151936 * 4     # more rows than fit at once: streaming
    assert L.rs_workspace_bytes(2, 1048576) == 256 + 2 * 1048576 * 4     # row too large for on-chip storage
    assert abi.status_string(abi.RS_ERR_VOCAB).startswith("Vocabulary size must be multiple of 4")
    assert L.rs_set_cluster_override(3) == 0 and L.rs_set_cluster_override(0) == 0


def test_python_package_exports_reference_names():
    import rapid_sampling_b200 as r
    for n in ("setup_rand", "batch_sampling_temperature_topk_topp", "batch_sampling_repetition_temperature_topk_topp"):
        assert callable(getattr(r, n))
    ext = r._load_ext()
    doc = ext.batch_sampling_repetition_temperature_topk_topp.__doc__
    for arg in ("logits", "penalties", "states", "presence_penalty", "repetition_penalty", "penalty_decay",
                "temperature", "top_k", "top_p"):
        assert arg in doc


def test_vocab_parallel_stage_refuses_bad_shards_without_a_gpu():
    """rs_vp_stage reads float4 groups at row_base + g, so a shard must be a multiple of 4 columns wide, 16-byte
    aligned, and the shards must tile the vocabulary in rank order; anything else is an error code, not a launch."""
    from rapid_sampling_b200 import abi
    L = abi.load()

    def call(**kw):
        c = abi.VpCall()
        c.logits = c.states = c.workspace = 4096
        c.penalties = None
        c.B, c.T, c.V_local, c.V_global, c.col0 = 2, 1, 8192, 32768, 8192
        c.top_k, c.temperature, c.top_p = 50, 0.8, 0.9
        c.rank, c.world = 1, 4
        for k, v in kw.items():
            setattr(c, k, v)
        return L.rs_vp_stage(C.byref(c), abi.VPF_MAX, 0)
    assert call(V_local=8190, V_global=32760) == abi.RS_ERR_VOCAB            # not a multiple of 4 columns
    assert call(V_local=4096) == abi.RS_ERR_VOCAB                            # shards do not tile the vocabulary
    assert call(col0=0) == abi.RS_ERR_VOCAB                                  # not this rank's columns
    assert call(logits=4100) == abi.RS_ERR_POINTER
    assert call(penalties=4104) == abi.RS_ERR_POINTER
    assert call(workspace=4098) == abi.RS_ERR_POINTER
    assert call(rank=4) == abi.RS_ERR_BATCH
    assert call(temperature=0.0) == abi.RS_ERR_TEMPERATURE
    assert L.rs_selftest_bounded_wait(None, 4, None) == abi.RS_ERR_POINTER
    assert L.rs_set_wait_polls(0) > 0
