"""rapid_sampling_b200 -- B200 (sm_100a) drop-in for the reference sampler's torch extension.

Exports the reference module's three functions (``sampling.cpp:5-9``) with the same names and
positional order::

    states = setup_rand(seed, B)
    ids = batch_sampling_temperature_topk_topp(logits, states, temperature, top_k, top_p)
    ids = batch_sampling_repetition_temperature_topk_topp(logits, penalties, states, presence_penalty,
                                                          repetition_penalty, penalty_decay,
                                                          temperature, top_k, top_p)

The functions live in a compiled PyTorch extension built in-tree by ``rapid_sampling_b200._build``.
There is no CPU or eager fallback: importing the functions without the built extension raises.
"""
import importlib
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
_ext = None


def _load_ext():
    global _ext
    if _ext is None:
        import torch  # noqa: F401  libtorch must be loaded before the extension
        try:
            _ext = importlib.import_module("rapid_sampling_b200._rs_torch")
        except ImportError as e:
            raise ImportError("rapid_sampling_b200: the compiled extension is missing (%s). Build it with "
                              "`python -m rapid_sampling_b200._build`; there is no CPU fallback." % e) from e
    return _ext


def setup_rand(seed, B):
    return _load_ext().setup_rand(seed, B)


def batch_sampling_temperature_topk_topp(logits, states, temperature, top_k, top_p):
    return _load_ext().batch_sampling_temperature_topk_topp(logits, states, temperature, top_k, top_p)


def batch_sampling_repetition_temperature_topk_topp(logits, penalties, states, presence_penalty, repetition_penalty,
                                                    penalty_decay, temperature, top_k, top_p):
    return _load_ext().batch_sampling_repetition_temperature_topk_topp(
        logits, penalties, states, presence_penalty, repetition_penalty, penalty_decay, temperature, top_k, top_p)


def batch_sampling_temperature_topk_topp_any(logits, states, temperature, top_k, top_p):
    """Same call for fp32, fp16 or bf16 logits (the reference accepts fp32 only, sampling.cu:976). 16-bit logits are
    read directly and widened exactly, so the ids equal those of the fp32 call on ``logits.float()``."""
    return _load_ext().batch_sampling_temperature_topk_topp_any(logits, states, temperature, top_k, top_p)


def batch_sampling_repetition_temperature_topk_topp_any(logits, penalties, states, presence_penalty, repetition_penalty,
                                                        penalty_decay, temperature, top_k, top_p):
    return _load_ext().batch_sampling_repetition_temperature_topk_topp_any(
        logits, penalties, states, presence_penalty, repetition_penalty, penalty_decay, temperature, top_k, top_p)


def batch_sampling_rows(logits, states, temperature=None, top_k=None, top_p=None, penalties=None, presence_penalty=0.0,
                        repetition_penalty=0.0, penalty_decay=0.0, return_prob=False):
    """Per-row parameters: `temperature` (float32), `top_k` (int32) and `top_p` (float32) are CUDA tensors of B values, or
    None for the neutral value in every row.  Row b is sampled exactly as a one-row call of the functions above with its
    values would sample it.  With `return_prob` the result is (ids, probability of each id under the full softmax, kept
    probability mass).  The reference takes scalars only (sampling.cpp:2-3)."""
    return _load_ext().batch_sampling_rows(logits, states, temperature, top_k, top_p, penalties, presence_penalty,
                                           repetition_penalty, penalty_decay, return_prob)


def kernel_launch_count():
    return _load_ext().kernel_launch_count()


def device_status():
    """Synchronises the current stream and returns the device status word of this device (0 = ok, else a negative
    RS_ERR_* code such as "a bounded on-chip wait gave up"), clearing it.  Sampling calls check a host mirror of the
    word by themselves and raise on the NEXT call; this is the explicit, synchronising form."""
    return _load_ext().device_status()


def release_workspaces():
    """Drops the per-(device, stream) scratch buffers the sampling calls keep between calls."""
    return _load_ext().release_workspaces()


__all__ = ["setup_rand", "batch_sampling_temperature_topk_topp", "batch_sampling_repetition_temperature_topk_topp",
           "batch_sampling_temperature_topk_topp_any", "batch_sampling_repetition_temperature_topk_topp_any", "batch_sampling_rows",
           "kernel_launch_count", "device_status", "release_workspaces"]
