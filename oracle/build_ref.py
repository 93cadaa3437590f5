"""Build recipe for the bit-level checker: the reference's own CUDA extension.

TEST INFRASTRUCTURE ONLY.  Compiles the reference's two source files *where they
lie* (default: the read-only reference checkout) into ``oracle/_ref/sample_ref*.so``
for sm_100a, with the flags of the reference's ``example.py:16``
(``-O3 -res-usage --extra-device-vectorization -Xptxas -O3``; no fast-math, so
``exp2f`` and ``/`` are the precise versions).  No reference source is copied
into this repository; only the built module lands in ``oracle/_ref/`` (git-ignored).

The built module exposes the reference's three functions (``sampling.cpp:5-9``):
``setup_rand``, ``batch_sampling_temperature_topk_topp`` and
``batch_sampling_repetition_temperature_topk_topp``.  Only GPU parity tests load it.

Never hand it a 3-D logits tensor: its scratch is allocated ``{B,V}``
(``sampling.cu:1014``) but indexed ``(b*T+T-1)*V`` (``sampling.cu:782``), which is
out of bounds for T >= 2.  ``load_ref()`` wraps the calls and refuses 3-D input.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "sample_ref"


def so_path():
    return os.path.join(OUT, NAME + sysconfig.get_config_var("EXT_SUFFIX"))


def build(ref_dir=None, verbose=False):
    """Compile the reference extension if its sources are reachable. Returns the .so path or None."""
    ref_dir = ref_dir or os.environ.get("RS_REFERENCE_DIR", "/root/reference")
    cu = os.path.join(ref_dir, "sampling.cu")
    cpp = os.path.join(ref_dir, "sampling.cpp")
    target = so_path()
    if not (os.path.exists(cu) and os.path.exists(cpp)):
        return target if os.path.exists(target) else None
    if os.path.exists(target) and os.path.getmtime(target) >= max(os.path.getmtime(cu), os.path.getmtime(cpp)):
        return target
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(OUT, exist_ok=True)
    inc = []
    for p in ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]:
        inc += ["-isystem", p]
    abi = "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)
    common = ["-DTORCH_EXTENSION_NAME=" + NAME, "-DTORCH_API_INCLUDE_EXTENSION_H", abi]
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    o_cu = os.path.join(OUT, "sampling.cuda.o")
    o_cpp = os.path.join(OUT, "sampling.o")
    cmds = [
        [nvcc, "-c", cu, "-o", o_cu, "-std=c++17", "--expt-relaxed-constexpr",
         "-gencode", "arch=compute_100a,code=sm_100a", "--compiler-options", "-fPIC",
         "-O3", "-res-usage", "--extra-device-vectorization", "-Xptxas", "-O3"] + common + inc,
        ["g++", "-c", cpp, "-o", o_cpp, "-std=c++17", "-O2", "-fPIC"] + common + inc,
        ["g++", "-shared", o_cu, o_cpp, "-o", target,
         "-L" + os.path.join(os.path.dirname(torch.__file__), "lib"),
         "-L/usr/local/cuda/lib64", "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch",
         "-ltorch_python", "-lcudart",
         "-Wl,-rpath," + os.path.join(os.path.dirname(torch.__file__), "lib")],
    ]
    for c in cmds:
        if verbose:
            print(" ".join(c), flush=True)
        subprocess.run(c, check=True, stdout=None if verbose else subprocess.DEVNULL,
                       stderr=None if verbose else subprocess.DEVNULL)
    for o in (o_cu, o_cpp):
        os.remove(o)
    return target


class _Ref:
    """Guarded handle on the reference module: 1-D/2-D logits only (see module docstring)."""

    def __init__(self, mod):
        self._m = mod

    def setup_rand(self, seed, B):
        return self._m.setup_rand(int(seed), int(B))

    def batch_sampling_temperature_topk_topp(self, logits, states, temperature, top_k, top_p):
        assert logits.dim() <= 2, "the reference kernel writes out of bounds for (B,T,V) input"
        assert logits.is_contiguous()
        return self._m.batch_sampling_temperature_topk_topp(logits, states, float(temperature), int(top_k), float(top_p))

    def batch_sampling_repetition_temperature_topk_topp(self, logits, penalties, states, presence, repetition,
                                                        decay, temperature, top_k, top_p):
        assert logits.dim() <= 2, "the reference kernel writes out of bounds for (B,T,V) input"
        assert logits.is_contiguous() and penalties.is_contiguous()
        return self._m.batch_sampling_repetition_temperature_topk_topp(
            logits, penalties, states, float(presence), float(repetition), float(decay),
            float(temperature), int(top_k), float(top_p))


def load_ref():
    """Import the prebuilt reference module (needs a GPU to be useful). Returns None if it was never built."""
    path = so_path()
    if not os.path.exists(path):
        return None
    import importlib.util
    import torch  # noqa: F401  (libtorch must be loaded first)
    spec = importlib.util.spec_from_file_location(NAME, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return _Ref(mod)


if __name__ == "__main__":
    p = build(verbose=True)
    print("built:" if p else "reference sources not found and no prebuilt module:", p)
    sys.exit(0 if p else 1)
