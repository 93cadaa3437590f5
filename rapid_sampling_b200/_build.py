"""In-tree build of the sm_100a sampler: the C-ABI CUDA library and the PyTorch binding.

``python -m rapid_sampling_b200._build`` (or ``build()``) produces, next to this file,
``librapid_sampling_b200.so`` (nvcc, no torch dependency) and ``_rs_torch<EXT_SUFFIX>`` (g++ with
the torch headers, linked against the former).  nvcc cross-compiles without a GPU.
"""
import os
import subprocess
import sys
import sysconfig

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
INCLUDE = os.path.join(os.path.dirname(HERE), "include")
LIB = os.path.join(HERE, "librapid_sampling_b200.so")
EXT_NAME = "_rs_torch"
EXT = os.path.join(HERE, EXT_NAME + sysconfig.get_config_var("EXT_SUFFIX"))

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--extra-device-vectorization", "-Xptxas", "-O3", "-Xcompiler", "-fPIC"]


def _newer(target, sources):
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd, verbose):
    if verbose:
        print(" ".join(cmd), flush=True)
    r = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if r.returncode != 0:
        raise RuntimeError("build step failed:\n%s\n%s" % (" ".join(cmd), r.stdout))
    if verbose and r.stdout:
        print(r.stdout)


def build_lib(force=False, verbose=False, ptxas_v=False):
    srcs = [os.path.join(CSRC, "rs_sampler.cu"), os.path.join(CSRC, "rs_vocab_parallel.cu"),
            os.path.join(CSRC, "rs_device.cuh"), os.path.join(INCLUDE, "rapid_sampling_b200.h")]
    if not force and _newer(LIB, srcs):
        return LIB
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    cmd = [nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_v else []) + ["-shared", "-o", LIB, srcs[0], srcs[1]]
    _run(cmd, verbose or ptxas_v)
    return LIB


def build_ext(force=False, verbose=False):
    src = os.path.join(CSRC, "rs_torch.cpp")
    if not force and _newer(EXT, [src, LIB]):
        return EXT
    import torch
    from torch.utils import cpp_extension as ce
    inc = []
    for p in ce.include_paths("cuda") + [sysconfig.get_paths()["include"]]:
        inc += ["-isystem", p]
    tlib = os.path.join(os.path.dirname(torch.__file__), "lib")
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", src, "-o", EXT,
           "-DTORCH_EXTENSION_NAME=" + EXT_NAME, "-DTORCH_API_INCLUDE_EXTENSION_H",
           "-D_GLIBCXX_USE_CXX11_ABI=%d" % int(torch._C._GLIBCXX_USE_CXX11_ABI)] + inc + \
          ["-L" + HERE, "-l:librapid_sampling_b200.so", "-L" + tlib,
           "-lc10", "-lc10_cuda", "-ltorch_cpu", "-ltorch_cuda", "-ltorch", "-ltorch_python",
           "-Wl,-rpath,$ORIGIN", "-Wl,-rpath," + tlib]
    _run(cmd, verbose)
    return EXT


def build(force=False, verbose=False):
    build_lib(force, verbose)
    build_ext(force, verbose)
    return LIB, EXT


if __name__ == "__main__":
    build(force="--force" in sys.argv, verbose=True)
    print("built", LIB, EXT)
