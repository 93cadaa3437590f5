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
              "--extra-device-vectorization", "-Xptxas", "-O3", "-Xcompiler", "-fPIC"] + \
    os.environ.get("RS_EXTRA_NVCC_FLAGS", "").split()


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


CU_SOURCES = ["rs_sampler.cu", "rs_rowcta.cu", "rs_vocab_parallel.cu"]
HEADERS = [os.path.join(CSRC, h) for h in ("rs_device.cuh", "rs_common.cuh", "rs_rowcta.cuh")] + \
    [os.path.join(INCLUDE, "rapid_sampling_b200.h")]
OBJ_DIR = os.path.join(HERE, "build")


def build_lib(force=False, verbose=False, ptxas_v=False):
    """Compiles every .cu file to an object of its own (in parallel), then links them into the library."""
    import concurrent.futures as cf
    nvcc = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    os.makedirs(OBJ_DIR, exist_ok=True)
    jobs = []
    for name in CU_SOURCES:
        src = os.path.join(CSRC, name)
        obj = os.path.join(OBJ_DIR, name[:-3] + ".o")
        if force or ptxas_v or not _newer(obj, [src] + HEADERS):
            jobs.append([nvcc] + NVCC_FLAGS + (["-Xptxas", "-v"] if ptxas_v else []) + ["-c", src, "-o", obj])
    with cf.ThreadPoolExecutor(max_workers=max(1, len(jobs))) as ex:
        list(ex.map(lambda c: _run(c, verbose or ptxas_v), jobs))
    objs = [os.path.join(OBJ_DIR, n[:-3] + ".o") for n in CU_SOURCES]
    if jobs or not _newer(LIB, objs):
        _run([nvcc, "-shared", "-o", LIB] + objs + ["-gencode", "arch=compute_100a,code=sm_100a"], verbose)
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
