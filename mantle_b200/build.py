"""Builds the CUDA sampler libraries in-tree for sm_100a.

    python -m mantle_b200.build [--force] [--verbose]

The result, mantle_b200/lib/libmantle_cuda_sampler.so, exports the C-ABI declared in
include/mantle_cuda_sampler.h and include/mantle_host_sampler.h; beside it,
libmantle_cuda_sampler_nccl.so (include/mantle_cuda_sampler_nccl.h) adds the one entry point that
needs NCCL, so that the sampler itself loads on hosts without it.  nvcc cross-compiles without a GPU.  The flags follow the
reference's kernel build (scripts/build_cuda.sh:54-72: -O3 -lineinfo and one -gencode),
with the architecture fixed to sm_100a and multiply-add fusion switched off, which the
sampler's float32 arithmetic contract requires.
"""
import os
import shutil
import subprocess
import sys

PKG = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(PKG)
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libmantle_cuda_sampler.so")
NCCL_LIB_PATH = os.path.join(LIB_DIR, "libmantle_cuda_sampler_nccl.so")
NCCL_SOURCES = ["sharded_nccl.cu"]

SOURCES = ["sampler_kernels.cu", "host_sampler.cu", "host_batch_sampler.cu"]
HEADERS = [
    os.path.join(ROOT, "include", "mantle_cuda_sampler.h"),
    os.path.join(ROOT, "include", "mantle_sample_params.h"),
    os.path.join(ROOT, "include", "mantle_host_sampler.h"),
    os.path.join(ROOT, "include", "mantle_batch_sampler.h"),
    os.path.join(ROOT, "include", "mantle_cuda_sampler_nccl.h"),
]

NVCC_FLAGS = [
    "-O3",
    "-std=c++17",
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-fmad=false",
    "-Xcompiler", "-fPIC",
    "-shared",
]


def find_nvcc():
    for cand in (shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the CUDA sampler library cannot be built")


def _stale(path=None):
    path = path or LIB_PATH
    if not os.path.exists(path):
        return True
    t = os.path.getmtime(path)
    deps = [os.path.join(CSRC, s) for s in SOURCES + NCCL_SOURCES] + HEADERS + [os.path.abspath(__file__)]
    deps += [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cuh", ".h"))]
    return any(os.path.getmtime(d) > t for d in deps)


def _run_nvcc(args, out, verbose):
    cmd = [find_nvcc()] + NVCC_FLAGS
    if verbose:
        cmd += ["-Xptxas", "-v"]
    # the PATH g++ on purpose: an inherited CXX may point at a wrapper nvcc cannot drive
    host = shutil.which("g++")
    if host:
        cmd += ["-ccbin", host]
    cmd += ["-o", out] + args
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or res.returncode != 0:
        sys.stderr.write(res.stdout)
    if res.returncode != 0:
        raise RuntimeError("nvcc failed (exit %d): %s" % (res.returncode, " ".join(cmd)))


def build_native(force=False, verbose=False):
    """Compiles the sampler library if it is missing or older than its sources.  Returns its path."""
    if not force and not _stale():
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    _run_nvcc([os.path.join(CSRC, s) for s in SOURCES], LIB_PATH, verbose)
    return LIB_PATH


def build_nccl(force=False, verbose=False):
    """Compiles the NCCL entry point (libmantle_cuda_sampler_nccl.so) against the sampler library
    and the system's libnccl.  Returns its path."""
    build_native(force=False, verbose=verbose)
    if not force and not _stale(NCCL_LIB_PATH) and os.path.getmtime(NCCL_LIB_PATH) >= os.path.getmtime(LIB_PATH):
        return NCCL_LIB_PATH
    _run_nvcc([os.path.join(CSRC, s) for s in NCCL_SOURCES]
              + ["-L" + LIB_DIR, "-lmantle_cuda_sampler", "-lnccl", "-Xlinker", "-rpath=$ORIGIN"],
              NCCL_LIB_PATH, verbose)
    return NCCL_LIB_PATH


if __name__ == "__main__":
    print(build_native(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
    print(build_nccl(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
