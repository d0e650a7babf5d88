"""In-tree build of the native libraries.

``libgcb200_host.so``  -- CPU oracles and host-side native helpers (g++, no CUDA needed)
``libgcb200_cuda.so``  -- every sm_100a kernel (nvcc ``-gencode arch=compute_100a,code=sm_100a``)

Both land in ``gradient_compression_b200/_lib/`` next to the sources they are built from, and are
bound with ctypes (plain C ABI: raw pointers + a ``cudaStream_t``), so a rebuild takes seconds and
needs neither libtorch headers nor pybind.  Run ``python -m gradient_compression_b200.build``.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIBDIR = os.path.join(HERE, "_lib")

HOST_SOURCES = ["host_oracle.cpp"]
CUDA_SOURCES = ["gc_kernels.cu", "gc_fused.cu", "gc_noalloc.cu", "gc_bn.cu", "gc_powersgd.cu", "gc_topk.cu", "gc_gemm_tc.cu", "gc_varpack.cu", "gc_augment.cu"]
NVCC_ARCH = ["-gencode", "arch=compute_100a,code=sm_100a"]


def _sources(names):
    return [os.path.join(CSRC, n) for n in names]


def _digest(paths, extra=""):
    h = hashlib.sha256(extra.encode())
    headers = sorted(p for p in os.listdir(CSRC) if p.endswith((".h", ".cuh")))
    for p in list(paths) + [os.path.join(CSRC, x) for x in headers]:
        with open(p, "rb") as f:
            h.update(f.read())
    return h.hexdigest()


def _stale(lib, digest):
    stamp = lib + ".sha256"
    if not os.path.exists(lib) or not os.path.exists(stamp):
        return True
    with open(stamp) as f:
        return f.read().strip() != digest


def _finish(lib, digest):
    with open(lib + ".sha256", "w") as f:
        f.write(digest)


def host_lib_path():
    return os.path.join(LIBDIR, "libgcb200_host.so")


def cuda_lib_path():
    return os.path.join(LIBDIR, "libgcb200_cuda.so")


def build_host(force=False, verbose=False):
    os.makedirs(LIBDIR, exist_ok=True)
    srcs = _sources(HOST_SOURCES)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-Wno-unknown-pragmas",
           "-I", CSRC, "-o", host_lib_path()] + srcs
    digest = _digest(srcs, " ".join(cmd))
    if not force and not _stale(host_lib_path(), digest):
        return host_lib_path()
    if shutil.which("g++") is None:
        raise RuntimeError("g++ not found: cannot build libgcb200_host.so")
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    _finish(host_lib_path(), digest)
    return host_lib_path()


def nvcc_path():
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def build_cuda(force=False, verbose=False, ptxas_info=False):
    os.makedirs(LIBDIR, exist_ok=True)
    srcs = _sources(CUDA_SOURCES)
    nvcc = nvcc_path()
    cmd = [nvcc or "nvcc"] + NVCC_ARCH + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-shared",
                                        "-I", CSRC, "-o", cuda_lib_path()] + srcs
    if ptxas_info:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    digest = _digest(srcs, " ".join(c for c in cmd if c not in ("-Xptxas", "-v")))
    if not force and not _stale(cuda_lib_path(), digest):
        return cuda_lib_path()
    if nvcc is None:
        raise RuntimeError("nvcc not found: cannot build libgcb200_cuda.so")
    if verbose:
        print(" ".join(cmd))
    subprocess.run(cmd, check=True)
    _finish(cuda_lib_path(), digest)
    return cuda_lib_path()


def build_all(force=False, verbose=False):
    return build_host(force, verbose), build_cuda(force, verbose)


if __name__ == "__main__":
    force = "--force" in sys.argv
    print(build_host(force, verbose=True))
    print(build_cuda(force, verbose=True, ptxas_info="--ptxas" in sys.argv))
