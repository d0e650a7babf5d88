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
CUDA_SOURCES = ["gc_kernels.cu", "gc_fused.cu", "gc_noalloc.cu", "gc_bn.cu", "gc_head.cu", "gc_powersgd.cu", "gc_topk.cu", "gc_gemm_tc.cu", "gc_conv_tc.cu", "gc_varpack.cu", "gc_augment.cu"]
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


def _flags_only(cmd):
    """The part of a compiler command that decides what gets built: everything except absolute paths, so that a library
    built in one checkout is recognised as current when the tree is copied somewhere else."""
    return " ".join(os.path.basename(c) if os.path.isabs(c) else c for c in cmd)


class _BuildLock:
    """Exclusive lock for the library directory: ranks of one job that all find a stale library build it once."""

    def __init__(self):
        self._f = None

    def __enter__(self):
        import fcntl

        os.makedirs(LIBDIR, exist_ok=True)
        self._f = open(os.path.join(LIBDIR, ".build.lock"), "w")
        fcntl.flock(self._f, fcntl.LOCK_EX)
        return self

    def __exit__(self, *exc):
        import fcntl

        fcntl.flock(self._f, fcntl.LOCK_UN)
        self._f.close()


def _compile(cmd, out):
    """Run the compiler into a temporary file and move it into place, so that nobody ever loads a half-written library."""
    tmp = out + f".tmp{os.getpid()}"
    cmd = [tmp if c == out else c for c in cmd]
    try:
        subprocess.run(cmd, check=True)
        os.replace(tmp, out)
    finally:
        if os.path.exists(tmp):
            os.remove(tmp)


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


def cuda_lib_path(debug_bounds=False):
    """``debug_bounds``: the build with -DGC_DEBUG_BOUNDS (computed gather / scatter indices checked before use, a failing
    one recorded in the arena's status word instead of being followed); loaded instead of the regular library when
    ``GCB200_DEBUG_BOUNDS=1``."""
    return os.path.join(LIBDIR, "libgcb200_cuda_dbg.so" if debug_bounds else "libgcb200_cuda.so")


def build_host(force=False, verbose=False):
    os.makedirs(LIBDIR, exist_ok=True)
    srcs = _sources(HOST_SOURCES)
    cmd = ["g++", "-O2", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-Wno-unknown-pragmas",
           "-I", CSRC, "-o", host_lib_path()] + srcs
    digest = _digest(srcs, _flags_only(cmd))
    if not force and not _stale(host_lib_path(), digest):
        return host_lib_path()
    if shutil.which("g++") is None:
        raise RuntimeError("g++ not found: cannot build libgcb200_host.so")
    with _BuildLock():
        if force or _stale(host_lib_path(), digest):          # another process may have built it while we waited
            if verbose:
                print(" ".join(cmd))
            _compile(cmd, host_lib_path())
            _finish(host_lib_path(), digest)
    return host_lib_path()


def build_host_sanitized(verbose=False):
    """The host library with AddressSanitizer and UndefinedBehaviorSanitizer, as ``libgcb200_host_san.so``.  Use:
    ``GCB200_HOST_LIB=<that file> ASAN_OPTIONS=detect_leaks=0 LD_PRELOAD=$(gcc -print-file-name=libasan.so) python -m pytest
    tests/test_philox_quant.py`` -- the oracles, packers and coders then run with every access and shift checked."""
    os.makedirs(LIBDIR, exist_ok=True)
    out = os.path.join(LIBDIR, "libgcb200_host_san.so")
    cmd = ["g++", "-O1", "-g", "-std=c++17", "-fPIC", "-shared", "-ffp-contract=off", "-fsanitize=address,undefined",
           "-fno-omit-frame-pointer", "-Wno-unknown-pragmas", "-I", CSRC, "-o", out] + _sources(HOST_SOURCES)
    if verbose:
        print(" ".join(cmd))
    with _BuildLock():
        _compile(cmd, out)
    return out


def nvcc_path():
    cand = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    return cand if os.path.exists(cand) else None


def _compile_cuda_objects(nvcc, srcs, objdir, ptxas_info, verbose, defines=()):
    """One ``nvcc -c`` per source, all at once: the sources are independent translation units."""
    from concurrent.futures import ThreadPoolExecutor

    os.makedirs(objdir, exist_ok=True)
    flags = NVCC_ARCH + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-I", CSRC] + [f"-D{d}" for d in defines]
    if ptxas_info:
        flags = ["-Xptxas", "-v"] + flags

    def one(src):
        obj = os.path.join(objdir, os.path.basename(src) + f".{os.getpid()}.o")
        cmd = [nvcc] + flags + ["-c", src, "-o", obj]
        if verbose:
            print(" ".join(cmd))
        subprocess.run(cmd, check=True)
        return obj

    with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
        return list(pool.map(one, srcs))


def build_cuda(force=False, verbose=False, ptxas_info=False, debug_bounds=False):
    os.makedirs(LIBDIR, exist_ok=True)
    srcs = _sources(CUDA_SOURCES)
    nvcc = nvcc_path()
    lib = cuda_lib_path(debug_bounds)
    defines = ("GC_DEBUG_BOUNDS",) if debug_bounds else ()
    # what decides the result: compiler, flags and sources (the stamp also covers every header)
    recipe = [nvcc or "nvcc"] + NVCC_ARCH + ["-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-shared",
                                           "-I", CSRC, "-o", lib] + [f"-D{d}" for d in defines] + srcs
    digest = _digest(srcs, _flags_only(recipe))
    if not force and not _stale(lib, digest):
        return lib
    if nvcc is None:
        raise RuntimeError(f"nvcc not found: cannot build {os.path.basename(lib)}")
    with _BuildLock():
        if force or _stale(lib, digest):
            objdir = os.path.join(LIBDIR, "obj_dbg" if debug_bounds else "obj")
            objs = []
            try:
                objs = _compile_cuda_objects(nvcc, srcs, objdir, ptxas_info, verbose, defines)
                link = [nvcc] + NVCC_ARCH + ["-shared", "-Xcompiler", "-fPIC", "-o", lib] + objs
                if verbose:
                    print(" ".join(link))
                _compile(link, lib)
            finally:
                for o in objs:
                    if os.path.exists(o):
                        os.remove(o)
            _finish(lib, digest)
    return lib


def build_all(force=False, verbose=False):
    return build_host(force, verbose), build_cuda(force, verbose)


if __name__ == "__main__":
    if "--sanitize" in sys.argv:
        print(build_host_sanitized(verbose=True))
        sys.exit(0)
    if "--debug-bounds" in sys.argv:
        print(build_cuda("--force" in sys.argv, verbose=True, debug_bounds=True))
        sys.exit(0)
    force = "--force" in sys.argv
    print(build_host(force, verbose=True))
    print(build_cuda(force, verbose=True, ptxas_info="--ptxas" in sys.argv))
