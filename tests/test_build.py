"""In-tree native build: stamps do not depend on where the tree lives, and concurrent builders do not clobber each other."""
import importlib.util
import os
import shutil
import subprocess
import sys

import gradient_compression_b200 as pkg


def _load_build(path):
    spec = importlib.util.spec_from_file_location("gcb200_build_copy", os.path.join(path, "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _copy_tree(dst):
    src = os.path.dirname(pkg.__file__)
    os.makedirs(dst)
    shutil.copy(os.path.join(src, "build.py"), dst)
    shutil.copytree(os.path.join(src, "csrc"), os.path.join(dst, "csrc"))
    return dst


def test_concurrent_builds_and_relocation(tmp_path):
    a = _copy_tree(str(tmp_path / "a"))
    code = ("import importlib.util, ctypes, sys; spec = importlib.util.spec_from_file_location('b', sys.argv[1] + '/build.py'); "
            "b = importlib.util.module_from_spec(spec); spec.loader.exec_module(b); ctypes.CDLL(b.build_host()); print('ok')")
    procs = [subprocess.Popen([sys.executable, "-c", code, a], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True)
             for _ in range(4)]
    outs = [p.communicate(timeout=300) for p in procs]
    assert all(p.returncode == 0 and "ok" in o[0] for p, o in zip(procs, outs)), outs
    assert not [f for f in os.listdir(os.path.join(a, "_lib")) if ".tmp" in f]
    # the same tree somewhere else: the library that travelled with it is current
    b_dir = str(tmp_path / "b")
    shutil.copytree(a, b_dir)
    b = _load_build(b_dir)
    lib = b.host_lib_path()
    before = os.path.getmtime(lib)
    assert b.build_host() == lib and os.path.getmtime(lib) == before
    # a changed source makes it stale
    with open(os.path.join(b_dir, "csrc", "host_oracle.cpp"), "a") as f:
        f.write("\n// touched\n")
    b.build_host()
    assert os.path.getmtime(lib) > before
