import os
import socket
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords or "multigpu" in item.keywords:
            item.add_marker(skip)


def reference_dir():
    """Where the reference project's sources are: ``$GRADCOMP_REFERENCE_DIR``, else the copy installed for the benchmark's
    reference arm under ``baseline/_ref`` of this checkout; None when neither exists (tests that need it skip)."""
    env = os.environ.get("GRADCOMP_REFERENCE_DIR")
    if env:
        return env if os.path.isdir(env) else None
    local = os.path.join(ROOT, "baseline", "_ref")
    return local if os.path.exists(os.path.join(local, "reducer.py")) else None


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, fn, args, backend):
    import torch.distributed as dist

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    if backend == "nccl":
        torch.cuda.set_device(rank)
    dist.init_process_group(backend, rank=rank, world_size=world)
    try:
        fn(rank, world, *args)
    finally:
        dist.destroy_process_group()


def run_distributed(fn, world=2, args=(), backend="gloo"):
    """Run ``fn(rank, world, *args)`` in ``world`` spawned processes with a process group."""
    import torch.multiprocessing as mp

    mp.spawn(_worker, args=(world, free_port(), fn, args, backend), nprocs=world, join=True)


@pytest.fixture
def dist_runner():
    return run_distributed
