"""Exhaustive interleaving check of the fused collectives' flag / epoch protocol, and proof that the checker finds the
faults the protocol is designed against."""
import pytest

from gradient_compression_b200.parallel import protocol_model as pm
from gradient_compression_b200.parallel.protocol_model import KERNELS, ProtocolViolation, check


@pytest.mark.parametrize("kernel", sorted(KERNELS))
@pytest.mark.parametrize("world,steps", [(2, 4), (3, 2)])
def test_every_kernel_is_safe_over_consecutive_steps(kernel, world, steps):
    assert check([kernel] * steps, world) > 0


def test_powersgd_launch_chain_and_mixed_sequences():
    # PowerSGD: three one-shot sums per training step (P, rank-1 tensors, Q), two training steps
    assert check(["small_sum"] * 6, 2) > 0
    assert check(["small_sum", "small_sum", "qsgd", "small_sum", "allreduce", "small_sum"], 2) > 0
    assert check(["qsgd", "twoscale", "allreduce"], 3) > 0


def _without(kernel, op):
    ops = list(KERNELS[kernel])
    ops.remove(op)
    return ops


def test_seeded_faults_are_found():
    # one-shot sum without the parity double buffer: the fast rank overwrites what the slow one still has to read
    single = [("write_own", "buf"), ("signal", "AUX"), ("wait", "AUX"), ("read_peers", "buf")]
    with pytest.raises(ProtocolViolation, match="later step"):
        check([single] * 2, 2)
    # all-reduce that does not wait for DONE: results are read before every peer has pushed its part
    with pytest.raises(ProtocolViolation, match="stale"):
        check([_without("allreduce", ("wait", "DONE"))], 2)
    # all-reduce without the closing round at all: the next step's staging overwrites a buffer still being reduced
    no_done = [op for op in KERNELS["allreduce"] if op[1:] != ("DONE",) and op != ("read_own", "result")]
    with pytest.raises(ProtocolViolation, match="later step"):
        check([no_done] * 2, 2)
    # READY signalled before the packed levels are written
    early = list(KERNELS["qsgd"])
    i, j = early.index(("write_own", "packed")), early.index(("signal", "READY"))
    early[i], early[j] = early[j], early[i]
    with pytest.raises(ProtocolViolation, match="stale"):
        check([early], 2)
    # a single norm slot per source instead of two: the next step's norm lands before the previous one was read
    with pytest.raises(ProtocolViolation):
        check([[("norm", "single")]] * 2, 2)
    assert check([[("norm",)]] * 4, 2) > 0
    # a wait for a signal nobody sends
    with pytest.raises(ProtocolViolation, match="deadlock"):
        check([[("wait", "READY")]], 2)


def test_grid_barrier_generation_counting():
    from gradient_compression_b200.parallel.protocol_model import check_grid_barrier

    assert check_grid_barrier(nblocks=2, rounds=4) > 0
    assert check_grid_barrier(nblocks=3, rounds=3) > 0
    assert check_grid_barrier(nblocks=4, rounds=2) > 0
    with pytest.raises(ProtocolViolation):          # generation bumped before the count is reset
        check_grid_barrier(nblocks=3, rounds=3, reset_before_release=False)


@pytest.mark.parametrize("kw", [dict(), dict(tiles=4, kblocks=1, stages=3), dict(tiles=3, kblocks=7, stages=2),
                                dict(tiles=6, kblocks=2, stages=5, epilogue_threads=3), dict(tiles=7, kblocks=4, stages=4)])
def test_gemm_pipeline_parities(kw):
    """Stage ring, double-buffered accumulator and their mbarrier parities of the persistent tensor-core GEMM."""
    from gradient_compression_b200.parallel.protocol_model import check_gemm_pipeline

    assert check_gemm_pipeline(**kw) > 0


def test_gemm_pipeline_seeded_faults():
    from gradient_compression_b200.parallel.protocol_model import check_gemm_pipeline

    with pytest.raises(ProtocolViolation):          # producer waits for the wrong parity of a fresh barrier
        check_gemm_pipeline(empty_parity_offset=0)
    with pytest.raises(ProtocolViolation):          # accumulator released after one of two epilogue threads arrived
        check_gemm_pipeline(acc_empty_count=1)
    assert check_gemm_pipeline(acc_buffers=1, tiles=3) > 0      # the arithmetic also holds for a single accumulator


def test_oneshot_buffers_of_different_sizes_need_a_fixed_parity_distance():
    """Consecutive one-shot launches of different sizes (buckets, several reducers on one arena): with the parity-1
    region placed right behind a parity-0 region of the CALL's size, a larger launch overwrites what a slower peer still
    reads from the previous launch; with the regions a fixed distance apart it cannot."""
    for sizes in ([1, 2], [2, 2, 1], [1, 3, 1, 2]):
        with pytest.raises(pm.ProtocolViolation):
            pm.check(pm.oneshot_schedule(sizes, half=None), world=2)
        assert pm.check(pm.oneshot_schedule(sizes, half=3), world=2) > 0
    assert pm.check(pm.oneshot_schedule([1, 2, 1], half=2), world=3) > 0


def test_shared_arena_is_drained_before_it_is_replaced():
    """Replacing a shared arena frees memory that peers have mapped: the old one may only be closed after the drain
    (local synchronise + group barrier) has run, and kernel families never share an arena."""
    from gradient_compression_b200.parallel import engine

    log = []

    class FakeArena:
        def __init__(self, nbytes, device, group):
            self.bytes = nbytes
            log.append(("create", nbytes))

        def close(self):
            log.append(("close", self.bytes))

    def drain(device, group):
        log.append(("drain",))

    grp = object()
    a = engine.shared_arena(100, "fake:0", grp, "oneshot", make=FakeArena, drain=drain)
    assert engine.shared_arena(50, "fake:0", grp, "oneshot", make=FakeArena, drain=drain) is a
    b = engine.shared_arena(200, "fake:0", grp, "oneshot", make=FakeArena, drain=drain)
    assert b is not a and log == [("create", 100), ("drain",), ("close", 100), ("create", 200)]
    c = engine.shared_arena(10, "fake:0", grp, "twoshot", make=FakeArena, drain=drain)
    assert c is not b and log[-1] == ("create", 10)
    for fam in ("oneshot", "twoshot"):
        engine._shared_arena.pop(("fake:0", id(grp), fam))
