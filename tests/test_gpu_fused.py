"""T4 on one GPU: the fused compress+collective kernels with W ranks emulated inside ONE cooperative
launch (``LocalGroup``), compared bit for bit against the CPU oracle evaluated per rank."""
import pytest
import torch

from gradient_compression_b200 import ops
from gradient_compression_b200.ops import philox

pytestmark = pytest.mark.gpu


def _inputs(world, n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(n, generator=g) * (1e-3 * (r + 1)) for r in range(world)]


def _group(world, n):
    from gradient_compression_b200.parallel import comm
    from gradient_compression_b200.parallel.engine import FusedOps

    grp = comm.LocalGroup(world, comm.required_bytes(n))
    return grp, FusedOps(grp, timeout_ms=5000)


def _oracle_qsgd(xs, bits, seed, step):
    world, s = len(xs), (1 << bits) - 1
    norm = max(float(x.abs().max()) for x in xs)
    tot = sum(ops.quantize_levels(x, norm, s, seed, philox.stream_id(r, philox.PURPOSE_ROUND), step).to(torch.int32)
              for r, x in enumerate(xs))
    return ops.dequantize_levels(tot.to(torch.int32), norm, s, world)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("n,bits", [(1, 4), (4099, 2), (4099, 4), (100003, 8), (100003, 12), ((1 << 20) + 3, 4)])
def test_fused_qsgd_emulated(world, n, bits):
    grp, fo = _group(world, n)
    try:
        xs = _inputs(world, n, n + bits)
        ins = [x.cuda() for x in xs]
        outs = [torch.empty(n, device="cuda") for _ in range(world)]
        for step in range(2):          # two calls: epochs advance, buffers are reused
            fo.qsgd(ins, outs, bits, 42, step)
            fo.check()
            expect = _oracle_qsgd(xs, bits, 42, step)
            for o in outs:
                assert torch.equal(o.cpu(), expect)
    finally:
        grp.close()


@pytest.mark.parametrize("world", [1, 2, 8])
def test_fused_qsgd_in_place(world):
    n = 50001
    grp, fo = _group(world, n)
    try:
        xs = _inputs(world, n, 7)
        bufs = [x.cuda() for x in xs]
        fo.qsgd(bufs, bufs, 4, 1, 0)
        fo.check()
        expect = _oracle_qsgd(xs, 4, 1, 0)
        assert all(torch.equal(b.cpu(), expect) for b in bufs)
    finally:
        grp.close()


def _oracle_twoscale(xs, lo, hi, seed, step):
    world, s_lo, s_hi = len(xs), (1 << lo) - 1, (1 << hi) - 1
    norm = max(float(x.abs().max()) for x in xs)
    q_lo = [ops.quantize_levels(x, norm, s_lo, seed, philox.stream_id(r, philox.PURPOSE_ROUND), step) for r, x in enumerate(xs)]
    q_hi = [ops.quantize_levels(x, norm, s_hi, seed, philox.stream_id(r, philox.PURPOSE_ROUND_HI), step) for r, x in enumerate(xs)]
    mask = torch.ones_like(q_lo[0], dtype=torch.bool)
    for q in q_hi:
        mask &= q.abs() <= s_lo
    tot = sum(torch.where(mask, h, l) for h, l in zip(q_hi, q_lo))
    a = ops.dequantize_levels(tot.to(torch.int32), norm, s_hi, world)
    b = ops.dequantize_levels(tot.to(torch.int32), norm, s_lo, world)
    return torch.where(mask, a, b)


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("n,lo,hi", [(4099, 2, 6), (100003, 6, 10), (100003, 8, 12)])
def test_fused_twoscale_emulated(world, n, lo, hi):
    grp, fo = _group(world, n)
    try:
        xs = _inputs(world, n, n + lo)
        ins = [x.cuda() for x in xs]
        outs = [torch.empty(n, device="cuda") for _ in range(world)]
        for step in range(2):
            fo.twoscale(ins, outs, lo, hi, 9, step)
            fo.check()
            expect = _oracle_twoscale(xs, lo, hi, 9, step)
            for o in outs:
                assert torch.equal(o.cpu(), expect)
    finally:
        grp.close()


def _oracle_multiscale(xs, levels, seed, step):
    world = len(xs)
    s = [(1 << b) - 1 for b in levels]
    norm = max(float(x.abs().max()) for x in xs)
    q = [[ops.quantize_levels(x, norm, s[l], seed, philox.stream_id(r, philox.PURPOSE_LEVEL0 + l), step) for l in range(len(s))]
         for r, x in enumerate(xs)]
    idx = None
    for r in range(world):
        mine = torch.zeros_like(q[r][0])
        for l in range(1, len(s)):
            mine[q[r][l].abs() <= s[0]] = l
        idx = mine if idx is None else torch.minimum(idx, mine)
    tot = torch.zeros_like(q[0][0])
    for r in range(world):
        for l in range(len(s)):
            tot += torch.where(idx == l, q[r][l], torch.zeros_like(tot))
    out = torch.zeros(xs[0].numel())
    for l in range(len(s)):
        out = torch.where(idx == l, ops.dequantize_levels(tot.to(torch.int32), norm, s[l], world), out)
    return out


@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("n,levels", [(4099, [2, 6]), (100003, [2, 6, 10]), (100003, [4, 8, 12, 16]), (50001, [8, 12])])
def test_fused_multiscale_emulated(world, n, levels):
    grp, fo = _group(world, n)
    try:
        xs = _inputs(world, n, n + len(levels))
        outs = [torch.empty(n, device="cuda") for _ in range(world)]
        for step in range(2):
            fo.multiscale([x.cuda() for x in xs], outs, levels, 5, step)
            fo.check()
            expect = _oracle_multiscale(xs, levels, 5, step)
            for o in outs:
                assert torch.equal(o.cpu(), expect)
    finally:
        grp.close()


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("n", [5, 4099, (1 << 20) + 3])
def test_fused_allreduce_emulated(world, n):
    grp, fo = _group(world, n)
    try:
        xs = _inputs(world, n, n)
        outs = [torch.empty(n, device="cuda") for _ in range(world)]
        fo.allreduce([x.cuda() for x in xs], outs)
        fo.check()
        acc = xs[0].clone()
        for x in xs[1:]:
            acc += x               # same left-to-right order as the kernel
        expect = acc * (1.0 / world)
        for o in outs:
            assert torch.equal(o.cpu(), expect)
        small = [torch.empty(n, device="cuda") for _ in range(world)]
        fo.small_sum([x.cuda() for x in xs], small, alpha=0.5)
        fo.check()
        acc = torch.zeros(n)
        for x in xs:
            acc += x
        assert all(torch.equal(o.cpu(), acc * 0.5) for o in small)
    finally:
        grp.close()


@pytest.mark.parametrize("world", [2, 4])
def test_one_shot_launches_of_alternating_sizes_share_one_arena(world):
    """PowerSGD's P and Q sums, Rand-K windows and bucketed reducers launch one-shot kernels of different sizes on one arena,
    back to back and with no closing round.  The two parity regions sit a fixed distance apart (a function of the arena,
    not of the call), so a small launch after a large one must not land in the region the previous launch's readers may
    still use: every result of a long alternating sequence has to be exact."""
    n = (1 << 18) + 3
    grp, fo = _group(world, n)
    try:
        sizes = [n, 7, 4099, n, 129, 65537, 5, n, 4099, 7]
        g = torch.Generator().manual_seed(world)
        for step, m in enumerate(sizes * 2):
            xs = [torch.randn(m, generator=g) for _ in range(world)]
            outs = [torch.empty(m, device="cuda") for _ in range(world)]
            fo.small_sum([x.cuda() for x in xs], outs, alpha=0.25)
            acc = torch.zeros(m)
            for x in xs:
                acc += x
            assert all(torch.equal(o.cpu(), acc * 0.25) for o in outs), (step, m)
        fo.check()
    finally:
        grp.close()


@pytest.mark.parametrize("world", [1, 2, 8])
@pytest.mark.parametrize("hi", [0, 6])
@pytest.mark.parametrize("zero", [False, True])
def test_fused_randk_emulated(world, hi, zero):
    n, k, start, lo, seed = 100003, 1000, 3000, 2 if hi else 4, 11
    grp, fo = _group(world, n)
    try:
        xs = _inputs(world, n, 5)
        outs = [torch.empty(n, device="cuda") for _ in range(world)]
        fo.randk([x.cuda() for x in xs], outs, seed, 0, start, k, lo, hi, zero, step=3)
        fo.check()
        idx = ops.randk_indices(seed, n, start, k)
        sel = [x[idx] for x in xs]
        vals = _oracle_twoscale(sel, lo, hi, seed, 3) if hi else _oracle_qsgd(sel, lo, seed, 3)
        for r, o in enumerate(outs):
            expect = torch.zeros(n) if zero else xs[r] * (1.0 / world)
            expect[idx] = vals
            assert torch.equal(o.cpu(), expect), (r, world)
    finally:
        grp.close()


@pytest.mark.parametrize("world", [1, 2, 8])
def test_fused_sparse_exchange_emulated(world):
    n, count = 100003, 777
    grp, fo = _group(world, n)
    try:
        g = torch.Generator().manual_seed(world)
        idxs = [torch.randperm(n, generator=g)[:count].to(torch.int32) for _ in range(world)]
        vals = [torch.randn(count, generator=g) for _ in range(world)]
        outs = [torch.full((n,), 7.0, device="cuda") for _ in range(world)]
        for _ in range(2):
            fo.sparse([v.cuda() for v in vals], outs, [i.cuda() for i in idxs], 1.0 / world)
            fo.check()
            expect = torch.zeros(n)
            for i, v in zip(idxs, vals):       # rank order, as in the kernel
                expect[i.long()] += (1.0 / world) * v
            for o in outs:
                assert torch.equal(o.cpu(), expect)
    finally:
        grp.close()


def test_bounded_wait_reports_timeout_and_context_survives():
    """A rank whose peers never launch: every wait runs out after the (short) limit, the kernel
    returns, the host reads STATUS_TIMEOUT, and the same context then completes a normal step."""
    from gradient_compression_b200.parallel import comm
    from gradient_compression_b200.parallel.engine import FusedOps

    n = 4099
    grp = comm.LocalGroup(2, comm.required_bytes(n))
    try:
        lonely = comm._ArenaBase()
        lonely.ctxs, lonely.device = (grp.ctxs[0],), grp.device     # launch rank 0 alone: rank 1 never signals
        fo = FusedOps(lonely, timeout_ms=200)
        x = torch.randn(n, device="cuda")
        fo.qsgd([x], [torch.empty_like(x)], 4, 1, 0)
        with pytest.raises(comm.CollectiveTimeout) as e:
            fo.check()
        assert e.value.peer == 1
        torch.cuda.synchronize()
        assert float(ops.absmax(x)) > 0        # the CUDA context is alive
    finally:
        grp.close()


def test_out_of_range_index_is_reported_and_never_followed():
    """An index list with entries outside the tensor (what a buggy caller could hand to the sparse exchange): the kernel
    skips those entries, applies the others, and the host gets STATUS_BOUNDS with the first bad index."""
    from gradient_compression_b200.parallel import comm

    n, count, world = 5003, 64, 2
    grp, fo = _group(world, n)
    try:
        g = torch.Generator().manual_seed(9)
        idxs = [torch.randperm(n, generator=g)[:count].to(torch.int32) for _ in range(world)]
        idxs[1][5] = n + 11                        # outside: must be skipped, not written
        idxs[1][6] = -3
        vals = [torch.randn(count, generator=g) for _ in range(world)]
        canary = torch.full((n + 64,), 7.0, device="cuda")
        outs = [canary[:n], torch.full((n,), 7.0, device="cuda")]
        fo.sparse([v.cuda() for v in vals], outs, [i.cuda() for i in idxs], 1.0 / world)
        with pytest.raises(comm.IndexOutOfBounds) as e:
            fo.check()
        assert e.value.index in (n + 11, -3)
        expect = torch.zeros(n)
        for r, (i, v) in enumerate(zip(idxs, vals)):
            keep = (i >= 0) & (i < n)
            expect[i[keep].long()] += (1.0 / world) * v[keep]
        assert torch.equal(outs[0].cpu(), expect) and torch.equal(outs[1].cpu(), expect)
        assert float(canary[n:].min()) == 7.0 and float(canary[n:].max()) == 7.0      # nothing beyond the tensor was touched
        fo.sparse([v.cuda() for v in vals], outs, [i.clamp(0, n - 1).cuda() for i in idxs], 1.0 / world)
        fo.check()                                 # the status was cleared: a clean launch reports nothing
    finally:
        grp.close()


def test_debug_bounds_build_runs_the_same_kernels():
    """The -DGC_DEBUG_BOUNDS build (every computed gather / scatter index checked before use) in a process of its own:
    Rand-K on an emulated group gives the regular build's result and reports no index, and a bad index handed to the
    sparse exchange is reported there too."""
    import subprocess
    import sys

    code = r'''
import torch
from gradient_compression_b200.ops import _native as nat
from gradient_compression_b200.parallel import comm
from gradient_compression_b200.parallel.engine import FusedOps
assert nat.cuda().gc_comm_debug_bounds() == 1
n, world = 40003, 2
grp = comm.LocalGroup(world, comm.required_bytes(n))
fo = FusedOps(grp, timeout_ms=5000)
xs = [torch.randn(n, generator=torch.Generator().manual_seed(r)).cuda() for r in range(world)]
outs = [torch.empty(n, device="cuda") for _ in range(world)]
fo.randk(xs, outs, 5, 0, n - 700, 1000, 8, 0, False, 0)     # a window that ends at the edge of the tensor
fo.check()
print("RANDK", float(outs[0].double().sum()), float(outs[1].double().abs().sum()))
idx = [torch.arange(10, dtype=torch.int32).cuda(), torch.tensor([1, 2, n + 1] + [3] * 7, dtype=torch.int32).cuda()]
try:
    fo.sparse([torch.ones(10).cuda()] * 2, outs, idx, 0.5)
    fo.check()
    print("NO ERROR")
except comm.IndexOutOfBounds as e:
    print("BOUNDS", e.index)
grp.close()
'''
    import os

    def run(debug):
        env = dict(os.environ, GCB200_DEBUG_BOUNDS="1" if debug else "0")
        src = code if debug else code.replace("== 1", "== 0")
        out = subprocess.run([sys.executable, "-c", src], env=env, capture_output=True, text=True, timeout=600,
                             cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
        assert out.returncode == 0, out.stderr[-2000:]
        return [l for l in out.stdout.splitlines() if l.startswith(("RANDK", "BOUNDS", "NO ERROR"))]

    dbg, rel = run(True), run(False)
    assert dbg == rel and dbg[1] == f"BOUNDS {40003 + 1}", (dbg, rel)


@pytest.mark.parametrize("world,bits", [(1, 8), (2, 4), (4, 2), (8, 8)])
def test_fused_qsgd_against_a_plain_pytorch_restatement(world, bits):
    """An oracle that shares no code with the kernels: inputs whose levels |x| / norm * s are whole numbers leave the
    stochastic rounding nothing to round (its probability is 0), so the result must be the plain mean of the inputs --
    written here with torch ops only, without the quantiser or the Philox stream of the native library."""
    n = 30011
    s = (1 << bits) - 1
    grp, fo = _group(world, n)
    try:
        g = torch.Generator().manual_seed(world * 100 + bits)
        xs = [torch.randint(-s, s + 1, (n,), generator=g).float() for _ in range(world)]
        xs[0][17] = float(s)                               # the max-norm is exactly s: level = |x|
        scale = 0.03125                                    # a power of two keeps every quotient exact
        ins = [(x * scale).cuda() for x in xs]
        outs = [torch.empty(n, device="cuda") for _ in range(world)]
        fo.qsgd(ins, outs, bits, 1234, 5)
        fo.check()
        levels = torch.stack(xs).sum(0)                    # sum of the signed integer levels
        norm = torch.tensor(s * scale)
        expect = levels * (norm / (s * world))             # dequantise: norm / (s W) * sum of levels, in fp32
        for o in outs:
            assert torch.allclose(o.cpu(), expect, rtol=2e-7, atol=0.0)
            assert torch.allclose(o.cpu(), torch.stack(xs).sum(0) * scale / world, rtol=1e-6, atol=0.0)
    finally:
        grp.close()
