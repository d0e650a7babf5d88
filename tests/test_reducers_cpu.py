"""T1/T2 on CPU: reducer semantics with one worker and with gloo ranks, parity against the
reference's own reducer classes where those are deterministic."""
import os
import sys

import pytest
import torch
import torch.distributed as dist

from gradient_compression_b200 import ops, reducers as R
from gradient_compression_b200.ops import philox

from .conftest import reference_dir

REFERENCE_DIR = reference_dir() or ""
SHAPES = [(16, 3, 3, 3), (16,), (32, 16, 3, 3), (32,), (10, 32), (10,)]
CFG = dict(seed=42, K=50, quantization_level=4, higher_quantization_level=8, quantization_levels=[2, 6, 10],
           compression=0.1, rank=2)


def _grads(seed):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(s, generator=g) * 1e-2 for s in SHAPES]


def _flat(ts):
    return torch.cat([t.reshape(-1) for t in ts])


def test_registry_has_every_reference_reducer():
    expected = {"NoneReducer", "NoneAllReducer", "QSGDReducer", "QSGDWECReducer", "QSGDWECModReducer",
                "TernGradReducer", "TernGradModReducer", "QSGDMaxNormReducer", "QSGDBPReducer", "QSGDBPAllReducer",
                "GlobalRandKMaxNormReducer", "NUQSGDModReducer", "NUQSGDMaxNormReducer", "TopKReducer",
                "TopKReducerRatio", "GlobalTopKReducer", "GlobalTopKReducerRatio", "QSGDMaxNormBiasedReducer",
                "QSGDMaxNormBiasedMemoryReducer", "NUQSGDMaxNormBiasedReducer", "NUQSGDMaxNormBiasedMemoryReducer",
                "QSGDMaxNormTwoScaleReducer", "GlobalRandKMaxNormTwoScaleReducer", "QSGDMaxNormMultiScaleReducer",
                "RankKReducer"}
    assert expected == set(R.REDUCERS)
    with pytest.raises(NotImplementedError):
        R.make_reducer("QSGDMaxNormMaskReducer", "cpu")


@pytest.mark.parametrize("name", sorted(R.REDUCERS))
def test_every_reducer_runs_single_worker(name):
    red = R.make_reducer(name, "cpu", None, CFG)
    for step in range(2):
        grads = _grads(step)
        send = [g.clone() for g in grads]
        bits = red.reduce(send, grads)
        assert bits > 0 and all(torch.isfinite(g).all() for g in grads)
        assert [g.shape for g in grads] == [torch.Size(s) for s in SHAPES]


def test_allreduce_identity_and_bits():
    grads = _grads(0)
    ref = [g.clone() for g in grads]
    bits = R.NoneAllReducer("cpu").reduce([g.clone() for g in grads], grads)
    assert all(torch.equal(a, b) for a, b in zip(grads, ref))
    assert bits == 32 * sum(g.numel() for g in grads)


def test_qsgd_maxnorm_matches_oracle_formula_and_bits():
    grads = _grads(1)
    flat = _flat(grads)
    red = R.QSGDMaxNormReducer("cpu", quantization_level=4, seed=42)
    out = [torch.empty_like(g) for g in grads]
    bits = red.reduce([g.clone() for g in grads], out)
    norm = flat.abs().max()
    q = ops.quantize_levels(flat, norm, 15, 42, philox.stream_id(0, philox.PURPOSE_ROUND), 0)
    assert torch.equal(_flat(out), ops.dequantize_levels(q, norm, 15, 1))
    n = flat.numel()
    assert bits == 32 + 8 * n                       # reference accounting: int8 container below 8 bits
    assert R.QSGDMaxNormReducer("cpu", quantization_level=8).reduce([g.clone() for g in grads], out) == 32 + 32 * n
    assert red.last_wire_bits == 32 + 8 * sum(ops.packed_sizes(n, 4))


def test_zero_copy_flat_views():
    flat = torch.randn(sum(torch.Size(s).numel() for s in SHAPES)) * 1e-2
    views, off = [], 0
    for s in SHAPES:
        k = torch.Size(s).numel()
        views.append(flat[off:off + k].view(s))
        off += k
    buf = R.TensorBuffer(views)
    assert buf.is_view and buf.buffer.data_ptr() == flat.data_ptr() and len(buf) == len(SHAPES)
    assert buf[2].shape == torch.Size(SHAPES[2])
    before = flat.clone()
    R.QSGDMaxNormReducer("cpu", quantization_level=8).reduce(views, views)   # in place through the views
    assert not torch.equal(flat, before) and (flat - before).abs().max() < before.abs().max() / 255 * 1.01
    assert not R.TensorBuffer([torch.randn(3), torch.randn(4)]).is_view


def test_twoscale_values_fit_low_range_and_unbiased():
    x = torch.randn(4000) * 1e-2
    est = torch.zeros_like(x)
    red = R.QSGDMaxNormTwoScaleReducer("cpu", lower_quantization_level=2, higher_quantization_level=6, seed=1)
    T = 300
    for _ in range(T):
        out = [torch.empty_like(x)]
        red.reduce([x.clone()], out)
        est += out[0]
    norm = x.abs().max()
    assert (est / T - x).abs().max() < 5 * norm / 3 / T ** 0.5
    small = x.abs() < norm * 2.5 / 63          # these almost always ride the fine scale
    assert (out[0][small] - x[small]).abs().max() <= norm / 63 * 1.001


def test_multiscale_index_rule():
    x = torch.tensor([1.0, 0.5, 0.04, 0.001, -0.2])
    red = R.QSGDMaxNormMultiScaleReducer("cpu", quantization_levels=[2, 6, 10], seed=3)
    out = [torch.empty_like(x)]
    red.reduce([x.clone()], out)
    # |x|/norm * s_l must stay <= 3 for the chosen scale l: 1.0 -> scale 0, 0.04 -> scale 1, 0.001 -> scale 2
    assert abs(out[0][0] - 1.0) < 1e-6
    assert abs(out[0][2] - 0.04) <= 1 / 63 + 1e-6 and abs(out[0][3] - 0.001) <= 1 / 1023 + 1e-6


def test_randk_visits_every_coordinate_once_per_pass():
    n, K = 1000, 64
    red = R.GlobalRandKMaxNormReducer("cpu", seed=5, K=K, quantization_level=8, unselected="zero")
    seen = torch.zeros(n)
    steps = (n + K - 1) // K
    for _ in range(steps):
        x = torch.ones(n)
        out = [torch.empty(n)]
        bits = red.reduce([x.clone()], out)
        seen += (out[0] != 0).float()
    assert torch.equal(seen, torch.ones(n))
    assert bits == 32 + 32 * (n - (steps - 1) * K)
    red.reduce([torch.ones(n)], out)          # next pass starts over with the same permutation
    assert int((out[0] != 0).sum()) == K


def test_topk_error_feedback_telescopes():
    red = R.TopKReducer("cpu", K=5)
    total_in, total_out = torch.zeros(sum(torch.Size(s).numel() for s in SHAPES)), 0
    for step in range(4):
        grads = _grads(10 + step)
        total_in += _flat(grads)
        out = [torch.empty_like(g) for g in grads]
        bits = red.reduce([g.clone() for g in grads], out)
        total_out = total_out + _flat(out)
        nz = [int((o != 0).sum()) for o in out]
        assert nz == [min(5, o.numel()) for o in out]
    assert torch.allclose(total_out + red._memory, total_in, atol=1e-6)
    assert bits == 64 * sum(min(5, torch.Size(s).numel()) for s in SHAPES)
    ratio = R.TopKReducerRatio("cpu", compression=0.1)
    out = [torch.empty_like(g) for g in grads]
    ratio.reduce([g.clone() for g in grads], out)
    assert [int((o != 0).sum()) for o in out] == [max(1, int(0.1 * o.numel())) for o in out]


def test_global_topk_modes():
    grads = _grads(3)
    flat = _flat(grads)
    out = [torch.empty_like(g) for g in grads]
    bits = R.GlobalTopKReducer("cpu", K=20).reduce([g.clone() for g in grads], out)
    o = _flat(out)
    idx = torch.topk(flat.abs(), 20)[1]
    expect = torch.zeros_like(flat)
    expect[idx] = flat[idx]
    assert torch.equal(o, expect) and bits == 96 * 20
    compat = R.GlobalTopKReducer("cpu", K=20, reference_compat=True)
    compat.reduce([g.clone() for g in grads], out)
    expect2 = flat.clone()
    expect2[idx] += flat[idx]
    assert torch.allclose(_flat(out), expect2)


def test_powersgd_matches_dense_restatement():
    grads = _grads(4)
    red = R.RankKReducer("cpu", rank=2, seed=9)
    out = [torch.empty_like(g) for g in grads]
    bits = red.reduce([g.clone() for g in grads], out)
    qflat = philox.normal(red._layout["q_total"], 9, philox.stream_id(0, philox.PURPOSE_QINIT), 0)
    for (i, n, m, r, po, qo) in red._layout["hi"]:
        M = grads[i].view(n, m)
        Q = qflat[qo:qo + m * r].view(m, r)
        P = M @ Q
        ops.gram_schmidt_(P)
        approx = P @ (M.t() @ P).t()
        assert torch.allclose(out[i].view(n, m), approx, atol=1e-5)
        s, e = sum(torch.Size(x).numel() for x in SHAPES[:i]), sum(torch.Size(x).numel() for x in SHAPES[:i + 1])
        assert torch.allclose(red._memory[s:e].view(n, m), M - approx, atol=1e-5)
    for i in red._layout["lo"]:
        assert torch.equal(out[i], grads[i])
    total = red._layout["p_elems"] + red._layout["q_elems"] + sum(grads[i].numel() for i in red._layout["lo"])
    assert bits == 32 * total
    # error feedback: second step adds the memory first
    g2 = _grads(5)
    mem = red._memory.clone()
    red.reduce([g.clone() for g in g2], out)
    hi_mask = torch.cat([torch.full((g.numel(),), float(g.dim() > 1)) for g in g2]).bool()
    assert torch.allclose((_flat(out) + red._memory)[hi_mask], (_flat(g2) + mem)[hi_mask], atol=1e-6)


def test_biased_memory_fix_and_compat():
    grads = _grads(6)
    fixed = R.QSGDMaxNormBiasedMemoryReducer("cpu", quantization_level=4)
    out = [torch.empty_like(g) for g in grads]
    fixed.reduce([g.clone() for g in grads], out)
    assert torch.allclose(fixed._memory, _flat(grads) - _flat(out), atol=1e-7)
    assert fixed._memory.abs().max() <= _flat(grads).abs().max() / 15 * 1.001
    compat = R.QSGDMaxNormBiasedMemoryReducer("cpu", quantization_level=4, reference_compat=True)
    compat.reduce([g.clone() for g in grads], out)
    assert compat._memory.abs().max() >= 1.0      # grad minus integer levels, as in the reference


def test_state_dict_roundtrip():
    red = R.GlobalRandKMaxNormReducer("cpu", seed=5, K=64, quantization_level=4)
    x = torch.randn(1000)
    red.reduce([x.clone()], [torch.empty(1000)])
    sd = red.state_dict()
    a, b = [torch.empty(1000)], [torch.empty(1000)]
    red.reduce([x.clone()], a)
    red2 = R.GlobalRandKMaxNormReducer("cpu", seed=5, K=64, quantization_level=4)
    red2.load_state_dict(sd)
    red2.reduce([x.clone()], b)
    assert torch.equal(a[0], b[0])


# ------------------------------------------------------------------------------- gloo ranks
def _gloo_body(rank, world):
    torch.manual_seed(0)
    shapes_n = sum(torch.Size(s).numel() for s in SHAPES)
    per_rank = [_grads(100 + r) for r in range(world)]
    mine = per_rank[rank]
    mean = sum(_flat(g) for g in per_rank) / world

    out = [torch.empty_like(g) for g in mine]
    R.NoneAllReducer("cpu").reduce([g.clone() for g in mine], out)
    assert torch.allclose(_flat(out), mean, atol=1e-7)
    R.NoneReducer("cpu").reduce([g.clone() for g in mine], out)
    assert torch.allclose(_flat(out), mean, atol=1e-7)

    # QSGD-MN: exact against the oracle evaluated for every rank's stream
    red = R.QSGDMaxNormReducer("cpu", quantization_level=4, seed=42)
    red.reduce([g.clone() for g in mine], out)
    norm = max(_flat(g).abs().max() for g in per_rank)
    tot = sum(ops.quantize_levels(_flat(per_rank[r]), norm, 15, 42, philox.stream_id(r, philox.PURPOSE_ROUND), 0)
              for r in range(world))
    assert torch.equal(_flat(out), ops.dequantize_levels(tot.to(torch.int32), norm, 15, world))

    # two-scale: the AND of the masks must make every rank use the same scale per element
    ts = R.QSGDMaxNormTwoScaleReducer("cpu", lower_quantization_level=2, higher_quantization_level=6, seed=42)
    ts.reduce([g.clone() for g in mine], out)
    gathered = [torch.empty(shapes_n) for _ in range(world)]
    dist.all_gather(gathered, _flat(out))
    assert all(torch.equal(gathered[0], g) for g in gathered)
    assert (_flat(out) - mean).abs().max() <= norm / 3 * 1.001

    # every other reducer at least agrees across ranks on the result (shared index sets / norms)
    for name in ["GlobalRandKMaxNormReducer", "GlobalRandKMaxNormTwoScaleReducer", "QSGDMaxNormMultiScaleReducer",
                 "TopKReducer", "GlobalTopKReducer", "QSGDWECModReducer", "TernGradReducer", "QSGDReducer",
                 "QSGDBPReducer", "QSGDBPAllReducer", "NUQSGDMaxNormReducer"]:
        cfg = dict(CFG)
        cfg["unselected"] = "zero"
        r_ = R.make_reducer(name, "cpu", None, cfg)
        if "RandK" in name:
            r_._unselected = "zero"
        r_.reduce([g.clone() for g in mine], out)
        dist.all_gather(gathered, _flat(out))
        assert all(torch.equal(gathered[0], g) for g in gathered), name

    # TopK: exact mean of sparse contributions
    tk = R.TopKReducer("cpu", K=5)
    tk.reduce([g.clone() for g in mine], out)
    expect = torch.zeros(shapes_n)
    off = 0
    for i, s in enumerate(SHAPES):
        k = torch.Size(s).numel()
        for r in range(world):
            t = per_rank[r][i].reshape(-1)
            idx = torch.topk(t.abs(), min(5, k))[1]
            expect[off + idx] += t[idx] / world
        off += k
    assert torch.allclose(_flat(out), expect, atol=1e-7)

    # PowerSGD: same as the dense restatement on the mean of M (linear in M before orthogonalisation)
    pr = R.RankKReducer("cpu", rank=1, seed=9)
    pr.reduce([g.clone() for g in mine], out)
    qflat = philox.normal(pr._layout["q_total"], 9, philox.stream_id(0, philox.PURPOSE_QINIT), 0)
    for (i, n, m, r, po, qo) in pr._layout["hi"]:
        Ms = [per_rank[w][i].view(n, m) for w in range(world)]
        Q = qflat[qo:qo + m * r].view(m, r)
        P = sum(M @ Q for M in Ms)
        ops.gram_schmidt_(P)
        Qn = sum(M.t() @ P for M in Ms) / world
        assert torch.allclose(out[i].view(n, m), P @ Qn.t(), atol=1e-5)
    for i in pr._layout["lo"]:
        assert torch.allclose(out[i], sum(per_rank[w][i] for w in range(world)) / world, atol=1e-7)


@pytest.mark.parametrize("world", [2, 3])
def test_reducers_across_gloo_ranks(dist_runner, world):
    dist_runner(_gloo_body, world=world)


# ------------------------------------------------------------------------------- reference as oracle
def _reference_body(rank, world):
    sys.path.insert(0, REFERENCE_DIR)
    import reducer as ref   # the reference's module, imported unmodified

    class _T:               # the reference's Timer interface, doing nothing
        def __call__(self, *a, **k):
            import contextlib
            return contextlib.nullcontext()

    mine = _grads(200 + rank)
    for ours_cls, ref_cls, kw in [(R.NoneAllReducer, ref.NoneAllReducer, {}), (R.TopKReducer, ref.TopKReducer, {"K": 7}),
                                  (R.TopKReducerRatio, ref.TopKReducerRatio, {"compression": 0.05})]:
        ours, theirs = ours_cls("cpu", None, **kw), ref_cls("cpu", _T(), **kw)
        for step in range(3):
            g = _grads(300 + 10 * step + rank)
            o1 = [torch.empty_like(t) for t in g]
            o2 = [torch.zeros_like(t) for t in g]
            b1 = ours.reduce([t.clone() for t in g], o1)
            b2 = theirs.reduce([t.clone() for t in g], o2)
            assert b1 == b2, ours_cls.__name__
            assert torch.allclose(_flat(o1), _flat(o2), atol=1e-7), ours_cls.__name__
    # bits accounting of the quantised family matches the reference's containers
    for name, kw in [("QSGDMaxNormReducer", {"quantization_level": 4}), ("QSGDMaxNormReducer", {"quantization_level": 8}),
                     ("QSGDMaxNormTwoScaleReducer", {"lower_quantization_level": 2, "higher_quantization_level": 6}),
                     ("GlobalRandKMaxNormReducer", {"K": 6, "quantization_level": 4, "seed": 1}),  # K divides N: the reference pops its remainder chunk first
                     ("RankKReducer", {"rank": 1})]:
        ours, theirs = getattr(R, name)("cpu", None, **kw), getattr(ref, name)("cpu", _T(), **kw)
        o = [torch.zeros_like(t) for t in mine]
        assert ours.reduce([t.clone() for t in mine], o) == theirs.reduce([t.clone() for t in mine], o), name


def _near_max_body(rank, world):
    # every rank holds the same tensor with most entries at +-max: each contributes level +-63 at 6 bits, the sum of four
    # (252) does not fit the int8 container the levels are produced in
    g = torch.Generator().manual_seed(3)
    x = torch.where(torch.rand(4096, generator=g) < 0.5, -1.0, 1.0) * 2.5
    x[::7] = torch.randn(586, generator=g).clamp(-2.5, 2.5)[: x[::7].numel()]
    out = [torch.empty_like(x)]
    spike = torch.zeros(4096)
    spike[5], spike[77] = 10.0, -1e-3          # one entry carries the whole L2 norm: its non-uniform level is 2**7 = 128
    for cls, kw, s in ((R.QSGDMaxNormReducer, {"quantization_level": 6}, 63), (R.NUQSGDMaxNormReducer, {"quantization_level": 7}, 128)):
        red = cls("cpu", seed=11, **kw)
        x = x if s == 63 else spike
        red.reduce([x.clone()], out)
        norm = x.abs().max() if s == 63 else torch.norm(x)
        mode = ops.MODE_STOCHASTIC if s == 63 else ops.MODE_NU
        tot = sum(ops.quantize_levels(x, norm, s, 11, philox.stream_id(r, philox.PURPOSE_ROUND), 0, mode=mode, dtype=torch.int32)
                  for r in range(world))
        assert int(tot.abs().max()) > 127
        assert torch.equal(out[0], ops.dequantize_levels(tot, norm, s, world))
    # the reference's behaviour (the int8 sum wraps) stays available
    x = torch.full((256,), 2.5)
    wrapped = [torch.empty_like(x)]
    R.QSGDMaxNormReducer("cpu", seed=11, quantization_level=6, reference_compat=True).reduce([x.clone()], wrapped)
    assert float((wrapped[0] - x).abs().max()) > 2.0


def test_level_sums_do_not_wrap_in_their_container(dist_runner):
    dist_runner(_near_max_body, world=4)


@pytest.mark.skipif(not os.path.exists(os.path.join(REFERENCE_DIR, "reducer.py")), reason="reference sources not mounted")
def test_parity_with_reference_reducers(dist_runner):
    dist_runner(_reference_body, world=2)
