"""T0: Philox, quantiser, packed wire layout and the compatibility packers against independent
restatements (pure python / torch)."""
import math

import pytest
import torch

from gradient_compression_b200 import ops
from gradient_compression_b200.ops import packing, philox


def test_philox_matches_pure_python():
    for seed, stream, step, n in [(0, 0, 0, 8), (42, philox.stream_id(3, 1), 7, 37), (2 ** 40 + 5, 999, 2 ** 31, 5)]:
        got = [x & 0xFFFFFFFF for x in philox.u32(n, seed, stream, step).tolist()]
        assert got == philox.philox_reference_u32(n, seed, stream, step)


def test_philox_known_answer():
    # Random123 known-answer vector: counter = key = 0 -> 6627e8d5 e169c58d bc57ac4c 9b00dbd8
    got = [x & 0xFFFFFFFF for x in philox.u32(4, 0, 0, 0).tolist()]
    assert got == [0x6627E8D5, 0xE169C58D, 0xBC57AC4C, 0x9B00DBD8]


def test_uniform_normal_statistics():
    u = philox.uniform(200000, 1, 2, 3)
    assert 0.0 <= float(u.min()) and float(u.max()) < 1.0
    assert abs(float(u.mean()) - 0.5) < 5e-3
    z = philox.normal(200000, 1, 2, 3)
    assert abs(float(z.mean())) < 1e-2 and abs(float(z.std()) - 1.0) < 1e-2
    # streams differ by rank, agree for the same key
    assert not torch.equal(philox.uniform(64, 1, philox.stream_id(0, 1)), philox.uniform(64, 1, philox.stream_id(1, 1)))
    assert torch.equal(philox.uniform(64, 9, 5, 2), philox.uniform(64, 9, 5, 2))


def _torch_quant(x, norm, s, u):
    l = x.abs() * (torch.tensor(float(s)) / norm)
    fl = l.floor()
    xi = fl + (u < (l - fl)).float()
    xi = torch.where(l < s, xi, torch.full_like(xi, s))
    return (torch.sign(x) * xi).to(torch.int32)


@pytest.mark.parametrize("bits", [1, 2, 4, 6, 8, 12])
@pytest.mark.parametrize("n", [1, 31, 1000, 4099])
def test_quantize_matches_torch_restatement(bits, n):
    g = torch.Generator().manual_seed(n + bits)
    x = torch.randn(n, generator=g) * 1e-3
    norm = ops.absmax(x)
    assert float(norm) == float(x.abs().max())
    s = (1 << bits) - 1
    q = ops.quantize_levels(x, norm, s, 42, 257, 5)
    u = philox.uniform(n, 42, 257, 5)
    assert torch.equal(q, _torch_quant(x, norm[0], s, u))
    assert int(q.abs().max()) <= s


def test_quantize_unbiased_and_bounded_variance():
    x = torch.randn(2000) * 1e-2
    norm = ops.absmax(x)
    s = 15
    acc = torch.zeros_like(x)
    T = 400
    for t in range(T):
        acc += ops.dequantize_levels(ops.quantize_levels(x, norm, s, 7, 1, t), norm, s)
    err = (acc / T - x).abs().max()
    assert float(err) < 4 * float(norm) / s / math.sqrt(T)


def test_zero_norm_and_nonfinite_guard():
    x = torch.zeros(100)
    q = ops.quantize_levels(x, ops.absmax(x), 255, 1, 1, 1)
    assert int(q.abs().max()) == 0
    assert torch.isfinite(ops.dequantize_levels(q, 0.0, 255)).all()
    y = torch.tensor([1.0, float("nan"), -2.0])
    assert math.isinf(float(ops.absmax(y)))


def test_biased_and_nonuniform_modes():
    x = torch.tensor([0.9, -0.49, 0.26, 0.0, 1.0, -1.0])
    q = ops.quantize_levels(x, 1.0, 3, mode=ops.MODE_BIASED)
    assert q.tolist() == [2, -1, 0, 0, 3, -3]
    qb = ops.quantize_levels(x, 1.0, 8, mode=ops.MODE_NU_BIASED)   # r = |x| * 8 -> floor to a power of two
    assert qb.tolist() == [4, -2, 2, 0, 8, -8]
    qs = ops.quantize_levels(x.repeat(500), 1.0, 8, 3, 4, 5, mode=ops.MODE_NU)
    vals = set(qs.abs().tolist())
    assert vals <= {0, 1, 2, 4, 8}
    est = ops.dequantize_levels(qs, 1.0, 8).view(500, -1).mean(0)
    assert torch.allclose(est, x, atol=0.05)


@pytest.mark.parametrize("bits", [1, 2, 3, 4, 7, 8, 12, 16])
@pytest.mark.parametrize("n", [1, 127, 128, 129, 1000])
def test_wire_pack_roundtrip(bits, n):
    s = (1 << bits) - 1
    q = torch.randint(-s, s + 1, (n,), dtype=torch.int32)
    mags, signs = ops.pack_levels(q, bits)
    mb, pb = ops.packed_sizes(n, bits)
    assert mags.numel() == mb and signs.numel() * 4 == pb
    assert torch.equal(ops.unpack_levels(mags, signs, n, bits), q)


def test_wire_layout_definition():
    # natural-order magnitudes, ballot-word sign planes: element e = row*128 + 4*lane + j -> word row*4+j, bit lane
    n = 256
    q = torch.zeros(n, dtype=torch.int32)
    q[5] = -3       # row 0, lane 1, j 1
    q[128 + 7] = 2  # row 1, lane 1, j 3
    mags, signs = ops.pack_levels(q, 4)
    assert int(mags[2]) == 3 << 4 and int(mags[64 + 3]) == 2 << 4
    assert int(signs[1]) == 1 << 1 and int(signs.abs().sum()) == 2
    bits = torch.zeros(n, dtype=torch.uint8)
    bits[5] = 1
    assert torch.equal(ops.plane_unpack(ops.plane_pack(bits), n), bits)


def test_qsgd_pack_equals_quantize_then_pack():
    x = torch.randn(3000) * 1e-3
    norm = ops.absmax(x)
    mags, signs = ops.qsgd_pack(x, norm, 4, 1, 2, 3)
    q = ops.quantize_levels(x, norm, 15, 1, 2, 3)
    m2, s2 = ops.pack_levels(q, 4)
    assert torch.equal(mags, m2) and torch.equal(signs, s2)
    y = ops.qsgd_unpack_dequant(mags, signs, 3000, norm, 4, world=2)
    assert torch.equal(y, ops.dequantize_levels(q, norm, 15, 2))


# ---------------------------------------------------------------- reference extension layouts
def _ref_varpack(vals):
    """Independent restatement of the greedy packer's layout (word = mode<<30 | payload)."""
    out, i, n = [], 0, len(vals)
    table = [(15, 2, 28), (7, 4, 26), (4, 7, 23), (3, 8, 22)]
    while i < n:
        for mode, (cnt, bits, top) in enumerate(table):
            if all(v < (1 << bits) for v in vals[i:i + cnt]):
                word = mode << 30
                for j, v in enumerate(vals[i:i + cnt]):
                    word |= v << (top - j * bits)
                out.append(word)
                i += cnt
                break
    return out


def test_varpack_layout_and_roundtrip():
    g = torch.Generator().manual_seed(0)
    for scale in (1, 5, 40, 255):
        src = torch.randint(0, scale + 1, (1003,), generator=g, dtype=torch.int32)
        words = packing.varpack(src)
        assert [w & 0xFFFFFFFF for w in words.tolist()] == _ref_varpack(src.tolist())
        assert torch.equal(packing.varunpack(words, src.numel()), src)
    assert [w & 0xFFFFFFFF for w in packing.varpack(torch.tensor([1, 2, 3])).tolist()] == [(1 << 28) | (2 << 26) | (3 << 24)]
    with pytest.raises(ValueError):
        packing.varpack(torch.tensor([256]))   # the reference loops forever here


def test_bytepack_layout_and_roundtrip():
    src = torch.tensor([1, 2, 3, 4, 5, 6, 7, 8, 9], dtype=torch.int32)
    words = packing.bytepack(src)
    assert words.tolist() == [0x0102030405060708, 0x09 << 56]
    signed = torch.tensor([-1, 127, -128, 0, 5], dtype=torch.int32)
    assert torch.equal(packing.byteunpack(packing.bytepack(signed), 5), signed)


def test_elias_roundtrip():
    q = torch.randint(-300, 301, (999,), dtype=torch.int32)
    norm, back = packing.elias_decode(packing.elias_encode(q, 0.375))
    assert norm == 0.375 and torch.equal(back, q)


def test_randk_permutation_properties():
    for n in (1, 7, 1000, 12345):
        idx = ops.randk_indices(42, n, 0, n)
        assert torch.equal(idx.sort()[0], torch.arange(n))
    a = ops.randk_indices(42, 10 ** 6, 5000, 100)
    assert torch.equal(a, ops.randk_indices(42, 10 ** 6, 5000, 100))
    assert not torch.equal(a, ops.randk_indices(43, 10 ** 6, 5000, 100))
    assert not torch.equal(a, ops.randk_indices(42, 10 ** 6, 5000, 100, npass=1))


def test_gram_schmidt_and_topk_and_sgd():
    p = torch.randn(50, 3)
    ref = p.clone()
    for i in range(3):   # column-by-column restatement
        ref[:, i] /= ref[:, i].norm() + 1e-8
        for j in range(i + 1, 3):
            ref[:, j] -= (ref[:, i] * ref[:, j]).sum() * ref[:, i]
    ops.gram_schmidt_(p)
    assert torch.allclose(p, ref, atol=1e-5)
    assert torch.allclose(p.t() @ p, torch.eye(3), atol=1e-4)
    x = torch.randn(1000)
    idx = ops.topk_abs_indices(x, 25)
    assert set(idx.tolist()) == set(torch.topk(x.abs(), 25)[1].tolist())
    prm, g, m = torch.randn(1001), torch.randn(1001), torch.zeros(1001)
    tp = torch.nn.Parameter(prm.clone())
    opt = torch.optim.SGD([tp], lr=0.1, momentum=0.9, weight_decay=5e-4, nesterov=True)
    for _ in range(3):
        tp.grad = g.clone()
        opt.step()
        ops.sgd_step(prm, g, m, lr=0.1, momentum=0.9, weight_decay=5e-4, nesterov=True)
    assert torch.allclose(prm, tp.data, atol=1e-6)
