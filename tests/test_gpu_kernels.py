"""T3: every single-GPU sm_100a kernel against its C++ oracle, bit for bit (same Philox counters),
on small and odd sizes."""
import pytest
import torch

from gradient_compression_b200 import ops
from gradient_compression_b200.ops import philox

pytestmark = pytest.mark.gpu
SIZES = [1, 31, 1024, 4099, (1 << 20) + 3]


def _x(n, seed=0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(n, generator=g) * 1e-3


@pytest.mark.parametrize("n", SIZES)
def test_philox_fills(n):
    for kind in (philox.uniform, philox.u32):
        assert torch.equal(kind(n, 42, 77, 3, device="cuda").cpu(), kind(n, 42, 77, 3))
    assert torch.allclose(philox.normal(n, 42, 77, 3, device="cuda").cpu(), philox.normal(n, 42, 77, 3), atol=2e-5)


@pytest.mark.parametrize("n", SIZES)
def test_absmax(n):
    x = _x(n)
    assert float(ops.absmax(x.cuda())) == float(x.abs().max())
    # unaligned base pointer and repeated calls (the ticket counter re-arms itself)
    y = _x(n + 1).cuda()[1:]
    for _ in range(3):
        assert float(ops.absmax(y)) == float(y.cpu().abs().max())


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("mode,s", [(ops.MODE_STOCHASTIC, 15), (ops.MODE_STOCHASTIC, 255), (ops.MODE_BIASED, 63),
                                    (ops.MODE_NU, 64), (ops.MODE_NU_BIASED, 64)])
def test_quantize_dequantize(n, mode, s):
    x = _x(n, 1)
    norm = ops.absmax(x)
    for dtype in (torch.int8 if s < 128 else torch.int32, torch.int32):
        q = ops.quantize_levels(x.cuda(), norm.cuda(), s, 42, 257, 9, mode=mode, dtype=dtype)
        qc = ops.quantize_levels(x, norm, s, 42, 257, 9, mode=mode, dtype=dtype)
        assert torch.equal(q.cpu(), qc)
        assert torch.equal(ops.dequantize_levels(q, norm.cuda(), s, 4).cpu(), ops.dequantize_levels(qc, norm, s, 4))


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("bits", [1, 2, 4, 6, 8, 12])
def test_qsgd_pack_unpack(n, bits):
    x = _x(n, 2)
    norm = ops.absmax(x)
    mags, signs = ops.qsgd_pack(x.cuda(), norm.cuda(), bits, 5, 513, 2)
    mc, sc = ops.qsgd_pack(x, norm, bits, 5, 513, 2)
    nb = ops.packed_sizes(n, bits)
    assert torch.equal(mags.cpu()[: nb[0]], mc) and torch.equal(signs.cpu(), sc)
    y = ops.qsgd_unpack_dequant(mags, signs, n, norm.cuda(), bits, 2)
    assert torch.equal(y.cpu(), ops.qsgd_unpack_dequant(mc, sc, n, norm, bits, 2))
    s = (1 << bits) - 1
    q = torch.randint(-s, s + 1, (n,), dtype=torch.int32)
    m2, s2 = ops.pack_levels(q.cuda(), bits)
    assert torch.equal(ops.unpack_levels(m2, s2, n, bits).cpu(), q)
    m3, s3 = ops.pack_levels(q, bits)
    assert torch.equal(m2.cpu(), m3) and torch.equal(s2.cpu(), s3)


def test_randk_gather_scatter():
    n, k = 100003, 1000
    x = _x(n, 3)
    vals, idx = ops.randk_gather(x.cuda(), 42, 5000, k, want_indices=True)
    ref_idx = ops.randk_indices(42, n, 5000, k)
    assert torch.equal(idx.cpu(), ref_idx) and torch.equal(vals.cpu(), x[ref_idx])
    y = torch.zeros(n, device="cuda")
    ops.randk_scatter(y, vals, 42, 5000, alpha=0.5)
    expect = torch.zeros(n)
    expect[ref_idx] = x[ref_idx] * 0.5
    assert torch.equal(y.cpu(), expect)


@pytest.mark.parametrize("n", SIZES)
def test_sgd_step(n):
    p, g, m = _x(n, 4), _x(n, 5), _x(n, 6)
    pc, mc = p.clone(), m.clone()
    pd, md = p.cuda(), m.cuda()
    for _ in range(2):
        ops.sgd_step(pc, g, mc, lr=0.1, momentum=0.9, weight_decay=5e-4, nesterov=True)
        ops.sgd_step(pd, g.cuda(), md, lr=0.1, momentum=0.9, weight_decay=5e-4, nesterov=True)
    assert torch.equal(pd.cpu(), pc) and torch.equal(md.cpu(), mc)


def test_reducers_on_gpu_match_cpu_single_worker():
    from gradient_compression_b200 import reducers as R

    shapes = [(16, 3, 3, 3), (16,), (32, 16, 3, 3), (32,), (10, 32), (10,)]
    cfg = dict(seed=42, K=50, quantization_level=4, higher_quantization_level=8, quantization_levels=[2, 6, 10],
               compression=0.1, rank=2)
    g = torch.Generator().manual_seed(0)
    grads = [torch.randn(s, generator=g) * 1e-2 for s in shapes]
    for name in ["QSGDMaxNormReducer", "QSGDMaxNormTwoScaleReducer", "GlobalRandKMaxNormReducer",
                 "GlobalRandKMaxNormTwoScaleReducer", "QSGDMaxNormMultiScaleReducer", "NoneAllReducer",
                 "QSGDMaxNormBiasedReducer", "TernGradModReducer"]:
        outs = {}
        for dev, backend in (("cpu", "dist"), ("cuda", "dist"), ("cuda", "fused")):
            red = R.make_reducer(name, dev, None, dict(cfg, backend=backend))
            out = [torch.empty_like(t, device=dev) for t in grads]
            for _ in range(2):
                red.reduce([t.clone().to(dev) for t in grads], out)
            outs[(dev, backend)] = torch.cat([o.reshape(-1).cpu() for o in out])
        assert torch.equal(outs[("cpu", "dist")], outs[("cuda", "dist")]), name
        assert torch.equal(outs[("cpu", "dist")], outs[("cuda", "fused")]), name


@pytest.mark.parametrize("rank", [1, 2, 4])
def test_powersgd_fused_matches_cpu_reference_path(rank):
    from gradient_compression_b200 import reducers as R

    shapes = [(64, 3, 3, 3), (64,), (64,), (128, 64, 3, 3), (128,), (256, 128, 1, 1), (10, 256), (10,), (7, 5, 3, 3)]
    outs, mems = {}, {}
    for dev, backend in (("cpu", "dist"), ("cuda", "fused")):
        red = R.RankKReducer(dev, rank=rank, seed=3, backend=backend)
        for step in range(3):           # error feedback carries over between steps
            g = torch.Generator().manual_seed(step)
            grads = [(torch.randn(s, generator=g) * 1e-2).to(dev) for s in shapes]
            out = [torch.empty_like(t) for t in grads]
            bits = red.reduce([t.clone() for t in grads], out)
        outs[dev] = torch.cat([o.reshape(-1).cpu() for o in out])
        mems[dev] = red._memory.cpu()
        assert bits == 32 * (red._layout["p_elems"] + red._layout["q_elems"] + 64 + 64 + 128 + 10)
    assert torch.allclose(outs["cpu"], outs["cuda"], rtol=1e-3, atol=1e-6)
    assert torch.allclose(mems["cpu"], mems["cuda"], rtol=1e-3, atol=1e-6)


def test_topk_select_many_segments():
    from gradient_compression_b200.ops.topk import TopKSelector

    g_ = torch.Generator().manual_seed(5)
    lens = [10, 4096, 4097, 100000, 7, 1 << 20]
    ks = [100, 1, 41, 1000, 7, 10485]
    segs, off = [], 0
    for l, k in zip(lens, ks):
        segs.append((off, l, k))
        off += l
    g = torch.randn(off, generator=g_)
    e = torch.randn(off, generator=g_) * 0.1
    sel = TopKSelector(segs, "cuda")
    for _ in range(2):                       # state and histograms re-arm themselves
        ed = e.clone().cuda()
        idx, val = sel.select(g.cuda(), ed)
        a = g + e
        idx, val, ed = idx.cpu().long(), val.cpu(), ed.cpu()
        o = 0
        for s, l, k in segs:
            k = min(k, l)
            mine = set(idx[o:o + k].tolist())
            ref = set((torch.topk(a[s:s + l].abs(), k)[1] + s).tolist())
            assert mine == ref, (s, l, k)
            o += k
        assert torch.equal(val, a[idx])
        expect = a.clone()
        expect[idx] = 0
        assert torch.equal(ed, expect)
    idx2, val2 = sel.select(g.cuda(), None)   # no error feedback: selection on g itself
    assert torch.equal(val2.cpu(), g[idx2.cpu().long()])


def test_topk_reducers_fused_match_cpu():
    from gradient_compression_b200 import reducers as R

    shapes = [(64, 3, 3, 3), (64,), (128, 64, 3, 3), (128,), (10, 128), (10,)]
    for name, kw in [("TopKReducer", {"K": 50}), ("TopKReducerRatio", {"compression": 0.01}), ("GlobalTopKReducer", {"K": 500})]:
        res = {}
        for dev, backend in (("cpu", "dist"), ("cuda", "dist"), ("cuda", "fused")):
            red = getattr(R, name)(dev, backend=backend, **kw)
            for step in range(3):
                g = torch.Generator().manual_seed(step)
                grads = [torch.randn(s, generator=g).to(dev) for s in shapes]
                out = [torch.empty_like(t) for t in grads]
                red.reduce([t.clone() for t in grads], out)
            res[(dev, backend)] = (torch.cat([o.reshape(-1).cpu() for o in out]), red._memory.cpu())
        for key in (("cuda", "dist"), ("cuda", "fused")):
            assert torch.equal(res[key][0], res[("cpu", "dist")][0]), (name, key)
            assert torch.equal(res[key][1], res[("cpu", "dist")][1]), (name, key)


@pytest.mark.parametrize("n", [1, 14, 15, 16, 255, 256, 257, 4099, (1 << 20) + 5])
@pytest.mark.parametrize("scale", [1, 3, 15, 100, 255])
def test_varpack_gpu_matches_host_packer(n, scale):
    from gradient_compression_b200.ops import packing

    g = torch.Generator().manual_seed(n * 7 + scale)
    src = torch.randint(0, scale + 1, (n,), generator=g, dtype=torch.int32)
    if n > 300:
        src[100:140] = 0            # long runs of small values next to large ones: every mode shows up
        src[200] = 255
    host_words = packing.varpack(src)
    dev_words = packing.varpack(src.cuda())
    assert torch.equal(dev_words.cpu(), host_words)
    assert torch.equal(packing.varunpack(dev_words, n).cpu(), src)
    assert torch.equal(packing.varunpack(dev_words).cpu(), packing.varunpack(host_words))


def test_varpack_gpu_rejects_out_of_range():
    from gradient_compression_b200.ops import packing

    with pytest.raises(ValueError):
        packing.varpack(torch.tensor([1, 2, 300], dtype=torch.int32, device="cuda"))


def test_bytepack_gpu_matches_host():
    from gradient_compression_b200.ops import packing

    src = torch.randint(-128, 128, (100003,), dtype=torch.int32)
    w_host, w_dev = packing.bytepack(src), packing.bytepack(src.cuda())
    assert torch.equal(w_dev.cpu(), w_host)
    assert torch.equal(packing.byteunpack(w_dev, src.numel()).cpu(), src)


@pytest.mark.parametrize("n,c,hw,k,bias", [(128, 2048, 4, 10, True), (128, 512, 1, 10, True), (7, 64, 3, 32, False), (33, 1024, 2, 10, True)])
def test_head_kernels_match_torch(n, c, hw, k, bias):
    """Average pool + linear + cross-entropy + top-1 / top-5 in one kernel, and its backward, against torch ops in fp32."""
    import torch.nn.functional as F

    from gradient_compression_b200.ops import head

    g = torch.Generator().manual_seed(n + c + k)
    feat = torch.randn(n, c, hw, hw, generator=g).cuda().contiguous(memory_format=torch.channels_last).requires_grad_(True)
    ref_feat = feat.detach().clone(memory_format=torch.preserve_format).requires_grad_(True)
    lin = torch.nn.Linear(c, k, bias=bias).cuda()
    ref_lin = torch.nn.Linear(c, k, bias=bias).cuda()
    ref_lin.load_state_dict(lin.state_dict())
    labels = torch.randint(0, k, (n,), generator=g).cuda()
    assert head.supported(feat, lin.weight, labels)
    loss, logits, met = head.head_loss(feat, lin, labels)
    (loss * 1.5).backward()
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        rl = ref_lin(ref_feat.mean((2, 3)))
        rloss = F.cross_entropy(rl, labels)
        (rloss * 1.5).backward()
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    assert torch.allclose(logits, rl, rtol=1e-4, atol=1e-4)
    assert float(loss) == pytest.approx(float(rloss), rel=1e-5)
    top = rl.topk(min(5, k), 1)[1].eq(labels.view(-1, 1))
    assert float(met[0]) == pytest.approx(float(rloss), rel=1e-5)
    assert float(met[1]) == pytest.approx(float(top[:, 0].float().mean()), abs=1e-6)
    assert float(met[2]) == pytest.approx(float(top.any(1).float().mean()), abs=1e-6)
    assert torch.allclose(feat.grad, ref_feat.grad, rtol=1e-4, atol=1e-7)
    assert torch.allclose(lin.weight.grad, ref_lin.weight.grad, rtol=1e-4, atol=1e-6)
    if bias:
        assert torch.allclose(lin.bias.grad, ref_lin.bias.grad, rtol=1e-4, atol=1e-6)
    loss2, _, met2 = head.head_loss(feat.detach(), lin, labels)        # the ticket was reset: a second call gives the same
    assert float(loss2) == float(loss) and torch.equal(met2, met)
