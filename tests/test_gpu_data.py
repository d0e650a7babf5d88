"""Device-resident CIFAR pipeline: oracle semantics on CPU, bit-identical batches on the GPU."""
import pytest
import torch

from gradient_compression_b200.train.data import MEAN, STD
from gradient_compression_b200.train.gpu_data import DeviceCIFAR


def test_eval_batches_are_plain_normalisation_and_cover_the_set():
    ds = DeviceCIFAR.synthetic(64, "cpu", seed=3, train=False)
    seen = []
    for i in range(ds.num_batches(16)):
        x, y = ds.batch(16, 0, i)
        ref = ds.images[i * 16:(i + 1) * 16].float().div(255).permute(0, 3, 1, 2)
        ref = (ref - torch.tensor(MEAN).view(1, 3, 1, 1)) / torch.tensor(STD).view(1, 3, 1, 1)
        assert torch.allclose(x, ref, atol=1e-6) and torch.equal(y, ds.labels[i * 16:(i + 1) * 16])
        assert x.is_contiguous(memory_format=torch.channels_last)
        seen += y.tolist()
    assert len(seen) == 64


def test_train_epoch_is_a_permutation_with_crop_and_flip():
    n = 200
    imgs = torch.zeros(n, 32, 32, 3, dtype=torch.uint8)
    imgs[:, :, :, 0] = (torch.arange(n) + 1).to(torch.uint8).view(n, 1, 1)   # red channel = image id + 1
    imgs[:, :, 0:16, 1] = 255                                                   # green: left half bright
    ds = DeviceCIFAR(imgs, torch.arange(n), "cpu", seed=1, train=True)
    ids, flips, shifts = [], 0, set()
    for i in range(ds.num_batches(20)):
        x, y = ds.batch(20, epoch=2, index=i)
        raw = x * torch.tensor(STD).view(1, 3, 1, 1) + torch.tensor(MEAN).view(1, 3, 1, 1)
        for b in range(20):
            ids.append(int(y[b]))
            inner = raw[b, 0][raw[b, 0] > 1e-6]                   # unpadded part carries the id
            assert inner.numel() > 0 and torch.allclose(inner * 255, torch.full_like(inner, float(y[b]) + 1), atol=1e-3)
            green = raw[b, 1]
            flips += int(green[16, 24] > 0.5 and green[16, 8] < 0.5)
            shifts.add(int((raw[b, 0] > 1e-6).any(0).float().argmax()))        # first non-padded column
    assert sorted(ids) == list(range(n))                          # every image exactly once per epoch
    assert 0.25 * n < flips < 0.75 * n and len(shifts) >= 4
    x2, y2 = ds.batch(20, epoch=3, index=0)
    assert not torch.equal(y2, ds.batch(20, epoch=2, index=0)[1])   # a new epoch reshuffles


@pytest.mark.gpu
def test_gpu_batches_match_cpu_oracle_bit_for_bit():
    cpu = DeviceCIFAR.synthetic(512, "cpu", seed=9, train=True)
    gpu = DeviceCIFAR(cpu.images, cpu.labels, "cuda", seed=9, train=True)
    for epoch, index in [(0, 0), (1, 3), (7, 1)]:
        xc, yc = cpu.batch(128, epoch, index)
        xg, yg = gpu.batch(128, epoch, index)
        assert torch.equal(xg.cpu(), xc) and torch.equal(yg.cpu(), yc)


def _host_batches(n=5):
    g = torch.Generator().manual_seed(9)
    return [(torch.randn(4, 3, 8, 8, generator=g), torch.randint(0, 10, (4,), generator=g)) for _ in range(n)]


def test_prefetcher_and_lagged_readback_on_cpu():
    from gradient_compression_b200.train.data import DevicePrefetcher, LaggedReadback

    batches = _host_batches()
    got = list(DevicePrefetcher(batches, "cpu", depth=2))
    assert len(got) == len(batches) and all(torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) for a, b in zip(got, batches))
    r = LaggedReadback("cpu", lag=1)
    seen = [r.push(torch.tensor(float(i))) for i in range(4)]
    assert seen == [None, 0.0, 1.0, 2.0] and r.drain() == [3.0]


@pytest.mark.gpu
def test_prefetcher_and_lagged_readback_on_gpu():
    """Batches arrive complete and in order although their copies run ahead on a side stream; scalars read one step
    late are the values of their own step even when the producing tensor is overwritten in place afterwards."""
    from gradient_compression_b200.train.data import DevicePrefetcher, LaggedReadback

    batches = [(x.pin_memory(), y.pin_memory()) for x, y in _host_batches(8)]
    conv = lambda x, y: (x.contiguous(memory_format=torch.channels_last), y)
    got = []
    for x, y in DevicePrefetcher(batches, "cuda", convert=conv, depth=3):
        assert x.is_cuda and x.is_contiguous(memory_format=torch.channels_last)
        got.append((x.sum() * 1.0, y.clone()))              # consume on the current stream
    assert len(got) == 8
    for (s, y), (hx, hy) in zip(got, batches):
        assert abs(float(s) - float(hx.sum())) < 1e-3 and torch.equal(y.cpu(), hy)
    r = LaggedReadback("cuda", lag=1)
    static = torch.zeros((), device="cuda")
    out = []
    for i in range(5):
        static.fill_(float(i))                              # the same tensor every step, as a replayed graph's output
        v = r.push(static)
        if v is not None:
            out.append(v)
    out += r.drain()
    assert out == [0.0, 1.0, 2.0, 3.0, 4.0]
