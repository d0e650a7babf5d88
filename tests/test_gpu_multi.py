"""T4 on real GPUs: one process per GPU, arenas mapped into each other with CUDA IPC, the fused
kernels of every rank running concurrently on different devices.  Results are compared bit for bit with
the CPU oracle evaluated for every rank's input and random stream."""
import os

import pytest
import torch

pytestmark = [pytest.mark.gpu, pytest.mark.multigpu]

N = 300007


def _inputs(world, n):
    return [torch.randn(n, generator=torch.Generator().manual_seed(1000 + r)) * (1e-3 * (r + 1)) for r in range(world)]


def _body(rank, world):
    import torch.distributed as dist

    from gradient_compression_b200 import ops, reducers as R
    from gradient_compression_b200.ops import philox
    from tests.test_gpu_fused import _oracle_qsgd, _oracle_twoscale

    dev = torch.device("cuda", rank)
    xs = _inputs(world, N)
    mine = xs[rank].to(dev)

    red = R.QSGDMaxNormReducer(dev, quantization_level=4, seed=42, backend="fused")
    for step in range(3):
        out = [torch.empty(N, device=dev)]
        red.reduce([mine.clone()], out)
        red._fused.ops.check()
        assert torch.equal(out[0].cpu(), _oracle_qsgd(xs, 4, 42, step)), f"qsgd step {step}"

    # same numbers through the collective backend (our kernels + NCCL)
    ref = R.QSGDMaxNormReducer(dev, quantization_level=4, seed=42, backend="dist")
    out2 = [torch.empty(N, device=dev)]
    ref.reduce([mine.clone()], out2)
    assert torch.equal(out2[0].cpu(), _oracle_qsgd(xs, 4, 42, 0))

    ts = R.QSGDMaxNormTwoScaleReducer(dev, lower_quantization_level=2, higher_quantization_level=6, seed=7, backend="fused")
    out = [torch.empty(N, device=dev)]
    ts.reduce([mine.clone()], out)
    ts._fused.ops.check()
    assert torch.equal(out[0].cpu(), _oracle_twoscale(xs, 2, 6, 7, 0)), "twoscale"

    ar = R.NoneAllReducer(dev, backend="fused")
    out = [torch.empty(N, device=dev)]
    ar.reduce([mine.clone()], out)
    ar._fused.ops.check()
    acc = xs[0].clone()
    for x in xs[1:]:
        acc += x
    assert torch.equal(out[0].cpu(), acc * (1.0 / world)), "allreduce"
    nccl = mine.clone()
    dist.all_reduce(nccl)
    assert torch.allclose(out[0], nccl / world, atol=1e-7)

    rk = R.GlobalRandKMaxNormReducer(dev, seed=5, K=10000, quantization_level=8, backend="fused")
    out = [torch.empty(N, device=dev)]
    rk.reduce([mine.clone()], out)
    rk._fused.ops.check()
    idx = ops.randk_indices(5, N, 0, 10000)
    expect = xs[rank] * (1.0 / world)
    expect[idx] = _oracle_qsgd([x[idx] for x in xs], 8, 5, 0)
    assert torch.equal(out[0].cpu(), expect), "randk"
    tk = {}
    for backend in ("fused", "dist"):
        red_tk = R.TopKReducerRatio(dev, compression=0.01, backend=backend)
        out = [torch.empty(N, device=dev)]
        red_tk.reduce([mine.clone()], out)
        tk[backend] = out[0].clone()
    assert torch.allclose(tk["fused"], tk["dist"], atol=1e-7), "topk"

    # PowerSGD: the fused pipeline against the same reducer on the collective backend (NCCL)
    shapes = [(64, 27), (64,), (128, 576), (128,), (10, 128), (10,)]
    res = {}
    for backend in ("fused", "dist"):
        pr = R.RankKReducer(dev, rank=2, seed=11, backend=backend)
        for step in range(2):
            g = torch.Generator().manual_seed(100 * rank + step)
            grads = [(torch.randn(s, generator=g) * 1e-2).to(dev) for s in shapes]
            out = [torch.empty_like(t) for t in grads]
            pr.reduce([t.clone() for t in grads], out)
        res[backend] = torch.cat([o.reshape(-1) for o in out])
    assert torch.allclose(res["fused"], res["dist"], rtol=1e-3, atol=1e-6), "powersgd"
    torch.cuda.synchronize()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_reducers_across_gpus(dist_runner, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dist_runner(_body, world=world, backend="nccl")


def _bucketed_body(rank, world):
    """Per-bucket fused reduces on a side stream, captured in a CUDA graph and replayed: every bucket of every replay must
    equal the CPU oracle of an independent QSGD instance with that bucket's seed and the Philox step the device derives."""
    from gradient_compression_b200.ops import _native as nat
    from gradient_compression_b200.parallel.bucketed import BucketedReducer
    from tests.test_gpu_fused import _oracle_qsgd

    dev = torch.device("cuda", rank)
    sizes = [70001, 130, 50000, 9000, 64]
    params = [torch.nn.Parameter(torch.zeros(s, device=dev)) for s in sizes]
    for p in params:
        p.grad = torch.zeros_like(p)
    srcs = [[torch.randn(s, generator=torch.Generator().manual_seed(500 + 10 * r + i)) * (1e-3 * (r + 1))
             for i, s in enumerate(sizes)] for r in range(world)]
    mine = [t.to(dev) for t in srcs[rank]]
    br = BucketedReducer(params, "QSGDMaxNormReducer", dev, None, {"quantization_level": 4, "seed": 3, "backend": "fused"},
                         bucket_mb=0.2, max_blocks=8, tail_mb=0)
    assert br.buckets == [[2, 3, 4], [0, 1]]
    nb = len(br.buckets)

    def run_once():
        for p, s in zip(params, mine):
            p.grad.copy_(s)
        br.start_step()
        for b in range(nb):
            br._launch(b)
        br.finish()

    def check(step_of_bucket, what):
        torch.cuda.synchronize()
        for j, idxs in enumerate(br.buckets):
            got = torch.cat([params[i].grad.reshape(-1) for i in idxs]).cpu()
            xs = [torch.cat([srcs[r][i] for i in idxs]) for r in range(world)]
            want = _oracle_qsgd(xs, 4, 3 * 1000003 + j, step_of_bucket(j))
            assert torch.equal(got, want), f"{what}, bucket {j}"

    run_once()                                   # eager: maps the arenas; every bucket's host-side step is 0
    check(lambda j: 0, "eager")
    arenas = []
    for r in br.reducers:
        arenas += [a for a in r._fused.arenas() if a not in arenas]
    for a in arenas:
        for c in a.ctxs:
            nat.cuda().gc_comm_set_step_from_device(c.handle, 1)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run_once()                               # host-side steps (now 1) are frozen into the graph; the device adds its launch count
    for replay in range(3):
        graph.replay()
        check(lambda j: 1 + nb + replay * nb + j, f"replay {replay}")
    for r in br.reducers:
        r._fused.ops.check()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_bucketed_graphed_reduce_across_gpus(dist_runner, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    dist_runner(_bucketed_body, world=world, backend="nccl")
