"""Whole training step on the GPU: eager vs CUDA-graph replay, loss goes down on a fixed batch, the fused
reducer draws fresh rounding noise on every replay."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _setup(graph, reducer="QSGDMaxNormReducer", arch="ResNet18"):
    from gradient_compression_b200 import make_reducer
    from gradient_compression_b200.parallel import FlatSGD
    from gradient_compression_b200.parallel.graph import GraphedStep
    from gradient_compression_b200.train import CIFAR

    dev = torch.device("cuda:0")
    task = CIFAR(dev, None, arch, seed=0, data="synthetic", synthetic_train_size=64, synthetic_test_size=32)
    opt = FlatSGD(task.arena, lr=0.02)
    red = make_reducer(reducer, dev, None, {"quantization_level": 8, "seed": 1, "K": 5000, "rank": 2})
    return task, GraphedStep(task, red, opt, enabled=graph, eager_warmup=2)


@pytest.mark.parametrize("reducer", ["QSGDMaxNormReducer", "NoneAllReducer", "GlobalRandKMaxNormReducer", "RankKReducer",
                                     "TopKReducerRatio", "QSGDMaxNormTwoScaleReducer"])
def test_graph_replay_trains(reducer):
    task, step = _setup(True, reducer)
    g = torch.Generator().manual_seed(0)
    x = torch.randn(64, 3, 32, 32, generator=g).cuda().contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 10, (64,), generator=g).cuda()
    losses = [float(step((x, y))) for _ in range(12)]
    assert step.graphed, getattr(step, "capture_error", "graph capture did not happen")
    assert step.kernels_per_step >= 2
    # finite, and the fixed batch gets fitted at some point (sparsifying / low-rank reducers with error feedback
    # are noisy over a dozen steps, so the last step alone is not the criterion)
    assert all(l == l and l < 1e4 for l in losses) and min(losses[1:]) < losses[0]


def test_graph_and_eager_agree_at_first_steps():
    """Same seeds: the eager warm-up steps of the graphed runner are the eager runner's steps."""
    task_a, eager = _setup(False)
    task_b, graphed = _setup(True)
    g = torch.Generator().manual_seed(1)
    x = torch.randn(32, 3, 32, 32, generator=g).cuda().contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 10, (32,), generator=g).cuda()
    la = [float(eager((x, y))) for _ in range(2)]
    lb = [float(graphed((x, y))) for _ in range(2)]
    assert la[0] == pytest.approx(lb[0], rel=1e-4) and la[1] == pytest.approx(lb[1], rel=5e-2)


def test_replays_draw_fresh_rounding_noise():
    """With the learning rate at zero the gradient is the same every step; the quantised result must still
    differ from replay to replay (the Philox step comes from a device-side launch counter)."""
    from gradient_compression_b200.ops import gemm

    # contractions split three or more ways add up in no fixed order; at batch 32 that noise flips a couple of ReLU masks per
    # step, which moves single gradient elements by several quantisation levels: keep them unsplit for this comparison
    gemm.configure_split(1)
    try:
        _fresh_noise()
    finally:
        gemm.configure_split(0)


def _fresh_noise():
    task, step = _setup(True)
    step.opt.set_lr(0.0)
    step.opt.hyper[1] = 0.0
    step.opt.hyper[2] = 0.0
    g = torch.Generator().manual_seed(2)
    x = torch.randn(32, 3, 32, 32, generator=g).cuda().contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 10, (32,), generator=g).cuda()
    outs = []
    for _ in range(6):
        step((x, y))
        outs.append(task.arena.flat_grads.clone())
    assert step.graphed
    assert not torch.equal(outs[-1], outs[-2])
    assert (outs[-1] - outs[-2]).abs().max() <= outs[-1].abs().max() / 255 * 2.01


def _bucketed_setup(graph, reducer="NoneAllReducer", bucket_mb=4.0, arch="ResNet18"):
    from gradient_compression_b200.parallel import FlatSGD
    from gradient_compression_b200.parallel.bucketed import BucketedReducer
    from gradient_compression_b200.parallel.graph import GraphedStep
    from gradient_compression_b200.train import CIFAR

    dev = torch.device("cuda:0")
    task = CIFAR(dev, None, arch, seed=0, data="synthetic", synthetic_train_size=64, synthetic_test_size=32)
    opt = FlatSGD(task.arena, lr=0.02)
    red = BucketedReducer(task.parameters, reducer, dev, None, {"quantization_level": 8, "seed": 1}, bucket_mb=bucket_mb)
    return task, GraphedStep(task, red, opt, enabled=graph, eager_warmup=2)


def _batch(seed, n=32):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, 3, 32, 32, generator=g).cuda().contiguous(memory_format=torch.channels_last)
    return x, torch.randint(0, 10, (n,), generator=g).cuda()


def test_bucketed_overlapped_step_equals_plain_step_for_an_exact_reducer():
    """Buckets reduced on a side stream while backward runs, captured in the step graph: with an exact reducer (mean over
    one worker) and the parameters held still (learning rate 0) the reduced gradient of every replay must be the plain
    eager step's, up to the rounding of the split-K weight gradients (their partial tiles add up in no fixed order).  The
    forward and input-gradient contractions run unsplit here: split three or more ways they too would add up in no fixed
    order, and ReLU masks that flip on that noise would drown the comparison."""
    from gradient_compression_b200.ops import gemm

    gemm.configure_split(1)
    try:
        _overlapped_equals_plain()
    finally:
        gemm.configure_split(0)


def _overlapped_equals_plain():
    task_a, plain = _setup(False, "NoneAllReducer")
    task_b, bucketed = _bucketed_setup(True, "NoneAllReducer")
    assert len(bucketed.reducer.buckets) > 3
    for st in (plain, bucketed):
        st.opt.set_lr(0.0)
        st.opt.hyper[1] = 0.0
        st.opt.hyper[2] = 0.0
    batch = _batch(5)
    for i in range(6):
        la, lb = plain(batch), bucketed(batch)
        torch.cuda.synchronize()
        ga, gb = task_a.arena.flat_grads, task_b.arena.flat_grads
        assert float(la) == pytest.approx(float(lb), rel=1e-5)
        assert float((ga - gb).norm() / ga.norm()) < 1e-4, i
    assert bucketed.graphed, bucketed.capture_error
    bucketed.check()


def test_bucketed_overlapped_qsgd_step_trains_and_reports_metrics():
    task, step = _bucketed_setup(True, "QSGDMaxNormReducer")
    batch = _batch(6, 64)
    losses = [float(step(batch)) for _ in range(12)]
    assert step.graphed, step.capture_error
    assert all(l == l and l < 1e4 for l in losses) and min(losses[1:]) < losses[0]
    m = {k: float(v) for k, v in step.metrics.items()}
    assert set(m) == {"cross_entropy_loss", "top1_accuracy", "top5_accuracy"}
    assert m["cross_entropy_loss"] == pytest.approx(losses[-1]) and 0.0 <= m["top1_accuracy"] <= m["top5_accuracy"] <= 1.0
    assert [float(v) for v in step.metrics_vec] == pytest.approx([m["cross_entropy_loss"], m["top1_accuracy"], m["top5_accuracy"]])
    n_buckets = len(step.reducer.buckets)
    assert step.bits_per_step == sum(32 + 32 * sum(task.parameters[i].numel() for i in b) for b in step.reducer.buckets)
    assert n_buckets > 1
    step.check()


def test_randk_window_advances_under_graph_replay():
    """The Rand-K index window lives on the device: replays must walk through the permutation (a window start frozen into
    the graph would train the same K coordinates forever)."""
    task, step = _setup(True, "GlobalRandKMaxNormReducer")
    batch = _batch(7)
    starts = []
    for _ in range(8):
        step(batch)
        torch.cuda.synchronize()
        starts.append(int(step.reducer._window.item()))
    assert step.graphed
    assert all(b - a == 5000 for a, b in zip(starts, starts[1:])), starts
    sd = step.reducer.state_dict()
    assert sd["queue"]["position"] == starts[-1]


def test_powersgd_query_changes_under_graph_replay():
    task, step = _setup(True, "RankKReducer")
    batch = _batch(8)
    qs = []
    for _ in range(7):
        step(batch)
        torch.cuda.synchronize()
        qs.append(int(step.reducer._step_dev.item()))
    assert step.graphed and qs == list(range(qs[0], qs[0] + 7))


def test_device_timeout_surfaces_within_two_steps_and_falls_back():
    """A reduce whose peer never launches (rank 0 of an emulated two-rank group runs alone, 200 ms wait limit): the
    kernel gives up and returns, the step's status mirror raises CollectiveTimeout at one of the next two calls, and with
    ``fallback="dist"`` the step continues on the reducer's torch.distributed backend instead."""
    from gradient_compression_b200.parallel import comm
    from gradient_compression_b200.parallel.engine import FusedEngine, FusedOps

    for fallback in (None, "dist"):
        task, step = _setup(False)
        step.fallback = fallback
        red = step.reducer
        n = task.arena.total
        grp = comm.LocalGroup(2, comm.required_bytes(n))
        try:
            lonely = comm._ArenaBase()
            lonely.ctxs, lonely.device, lonely.bytes = (grp.ctxs[0],), grp.device, grp.bytes
            eng = FusedEngine(red)
            eng._ensure = lambda n_, oneshot_region_bytes=None: eng._ops.setdefault("twoshot", FusedOps(lonely, timeout_ms=200))
            eng._ops["twoshot"] = FusedOps(lonely, timeout_ms=200)
            eng.ops = eng._ops["twoshot"]
            red._fused = eng
            batch = _batch(9)
            step(batch)                          # the reduce of this step times out on the device
            if fallback is None:
                with pytest.raises(comm.CollectiveTimeout):
                    for _ in range(2):
                        torch.cuda.synchronize()
                        step(batch)
            else:
                for _ in range(3):
                    torch.cuda.synchronize()
                    loss = step(batch)
                torch.cuda.synchronize()
                assert len(step.fallback_events) == 1 and "timed out" in step.fallback_events[0]
                assert red.backend == "dist" and float(loss) == float(loss)
        finally:
            torch.cuda.synchronize()
            grp.close()


ZOO = ["LeNet", "ResNet18", "ResNet50", "PreActResNet18", "densenet_cifar", "MobileNet", "MobileNetV2", "SENet18", "PNASNetB",
       "EfficientNetB0", "RegNetX_200MF", "ShuffleNetG2", "ShuffleNetV2_x0_5", "ResNeXt29_32x4d", "GoogLeNet", "DPN26", "VGG11",
       "VGG16"]


@pytest.mark.parametrize("name", ZOO)
def test_zoo_model_gradients_on_the_kernels_match_the_torch_path(name):
    """One forward + backward of a zoo model on the GPU with this library's convolution / BN / pooling kernels wherever a layer
    qualifies, against the same model and weights on cuDNN + torch ops in fp32.  Deep batch-norm networks at random
    initialisation amplify TF32 rounding a lot (cuDNN's own TF32 gradients of ResNet-50 differ from its fp32 ones by half their
    norm), so the yardstick is torch's TF32 run: this library's distance to the fp32 gradients must be of the same size.
    Catches a layer shape that a kernel accepts but mishandles."""
    from gradient_compression_b200 import models
    from gradient_compression_b200.ops import conv as convmod
    from gradient_compression_b200.ops import gemm

    torch.manual_seed(3)
    net = getattr(models, name)().cuda().to(memory_format=torch.channels_last)
    x = torch.randn(16, 3, 32, 32, device="cuda").contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 10, (16,), device="cuda")
    state = {k: v.clone() for k, v in net.state_dict().items()}

    def run(kernels, tf32):
        net.load_state_dict(state)
        net.zero_grad(set_to_none=True)
        old = (convmod.ENABLED, torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32)
        convmod.ENABLED, torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = kernels, tf32, tf32
        try:
            loss = torch.nn.functional.cross_entropy(net(x), y)
            loss.backward()
        finally:
            convmod.ENABLED, torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = old
        return float(loss.detach()), torch.cat([p.grad.reshape(-1) for p in net.parameters() if p.grad is not None])

    (la, ga), (lb, gb), (lc, gc) = run(True, True), run(False, True), run(False, False)
    gemm.check()
    assert ga.shape == gc.shape and torch.isfinite(ga).all() and la == la
    ours = float((ga - gc).norm() / gc.norm())
    torch_tf32 = float((gb - gc).norm() / gc.norm())
    assert ours <= 1.3 * torch_tf32 + 0.05, (ours, torch_tf32)
    assert abs(la - lc) <= 3.0 * abs(lb - lc) + 2e-2 * max(1.0, abs(lc)), (la, lb, lc)
