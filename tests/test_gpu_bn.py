"""Fused BN (+ residual) (+ ReLU) kernels against the plain PyTorch fp32 chain bn -> add -> relu."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _case(n, c, h, w, residual, relu, seed=0):
    from gradient_compression_b200.ops.bn import bn_act, kernel_path_ok

    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(n, c, h, w, generator=g) * 2 + 0.5).cuda().contiguous(memory_format=torch.channels_last)
    r = torch.randn(n, c, h, w, generator=g).cuda().contiguous(memory_format=torch.channels_last) if residual else None
    dy = torch.randn(n, c, h, w, generator=g).cuda().contiguous(memory_format=torch.channels_last)
    assert kernel_path_ok(x)
    bn_a, bn_b = torch.nn.BatchNorm2d(c).cuda(), torch.nn.BatchNorm2d(c).cuda()
    with torch.no_grad():
        bn_a.weight.copy_(torch.rand(c, generator=g) + 0.5)
        bn_a.bias.copy_(torch.randn(c, generator=g) * 0.1)
    bn_b.load_state_dict(bn_a.state_dict())
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    ra = r.clone().requires_grad_(True) if residual else None
    rb = r.clone().requires_grad_(True) if residual else None
    ya = bn_act(bn_a, xa, ra, relu)
    yb = bn_b(xb)
    if residual:
        yb = yb + rb
    if relu:
        yb = F.relu(yb)
    ya.backward(dy)
    yb.backward(dy)
    tol = dict(rtol=1e-4, atol=1e-4)
    assert torch.allclose(ya, yb, **tol)
    assert torch.allclose(xa.grad, xb.grad, **tol)
    assert torch.allclose(bn_a.weight.grad, bn_b.weight.grad, rtol=1e-4, atol=1e-3)
    assert torch.allclose(bn_a.bias.grad, bn_b.bias.grad, rtol=1e-4, atol=1e-3)
    if residual:
        assert torch.allclose(ra.grad, rb.grad, **tol)
    assert torch.allclose(bn_a.running_mean, bn_b.running_mean, atol=1e-5)
    assert torch.allclose(bn_a.running_var, bn_b.running_var, rtol=1e-4, atol=1e-5)
    assert int(bn_a.num_batches_tracked) == int(bn_b.num_batches_tracked) == 1
    # eval mode uses the running statistics
    bn_a.eval(), bn_b.eval()
    with torch.no_grad():
        ea = bn_act(bn_a, x, r, relu)
        eb = bn_b(x)
        eb = eb + r if residual else eb
        eb = F.relu(eb) if relu else eb
    assert torch.allclose(ea, eb, **tol)


@pytest.mark.parametrize("shape", [(128, 64, 32, 32), (16, 256, 8, 8), (4, 2048, 4, 4), (3, 16, 5, 7), (2, 512, 1, 1)])
@pytest.mark.parametrize("residual", [False, True])
@pytest.mark.parametrize("relu", [False, True])
def test_bn_act_matches_torch(shape, residual, relu):
    _case(*shape, residual, relu)


def test_unsupported_channel_counts_fall_back():
    from gradient_compression_b200.ops.bn import bn_act, kernel_path_ok

    x = torch.randn(4, 6, 8, 8, device="cuda")
    assert not kernel_path_ok(x)
    bn = torch.nn.BatchNorm2d(6).cuda()
    assert torch.allclose(bn_act(bn, x), F.relu(torch.nn.BatchNorm2d(6).cuda()(x)), atol=1e-5)


def test_resnet50_step_matches_unfused_model():
    """Whole-model check.  A randomly initialised ResNet-50 at batch 16 is ill-conditioned: a 1e-6 relative
    perturbation of the input already moves its gradients by ~1.5 % with fp32 convolutions.  The fused path
    must stay within that natural sensitivity of the unfused (torch bn / add / relu) model."""
    from gradient_compression_b200 import models
    from gradient_compression_b200.ops import bn as bnmod

    torch.manual_seed(0)
    net = models.ResNet50().cuda().to(memory_format=torch.channels_last)
    x = torch.randn(16, 3, 32, 32, device="cuda").contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 10, (16,), device="cuda")
    state = {k: v.clone() for k, v in net.state_dict().items()}

    def run(fused, xin):
        net.load_state_dict(state)
        net.zero_grad()
        orig = bnmod.kernel_path_ok
        if not fused:
            bnmod.kernel_path_ok = lambda t: False
        try:
            loss = F.cross_entropy(net(xin), y)
            loss.backward()
        finally:
            bnmod.kernel_path_ok = orig
        return float(loss.detach()), [p.grad.clone() for p in net.parameters()]

    def rel(g1, g2):
        num = sum(float(((a - b) ** 2).sum()) for a, b in zip(g1, g2))
        return (num / sum(float((b ** 2).sum()) for b in g2)) ** 0.5

    old = torch.backends.cudnn.allow_tf32
    torch.backends.cudnn.allow_tf32 = False
    try:
        loss_f, g_f = run(True, x)
        loss_u, g_u = run(False, x)
        _, g_p = run(False, x * (1 + 1e-6))
    finally:
        torch.backends.cudnn.allow_tf32 = old
    assert abs(loss_f - loss_u) < 1e-4
    assert rel(g_f, g_u) < 2.0 * rel(g_p, g_u) + 1e-3
    assert float((g_f[-1] - g_u[-1]).norm() / g_u[-1].norm()) < 1e-4      # the head's bias gradient is well conditioned


@pytest.fixture
def tc_conv():
    """Tensor-core 1x1 convolutions on for every size, restored afterwards."""
    from gradient_compression_b200.ops import conv as convmod

    old = (convmod.ENABLED, convmod.MIN_ROWS)
    convmod.ENABLED, convmod.MIN_ROWS = True, 0
    yield convmod
    convmod.ENABLED, convmod.MIN_ROWS = old


@pytest.mark.parametrize("shape", [(128, 64, 32, 32, 256), (16, 256, 8, 8, 64), (8, 512, 4, 4, 2048), (5, 16, 7, 9, 32)])
@pytest.mark.parametrize("residual", [False, True])
@pytest.mark.parametrize("relu", [False, True])
def test_conv1x1_bn_act_matches_torch(tc_conv, shape, residual, relu):
    """1x1 convolution on the tcgen05 GEMM with BN statistics from its epilogue vs cuDNN conv + torch bn."""
    from gradient_compression_b200.ops.conv import _mode, conv_bn_act

    n, cin, h, w, cout = shape
    g = torch.Generator().manual_seed(cin + cout)
    cl = torch.channels_last
    x = torch.randn(n, cin, h, w, generator=g).cuda().contiguous(memory_format=cl)
    r = torch.randn(n, cout, h, w, generator=g).cuda().contiguous(memory_format=cl) if residual else None
    dy = torch.randn(n, cout, h, w, generator=g).cuda().contiguous(memory_format=cl)
    conv_a = torch.nn.Conv2d(cin, cout, 1, bias=False).cuda().to(memory_format=cl)
    conv_b = torch.nn.Conv2d(cin, cout, 1, bias=False).cuda().to(memory_format=cl)
    conv_b.load_state_dict(conv_a.state_dict())
    bn_a, bn_b = torch.nn.BatchNorm2d(cout).cuda(), torch.nn.BatchNorm2d(cout).cuda()
    with torch.no_grad():
        bn_a.weight.copy_(torch.rand(cout, generator=g) + 0.5)
        bn_a.bias.copy_(torch.randn(cout, generator=g) * 0.1)
    bn_b.load_state_dict(bn_a.state_dict())
    assert _mode(conv_a, bn_a, x) == "gemm"
    xa, xb = x.clone().requires_grad_(True), x.clone().requires_grad_(True)
    ra = r.clone().requires_grad_(True) if residual else None
    rb = r.clone().requires_grad_(True) if residual else None
    ya = conv_bn_act(conv_a, bn_a, xa, ra, relu)
    yb = bn_b(conv_b(xb))
    if residual:
        yb = yb + rb
    if relu:
        yb = F.relu(yb)
    ya.backward(dy)
    yb.backward(dy)
    from gradient_compression_b200.ops import gemm
    gemm.check()
    tol = dict(rtol=5e-3, atol=5e-3)       # both sides multiply in TF32; they round differently

    def close(a, b):
        """Agreement at TF32 level in the Frobenius norm.  Both sides round operands to 10 mantissa bits, in
        different summation orders; with ReLU a few pre-activations within rounding distance of zero land on
        different sides, which changes those elements' gradient by O(dy)."""
        a, b = a.detach(), b.detach()
        return float((a - b).norm() / b.norm()) < (6e-2 if relu else 5e-3)

    assert close(ya, yb)
    assert close(xa.grad, xb.grad)
    assert close(conv_a.weight.grad, conv_b.weight.grad)
    assert close(bn_a.weight.grad, bn_b.weight.grad) and close(bn_a.bias.grad, bn_b.bias.grad)
    if residual:
        assert close(ra.grad, rb.grad)
    assert torch.allclose(bn_a.running_mean, bn_b.running_mean, atol=1e-3)
    assert torch.allclose(bn_a.running_var, bn_b.running_var, rtol=5e-3, atol=1e-3)


@pytest.mark.parametrize("in_place", [False, True])
def test_input_gradient_follows_weight_updates(tc_conv, in_place):
    """The input-gradient kernels read the filter where it lies (``in_place``) or, for shapes that path does not cover,
    cached transposed copies.  The copies must follow (a) the fused SGD kernel, which writes parameters through raw pointers
    and re-transposes all of them in one launch, and (b) in-place torch updates, which the version counter reveals."""
    from gradient_compression_b200.ops import conv as convmod
    from gradient_compression_b200.ops.conv import conv_bn_act
    from gradient_compression_b200.parallel.arena import FlatArena, FlatSGD

    old = convmod.DGRAD_IN_PLACE
    convmod.DGRAD_IN_PLACE = in_place
    try:
        _input_gradient_follows(conv_bn_act, FlatArena, FlatSGD, in_place)
    finally:
        convmod.DGRAD_IN_PLACE = old


def _input_gradient_follows(conv_bn_act, FlatArena, FlatSGD, in_place):

    cl = torch.channels_last
    torch.manual_seed(5)
    convs = torch.nn.ModuleList([torch.nn.Conv2d(32, 64, 1, bias=False), torch.nn.Conv2d(64, 32, 1, bias=False)]).cuda().to(memory_format=cl)
    bns = torch.nn.ModuleList([torch.nn.BatchNorm2d(64), torch.nn.BatchNorm2d(32)]).cuda()
    arena = FlatArena(list(convs.parameters()) + list(bns.parameters()))
    opt = FlatSGD(arena, lr=0.5, momentum=0.0, weight_decay=0.0, nesterov=False)
    x = torch.randn(8, 32, 16, 16, device="cuda").contiguous(memory_format=cl)
    dy = torch.randn(8, 32, 16, 16, device="cuda").contiguous(memory_format=cl)

    def input_grads():
        xa = x.clone().requires_grad_(True)
        conv_bn_act(convs[1], bns[1], conv_bn_act(convs[0], bns[0], xa, None, True), None, False).backward(dy)
        xb = x.clone().requires_grad_(True)
        h = F.relu(F.batch_norm(F.conv2d(xb, convs[0].weight), None, None, bns[0].weight, bns[0].bias, True))
        F.batch_norm(F.conv2d(h, convs[1].weight), None, None, bns[1].weight, bns[1].bias, True).backward(dy)
        return xa.grad, xb.grad

    for step in range(4):
        arena.zero_grad()
        ga, gb = input_grads()
        assert float((ga - gb).norm() / gb.norm()) < 6e-2, step
        if step < 2:
            opt.step()                                   # raw-pointer update + batched re-transpose
        else:
            with torch.no_grad():                        # in-place torch update: the version counter moves
                for c in convs:
                    c.weight.add_(torch.randn_like(c.weight) * 0.3)
    if not in_place:
        assert getattr(arena, "_dgrad_weight_table", None) is not None and arena._dgrad_weight_table[1].shape[0] == 2


@pytest.mark.parametrize("owned", [True, False])
def test_identity_block_gradient_link(tc_conv, owned):
    """x feeds conv1 and the skip connection.  With a GradLink the input-gradient GEMM of conv1 accumulates onto the
    skip connection's gradient; the result must equal autograd's own sum.  ``owned=False`` routes the skip through a
    plain torch add, whose gradient tensor is shared with the other branch and must not be written in place."""
    from gradient_compression_b200.ops.conv import GradLink, conv_bn_act

    cl = torch.channels_last
    torch.manual_seed(11)
    conv1, conv3 = torch.nn.Conv2d(64, 32, 1, bias=False).cuda().to(memory_format=cl), torch.nn.Conv2d(32, 64, 1, bias=False).cuda().to(memory_format=cl)
    bn1, bn3 = torch.nn.BatchNorm2d(32).cuda(), torch.nn.BatchNorm2d(64).cuda()
    x0 = torch.randn(16, 64, 16, 16, device="cuda").contiguous(memory_format=cl)
    dy = torch.randn(16, 64, 16, 16, device="cuda").contiguous(memory_format=cl)

    def block(x, use_link):
        link = GradLink() if use_link else None
        y = conv_bn_act(conv1, bn1, x, link=link)
        res = link.residual(x) if use_link else x
        if owned:
            return conv_bn_act(conv3, bn3, y, residual=res)
        return torch.relu(conv_bn_act(conv3, bn3, y, relu=False) + res)

    grads = []
    for use_link in (True, False):
        for p in (conv1.weight, conv3.weight):
            p.grad = None
        x = (x0 * 1.0).requires_grad_(True)           # non-leaf input, as inside a network
        x.retain_grad()
        out = block(x, use_link)
        out.backward(dy)
        grads.append((x.grad.clone(), conv1.weight.grad.clone(), dy.clone()))
    (gx_l, gw_l, dy_l), (gx_p, gw_p, _) = grads
    assert torch.equal(dy_l, dy)                       # the incoming gradient was not written to
    assert float((gx_l - gx_p).norm() / gx_p.norm()) < 1e-6
    assert float((gw_l - gw_p).norm() / gw_p.norm()) < 1e-6


@pytest.mark.parametrize("stride", [1, 2])
def test_projection_block_hands_its_input_gradient_to_the_first_convolution(tc_conv, stride):
    """x feeds conv1 and the projection shortcut.  The shortcut's backward runs first and donates its input gradient to
    conv1's input-gradient kernel, which adds onto it; the result must equal autograd's own sum of the two."""
    from gradient_compression_b200.models.resnet import Bottleneck
    from gradient_compression_b200.ops import conv as convmod

    cl = torch.channels_last
    torch.manual_seed(5 + stride)
    block = Bottleneck(64, 32, stride).cuda().to(memory_format=cl)
    x0 = torch.randn(8, 64, 16, 16, device="cuda").contiguous(memory_format=cl)
    grads = []
    for enabled in (True, False):
        convmod.LINK_ENABLED = enabled
        try:
            block.zero_grad(set_to_none=True)
            x = (x0 * 1.0).requires_grad_(True)
            x.retain_grad()
            out = block(x)
            torch.manual_seed(9)
            out.backward(torch.randn_like(out))
        finally:
            convmod.LINK_ENABLED = True
        grads.append((x.grad.clone(), block.conv1.weight.grad.clone(), block.shortcut[0].weight.grad.clone()))
    for a, b in zip(*grads):
        assert float((a - b).norm() / b.norm()) < 1e-5


@pytest.mark.parametrize("m,c", [(2048, 512), (777, 140), (128, 2048), (32, 64), (1, 8)])
@pytest.mark.parametrize("relu", [False, True])
@pytest.mark.parametrize("residual", [False, True])
@pytest.mark.parametrize("from_partials", [False, True])
def test_small_activation_kernels_match_float64(m, c, relu, residual, from_partials):
    """Statistics + running-statistics update + apply in one launch, and both gradient sums + input gradient (+ residual
    gradient) in one launch, for activations of at most 2048 rows, against torch in float64."""
    from gradient_compression_b200.ops import _native as nat

    lib, st = nat.cuda(), nat.stream_ptr
    assert lib.gc_cuda_bn_small_supported(m, c)
    g = torch.Generator().manual_seed(m + c)
    x = (torch.randn(m, c, generator=g) * 1.7 + 3.0).cuda()
    res = torch.randn(m, c, generator=g).cuda() if residual else None
    gamma, beta = (torch.rand(c, generator=g) + 0.5).cuda(), torch.randn(c, generator=g).cuda()
    rm, rv = torch.zeros(c, device="cuda"), torch.ones(c, device="cuda")
    stats, y = torch.empty(2 * c, device="cuda"), torch.empty(m, c, device="cuda")
    partials = None
    if from_partials:          # what a convolution kernel's epilogue emits: per 128-row tile, column sums and sums of squares
        tiles = (m + 127) // 128
        partials = torch.zeros(tiles, 2, c, device="cuda")
        for t in range(tiles):
            blk = x[t * 128:(t + 1) * 128].double()
            partials[t, 0], partials[t, 1] = blk.sum(0).float(), (blk * blk).sum(0).float()
    nat.check(lib.gc_cuda_bn_small_forward(x.data_ptr(), m, c, nat.ptr(partials), 0 if partials is None else partials.shape[0],
                                           gamma.data_ptr(), beta.data_ptr(), nat.ptr(res), int(relu), rm.data_ptr(), rv.data_ptr(), 0.1,
                                           1e-5, stats.data_ptr(), y.data_ptr(), st()), "small_fwd")
    xd = x.double().requires_grad_(True)
    rd = res.double().requires_grad_(True) if residual else None
    rm_r, rv_r = torch.zeros(c, dtype=torch.float64, device="cuda"), torch.ones(c, dtype=torch.float64, device="cuda")
    gd, bd = gamma.double().requires_grad_(True), beta.double().requires_grad_(True)
    if m > 1:
        yr = F.batch_norm(xd, rm_r, rv_r, gd, bd, True, 0.1, 1e-5)
    else:                      # torch refuses a single value per channel in training mode; the kernel's definition: var = 0
        yr = (xd - xd) * gd / (1e-5 ** 0.5) + bd
    if residual:
        yr = yr + rd
    if relu:
        yr = F.relu(yr)
    tol = 2e-3 if from_partials else 2e-4        # unshifted fp32 sums of squares around a mean of 3 lose a few digits
    assert torch.allclose(y.double(), yr, rtol=tol, atol=tol)
    if m > 1:
        assert torch.allclose(rm.double(), rm_r, rtol=1e-4, atol=1e-5) and torch.allclose(rv.double(), rv_r, rtol=tol, atol=1e-5)
    dy = torch.randn(m, c, generator=g).cuda()
    sums, dx = torch.empty(2 * c, device="cuda"), torch.empty(m, c, device="cuda")
    dres = torch.empty(m, c, device="cuda") if residual else None
    nat.check(lib.gc_cuda_bn_small_backward(dy.data_ptr(), x.data_ptr(), y.data_ptr() if (residual and relu) else None, m, c,
                                            stats.data_ptr(), gamma.data_ptr(), beta.data_ptr(), int(relu), sums.data_ptr(),
                                            dx.data_ptr(), nat.ptr(dres), st()), "small_bwd")
    if m > 1 and not from_partials:
        yr.backward(dy.double())
        scale = float(xd.grad.abs().max()) + 1e-6
        assert float((dx.double() - xd.grad).abs().max()) <= 2e-3 * scale + 1e-5
        assert torch.allclose(sums[:c].double(), bd.grad, rtol=1e-3, atol=1e-3)
        assert torch.allclose(sums[c:].double(), gd.grad, rtol=2e-3, atol=2e-3)
        if residual:
            assert float((dres.double() - rd.grad).abs().max()) <= 1e-5


@pytest.mark.parametrize("name", ["ResNet18", "VGG11"])
def test_batch_counters_follow_the_fused_loss_path(name):
    """``forward_loss`` (the path the trainer and the graphed step take) does not go through ``__call__``: the deferred
    ``num_batches_tracked`` increments must still land, once per training forward."""
    from gradient_compression_b200 import models
    from gradient_compression_b200.ops import bn as bnmod

    model = getattr(models, name)().cuda().to(memory_format=torch.channels_last)
    x = torch.randn(4, 3, 32, 32, device="cuda").contiguous(memory_format=torch.channels_last)
    y = torch.randint(0, 10, (4,), device="cuda")
    model.train()
    for _ in range(3):
        model.forward_loss(x, y)
    assert not bnmod._pending_counters
    counters = [m.num_batches_tracked for m in model.modules() if isinstance(m, torch.nn.BatchNorm2d)]
    assert len(counters) >= 8 and all(int(c) == 3 for c in counters)


def test_batch_counters_are_batched_but_exact():
    """``num_batches_tracked`` of every batch norm of a zoo model moves by one per training forward (one multi-tensor
    launch at the end of the forward), stays put in eval mode, and is counted per use when a layer runs twice."""
    from gradient_compression_b200 import models
    from gradient_compression_b200.ops import bn as bnmod

    model = models.ResNet18().cuda()
    x = torch.randn(4, 3, 32, 32, device="cuda")
    model.train()
    for _ in range(3):
        model(x)
    assert not bnmod._pending_counters
    counters = [m.num_batches_tracked for m in model.modules() if isinstance(m, torch.nn.BatchNorm2d)]
    assert len(counters) > 10 and all(int(c) == 3 for c in counters)
    model.eval()
    model(x)
    assert all(int(c) == 3 for c in counters)
    # one layer used twice in a forward
    class Twice(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.bn = torch.nn.BatchNorm2d(8)
            bnmod.defer_batch_counters(self)

        def forward(self, t):
            return bnmod.bn_act(self.bn, bnmod.bn_act(self.bn, t))

    tw = Twice().cuda()
    tw(torch.randn(4, 8, 8, 8, device="cuda").contiguous(memory_format=torch.channels_last))
    assert int(tw.bn.num_batches_tracked) == 2
