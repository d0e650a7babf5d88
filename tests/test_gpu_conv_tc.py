"""Implicit-GEMM convolutions on tcgen05 (forward, input gradient, weight gradient, stem gather) against PyTorch
references computed in float64 (``F.conv2d`` / ``aten.convolution_backward``; no TF32 and no transform-domain algorithm
can be picked for doubles).  Exact on small-integer inputs (every product and partial sum is representable in TF32
operands and fp32 sums), TF32 tolerance on random ones."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


class _fp32:
    """fp32 reference arithmetic: no TF32 in cuDNN or cuBLAS while the block runs."""

    def __enter__(self):
        self.c, self.m = torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32
        torch.backends.cudnn.allow_tf32 = False
        torch.backends.cuda.matmul.allow_tf32 = False

    def __exit__(self, *exc):
        torch.backends.cudnn.allow_tf32, torch.backends.cuda.matmul.allow_tf32 = self.c, self.m


def _cl(t):
    return t.contiguous(memory_format=torch.channels_last)


def _ints(shape, g, lo=-3, hi=4):
    return torch.randint(lo, hi, shape, generator=g).float()


def _conv64(x, w, bias, stride, pad):
    return F.conv2d(x.double(), w.double(), None if bias is None else bias.double(), stride=stride, padding=pad).float()


def _conv_backward64(dy, x, w, stride, pad, which):
    mask = [which == 0, which == 1, False]
    return torch.ops.aten.convolution_backward(dy.double(), x.double(), w.double(), None, [stride, stride], [pad, pad], [1, 1],
                                               False, [0, 0], 1, mask)[which].float()


def _same(a, b):
    """Exact equality with a readable failure: how many elements differ and by how much."""
    diff = (a - b).abs()
    bad = int((diff > 0).sum())
    assert bad == 0, f"{bad} of {a.numel()} elements differ, max |diff| {float(diff.max())}, max |ref| {float(b.abs().max())}"


# (N, H, W, Cin, Cout, R, stride, pad): the 3x3 layers of the CIFAR ResNets and VGGs at batch 128 and odd batches, the
# strided 3x3 layers and strided 1x1 projection shortcuts of the ResNets
SHAPES = [
    (4, 32, 32, 64, 64, 3, 1, 1), (3, 32, 32, 64, 128, 3, 1, 1), (8, 16, 16, 128, 128, 3, 1, 1), (5, 16, 16, 128, 256, 3, 1, 1),
    (16, 8, 8, 256, 256, 3, 1, 1), (7, 8, 8, 256, 512, 3, 1, 1), (32, 4, 4, 512, 512, 3, 1, 1), (9, 4, 4, 512, 512, 3, 1, 1),
    (64, 2, 2, 512, 512, 3, 1, 1), (5, 2, 2, 512, 512, 3, 1, 1), (128, 32, 32, 64, 64, 3, 1, 1),
    (4, 32, 32, 128, 128, 3, 2, 1), (6, 16, 16, 256, 256, 3, 2, 1), (16, 8, 8, 512, 512, 3, 2, 1),
    (4, 32, 32, 256, 512, 1, 2, 0), (8, 16, 16, 512, 1024, 1, 2, 0), (16, 8, 8, 1024, 2048, 1, 2, 0),
]


@pytest.mark.parametrize("shape", SHAPES)
def test_conv_forward_exact_on_small_integers(shape):
    from gradient_compression_b200.ops import conv, gemm

    n, h, w, cin, cout, r, stride, pad = shape
    g = torch.Generator().manual_seed(sum(shape))
    x = _cl(_ints((n, cin, h, w), g).cuda())
    wt = _cl(_ints((cout, cin, r, r), g, -2, 3).cuda())
    bias = _ints((cout,), g).cuda()
    lib = conv.nat.cuda()
    assert lib.gc_cuda_conv_fwd_supported(n, h, w, cin, cout, r, stride, pad)
    ref = _conv64(x, wt, bias, stride, pad)
    m = ref.shape[0] * ref.shape[2] * ref.shape[3]
    partials = torch.zeros(gemm.m_tiles(m), 2, cout, device="cuda")
    out = conv.conv_forward(x, wt, bias, stride, pad, col_partials=partials)
    gemm.check()
    assert out.shape == ref.shape and out.is_contiguous(memory_format=torch.channels_last)
    _same(out, ref)
    # epilogue statistics: column sums and sums of squares over all positions
    rd = ref.double()
    assert torch.allclose(partials[:, 0].double().sum(0), rd.sum((0, 2, 3)), rtol=1e-5, atol=1e-3)
    assert torch.allclose(partials[:, 1].double().sum(0), (rd * rd).sum((0, 2, 3)), rtol=1e-5, atol=1e-3)


@pytest.mark.parametrize("shape", SHAPES[:8] + SHAPES[11:13])
def test_conv_forward_random_within_tf32(shape):
    from gradient_compression_b200.ops import conv, gemm

    n, h, w, cin, cout, r, stride, pad = shape
    g = torch.Generator().manual_seed(sum(shape) + 1)
    x = _cl(torch.randn(n, cin, h, w, generator=g).cuda())
    wt = _cl(torch.randn(cout, cin, r, r, generator=g).cuda())
    ref = _conv64(x, wt, None, stride, pad)
    out = conv.conv_forward(x, wt, None, stride, pad)
    gemm.check()
    assert float((out - ref).abs().max() / ref.abs().max()) < 3e-3


@pytest.mark.parametrize("tile_n", [64, 128, 256])
def test_conv_forward_every_tile_width(tile_n):
    from gradient_compression_b200.ops import conv, gemm

    g = torch.Generator().manual_seed(tile_n)
    x = _cl(_ints((6, 256, 16, 16), g).cuda())
    wt = _cl(_ints((256, 256, 3, 3), g, -2, 3).cuda())
    ref = _conv64(x, wt, None, 1, 1)
    gemm.configure("auto", tile_n)
    try:
        out = conv.conv_forward(x, wt, None, 1, 1)
    finally:
        gemm.configure("auto", 0)
    gemm.check()
    _same(out, ref)


@pytest.mark.parametrize("splits", [1, 2, 3, 5])
@pytest.mark.parametrize("shape", [(32, 4, 4, 512, 512, 3, 1, 1), (9, 8, 8, 256, 256, 3, 1, 1), (16, 8, 8, 512, 512, 3, 2, 1),
                                   (8, 16, 16, 512, 1024, 1, 2, 0)])
def test_conv_forward_split_contraction(shape, splits):
    """The same convolution with its contraction cut into `splits` work items per output tile (partial tiles added in L2
    onto a zeroed output; the bias rides on the first split only) and onto an output that already holds values."""
    from gradient_compression_b200.ops import conv, gemm

    n, h, w, cin, cout, r, stride, pad = shape
    g = torch.Generator().manual_seed(sum(shape) + splits)
    x = _cl(_ints((n, cin, h, w), g).cuda())
    wt = _cl(_ints((cout, cin, r, r), g, -2, 3).cuda())
    bias = _ints((cout,), g).cuda()
    ref = _conv64(x, wt, bias, stride, pad)
    gemm.configure_split(splits)
    try:
        out = conv.conv_forward(x, wt, bias, stride, pad)
        prior = _cl(_ints(tuple(ref.shape), g).cuda())
        acc = conv.conv_forward(x, wt, bias, stride, pad, out=prior.clone(memory_format=torch.preserve_format), accumulate=True)
    finally:
        gemm.configure_split(0)
    gemm.check()
    _same(out, ref)
    _same(acc, ref + prior)


@pytest.mark.parametrize("splits", [0, 2, 4])
@pytest.mark.parametrize("m,n,k,ldc", [(2048, 512, 2048, 512), (2048, 2048, 512, 2048), (1000, 96, 1024, 128), (512, 256, 4096, 256)])
def test_gemm_split_contraction(m, n, k, ldc, splits):
    from gradient_compression_b200.ops import gemm

    g = torch.Generator().manual_seed(m + n + k + splits)
    a = _ints((m, k), g).cuda()
    b = _ints((n, k), g, -2, 3).cuda()
    bias = _ints((n,), g).cuda()
    buf = torch.full((m, ldc), 7.0, device="cuda")
    ref = (a.double() @ b.double().t() + bias.double()).float()
    gemm.configure_split(splits)
    try:
        gemm.gemm_tf32(a, b, bias=bias, out=buf[:, :n])
    finally:
        gemm.configure_split(0)
    gemm.check()
    _same(buf[:, :n], ref)
    if ldc > n:
        assert float((buf[:, n:] - 7.0).abs().max()) == 0.0      # the zeroing of a split output stays inside its columns


@pytest.mark.parametrize("shape", [s for s in SHAPES if s[6] == 1])
def test_conv_input_gradient_exact_on_small_integers(shape):
    """dX = forward kernel on dY with the rotated, channel-swapped filter; also accumulating onto a tensor."""
    from gradient_compression_b200.ops import conv, gemm

    n, h, w, cin, cout, r, stride, pad = shape
    g = torch.Generator().manual_seed(sum(shape) + 2)
    x = _cl(_ints((n, cin, h, w), g).cuda())
    wt = _cl(_ints((cout, cin, r, r), g, -2, 3).cuda())
    dy = _cl(_ints((n, cout, h, w), g).cuda())
    ref = _conv_backward64(dy, x, wt, 1, pad, 0)
    wd = conv._dgrad_weights.get(wt)
    dx = conv.conv_forward(dy, wd, None, 1, r - 1 - pad)
    gemm.check()
    _same(dx, ref)
    base = _cl(_ints((n, cin, h, w), g).cuda())
    acc = base.clone(memory_format=torch.preserve_format)
    conv.conv_forward(dy, wd, None, 1, r - 1 - pad, out=acc, accumulate=True)
    gemm.check()
    _same(acc, base + ref)


@pytest.mark.parametrize("tile_n", [0, 64, 128, 256])
@pytest.mark.parametrize("shape", [s for s in SHAPES if s[6] == 1] + [(6, 16, 16, 96, 64, 3, 1, 1), (4, 7, 9, 64, 160, 1, 1, 0),
                                                                     (128, 4, 4, 2048, 512, 1, 1, 0), (5, 8, 8, 64, 64, 3, 1, 0),
                                                                     (4, 8, 8, 48, 64, 3, 1, 1), (6, 8, 8, 80, 96, 1, 1, 0)])
def test_conv_input_gradient_reading_the_filter_in_place(shape, tile_n):
    """dX with the forward filter [Cout][R][S][Cin] as the MN-major B operand (taps rotated by the kernel's addressing, no
    transposed copy); plain, accumulating, and with the contraction split where the cost model says so."""
    from gradient_compression_b200.ops import conv, gemm

    n, h, w, cin, cout, r, stride, pad = shape
    if tile_n and tile_n // 2 >= cin:
        pytest.skip("tile wider than the output")
    g = torch.Generator().manual_seed(sum(shape) + 12)
    x = _cl(_ints((n, cin, h, w), g).cuda())
    wt = _cl(_ints((cout, cin, r, r), g, -2, 3).cuda())
    ho, wo = h + 2 * pad - r + 1, w + 2 * pad - r + 1
    dy = _cl(_ints((n, cout, ho, wo), g).cuda())
    lib = conv.nat.cuda()
    assert lib.gc_cuda_conv_dgrad_supported(n, h, w, cin, cout, r, pad)
    ref = _conv_backward64(dy, x, wt, 1, pad, 0)
    base = _cl(_ints((n, cin, h, w), g).cuda())
    dx, acc = torch.full_like(x, 7.0), base.clone(memory_format=torch.preserve_format)
    gemm.configure("auto", tile_n)
    try:
        for out, accumulate in ((dx, 0), (acc, 1)):
            conv.nat.check(lib.gc_cuda_conv_dgrad(dy.data_ptr(), wt.data_ptr(), out.data_ptr(), n, h, w, cin, cout, r, pad, accumulate,
                                                  gemm._error_flag(x.device).data_ptr(), conv.nat.stream_ptr()), "conv_dgrad")
    finally:
        gemm.configure("auto", 0)
    gemm.check()
    _same(dx, ref)
    _same(acc, base + ref)


def test_dgrad_filter_refresh_kernel_matches_torch():
    """The batched kernel that rebuilds rotated / transposed filters after an optimiser step."""
    from gradient_compression_b200.ops import conv

    g = torch.Generator().manual_seed(11)
    ws = [torch.nn.Parameter(_cl(torch.randn(c_out, c_in, r, r, generator=g).cuda()))
          for c_out, c_in, r in [(64, 64, 3), (96, 40, 1), (128, 64, 3), (32, 256, 1)]]
    table = conv._DgradWeights()
    expect = [table.get(w).clone() for w in ws]            # torch path (flip + permute)
    expect2 = [table.get(w, 2, (w.shape[2] - 1) // 2).clone() for w in ws]       # stride-2 layout: one matrix per parity class
    for e in table.entries.values():
        e[1].zero_()
    table.invalidate()

    class Owner:
        pass

    table.refresh(Owner(), ws)
    torch.cuda.synchronize()
    for w, want, want2 in zip(ws, expect, expect2):
        assert torch.equal(table.entries[(id(w), 1)][1], want)
        assert torch.equal(table.entries[(id(w), 2)][1], want2)


@pytest.mark.parametrize("shape", [s for s in SHAPES if s[6] == 2] + [(3, 8, 8, 64, 96, 3, 2, 1), (5, 4, 4, 128, 64, 1, 2, 0)])
def test_conv_stride2_input_gradient_exact_on_small_integers(shape):
    """Four launches, one per parity class of input pixels, each storing through a strided 4-D map and reading its taps of the
    forward filter in place."""
    from gradient_compression_b200.ops import conv, gemm

    n, h, w, cin, cout, r, stride, pad = shape
    g = torch.Generator().manual_seed(sum(shape) + 4)
    x = _cl(_ints((n, cin, h, w), g).cuda())
    wt = _cl(_ints((cout, cin, r, r), g, -2, 3).cuda())
    dy = _cl(_ints((n, cout, h // 2, w // 2), g).cuda())
    lib = conv.nat.cuda()
    assert lib.gc_cuda_conv_dgrad_s2_supported(n, h, w, cin, cout, r, pad)
    ref = _conv_backward64(dy, x, wt, 2, pad, 0)
    dx = torch.full_like(x, 7.0)
    conv.nat.check(lib.gc_cuda_conv_dgrad_s2(dy.data_ptr(), wt.data_ptr(), dx.data_ptr(), n, h, w, cin, cout, r, pad,
                                             gemm._error_flag(x.device).data_ptr(), conv.nat.stream_ptr()), "conv_dgrad_s2")
    gemm.check()
    _same(dx, ref)


@pytest.mark.parametrize("shape", [s for s in SHAPES if s[3] % 64 == 0])
def test_conv_weight_gradient_exact_on_small_integers(shape):
    from gradient_compression_b200.ops import conv, gemm

    n, h, w, cin, cout, r, stride, pad = shape
    g = torch.Generator().manual_seed(sum(shape) + 3)
    x = _cl(_ints((n, cin, h, w), g, -2, 3).cuda())
    wt = _cl(_ints((cout, cin, r, r), g).cuda())
    ho, wo = (h + 2 * pad - r) // stride + 1, (w + 2 * pad - r) // stride + 1
    dy = _cl(_ints((n, cout, ho, wo), g, -2, 3).cuda())
    assert conv.nat.cuda().gc_cuda_conv_wgrad_supported(n, h, w, cin, cout, r, stride, pad)
    ref = _conv_backward64(dy, x, wt, stride, pad, 1)
    dw = conv.conv_wgrad(dy, x, r, stride, pad).view(cout, r, r, cin).permute(0, 3, 1, 2)
    gemm.check()
    _same(dw, ref)


@pytest.mark.parametrize("n,cout", [(4, 64), (7, 64), (128, 64)])
def test_stem_gather_and_gemm_match_conv(n, cout):
    """The 3-channel first layer: gathered rows of 32 floats, then the K = 32 GEMM."""
    from gradient_compression_b200.ops import conv, gemm

    g = torch.Generator().manual_seed(n)
    x = _cl(_ints((n, 3, 32, 32), g).cuda())
    wt = _cl(_ints((cout, 3, 3, 3), g, -2, 3).cuda())
    ref = _conv64(x, wt, None, 1, 1)
    lib = conv.nat.cuda()
    a = torch.empty(n * 32 * 32, conv.STEM_K, device="cuda")
    wpad = torch.empty(cout, conv.STEM_K, device="cuda")
    conv.nat.check(lib.gc_cuda_im2col_small(x.data_ptr(), a.data_ptr(), n, 32, 32, 3, 3, 1, conv.STEM_K, wt.data_ptr(),
                                            wpad.data_ptr(), cout, conv.nat.stream_ptr()), "im2col_small")
    out = gemm.gemm_tf32(a, wpad).view(n, 32, 32, cout).permute(0, 3, 1, 2)
    gemm.check()
    _same(out, ref)
    assert torch.equal(wpad[:, :27], wt.permute(0, 2, 3, 1).reshape(cout, 27)) and float(wpad[:, 27:].abs().max()) == 0.0


def _block(cin, cout, r, stride, bias):
    conv_ = torch.nn.Conv2d(cin, cout, r, stride=stride, padding=(r - 1) // 2, bias=bias)
    bn_ = torch.nn.BatchNorm2d(cout)
    with torch.no_grad():
        bn_.weight.uniform_(0.5, 1.5)
        bn_.bias.uniform_(-0.5, 0.5)
    return conv_, bn_


@pytest.mark.parametrize("cin,cout,r,stride,hw,bias,res", [
    (64, 64, 3, 1, 32, False, False), (64, 128, 3, 1, 16, True, False), (128, 128, 3, 2, 16, False, False),
    (3, 64, 3, 1, 32, False, False), (3, 64, 3, 1, 32, True, False), (256, 512, 1, 2, 16, False, False),
    (256, 256, 3, 1, 8, False, True), (512, 512, 3, 1, 2, True, False), (256, 64, 1, 1, 8, False, False),
    (512, 512, 3, 1, 4, False, True), (2048, 512, 1, 1, 4, False, False)])
def test_conv_bn_act_matches_unfused_modules(cin, cout, r, stride, hw, bias, res):
    """The fused layer (tensor-core convolution + epilogue statistics + BN apply, and its backward) against the same
    modules run one after the other in fp32."""
    from gradient_compression_b200.ops import conv, gemm

    torch.manual_seed(cin + cout + r + stride + hw)
    conv_, bn_ = _block(cin, cout, r, stride, bias)
    conv_, bn_ = conv_.cuda().to(memory_format=torch.channels_last), bn_.cuda()
    conv_r, bn_r = _block(cin, cout, r, stride, bias)
    conv_r, bn_r = conv_r.cuda().double(), bn_r.cuda().double()
    conv_r.load_state_dict(conv_.state_dict())
    bn_r.load_state_dict(bn_.state_dict())
    n = 8
    x = _cl(torch.randn(n, cin, hw, hw, device="cuda")).requires_grad_(cin > 3)
    xr = x.detach().double().requires_grad_(cin > 3)
    ho = (hw + 2 * ((r - 1) // 2) - r) // stride + 1
    resid = _cl(torch.randn(n, cout, ho, ho, device="cuda")).requires_grad_(True) if res else None
    resid_r = resid.detach().double().requires_grad_(True) if res else None
    assert conv._mode(conv_, bn_, x) is not None
    y = conv.conv_bn_act(conv_, bn_, x, residual=resid)
    yr = bn_r(conv_r(xr))
    if res:
        yr = yr + resid_r
    yr = F.relu(yr)
    gy = _cl(torch.randn_like(y))
    y.backward(gy)
    yr.backward(gy.double())
    gemm.check()

    def close(a, b, tol=5e-3):
        """Agreement at TF32 level in the Frobenius norm (with ReLU a few pre-activations within rounding distance of
        zero land on different sides, which changes those elements' gradient by O(dy))."""
        a, b = a.detach().double(), b.detach().double()
        err = float((a - b).norm() / b.norm().clamp_min(1e-30))
        assert err <= tol, f"relative Frobenius error {err} above {tol}"
        return True

    assert close(y, yr)
    assert close(bn_.running_mean, bn_r.running_mean) and close(bn_.running_var, bn_r.running_var)
    assert close(conv_.weight.grad, conv_r.weight.grad, 6e-2)
    assert close(bn_.weight.grad, bn_r.weight.grad, 6e-2) and close(bn_.bias.grad, bn_r.bias.grad, 6e-2)
    if cin > 3:
        assert close(x.grad, xr.grad, 6e-2)
    if res:
        assert close(resid.grad, resid_r.grad, 6e-2)
    if bias:
        assert float(conv_.bias.grad.abs().max()) == 0.0 and float(conv_r.bias.grad.abs().max()) < 1e-2


@pytest.mark.parametrize("cin,cout,hw,n,training", [(64, 64, 32, 4, True), (128, 256, 8, 16, True), (512, 512, 2, 32, True),
                                                     (3, 64, 32, 8, True), (256, 256, 4, 8, False)])
def test_conv_bn_relu_maxpool_in_one_pass(cin, cout, hw, n, training):
    """VGG's conv + BN + ReLU + 2x2 max-pool with the pool folded into the BN kernels (the full-resolution activation is never
    written; the backward routes the pooled gradient to each window's winner) against the four modules in float64."""
    from gradient_compression_b200.ops import conv, gemm

    torch.manual_seed(cin + cout + hw)
    conv_, bn_ = _block(cin, cout, 3, 1, True)
    conv_, bn_ = conv_.cuda().to(memory_format=torch.channels_last), bn_.cuda()
    conv_r, bn_r = _block(cin, cout, 3, 1, True)
    conv_r, bn_r = conv_r.cuda().double(), bn_r.cuda().double()
    conv_r.load_state_dict(conv_.state_dict())
    bn_r.load_state_dict(bn_.state_dict())
    for mod in (conv_, bn_, conv_r, bn_r):
        mod.train(training)
    x = _cl(torch.randn(n, cin, hw, hw, device="cuda")).requires_grad_(cin > 3 and training)
    xr = x.detach().double().requires_grad_(cin > 3 and training)
    with torch.set_grad_enabled(training):          # (an eval-mode layer takes the kernels only where no gradient is asked for)
        assert conv._mode(conv_, bn_, x) is not None and conv.nat.cuda().gc_cuda_bn_pool_supported(n, hw, hw, cout)
        y = conv.conv_bn_act(conv_, bn_, x, pool=True)
        yr = F.max_pool2d(F.relu(bn_r(conv_r(xr))), 2, 2)
    assert y.shape == yr.shape

    def close(a, b, tol):
        a, b = a.detach().double(), b.detach().double()
        err = float((a - b).norm() / b.norm().clamp_min(1e-30))
        assert err <= tol, f"relative Frobenius error {err} above {tol}"

    close(y, yr, 5e-3)
    if training:
        gy = _cl(torch.randn_like(y))
        y.backward(gy)
        yr.backward(gy.double())
        gemm.check()
        close(conv_.weight.grad, conv_r.weight.grad, 6e-2)
        close(bn_.weight.grad, bn_r.weight.grad, 6e-2)
        close(bn_.bias.grad, bn_r.bias.grad, 6e-2)
        close(bn_.running_var, bn_r.running_var, 5e-3)
        if cin > 3:
            close(x.grad, xr.grad, 6e-2)


def test_bn_pool_kernels_match_the_unfused_kernels_exactly():
    """Same arithmetic as BN apply followed by torch's max-pool: the pooled forward is bit-identical; the backward equals the
    plain BN backward fed with torch's max-pool backward up to the order of the channel sums."""
    from gradient_compression_b200.ops import bn as bnmod
    from gradient_compression_b200.ops import _native as nat

    lib, st = nat.cuda(), nat.stream_ptr
    n, c, h, w = 6, 128, 12, 20
    g = torch.Generator().manual_seed(4)
    y = _cl(torch.randn(n, c, h, w, generator=g).cuda() * 2 + 0.3)
    gamma, beta = torch.randn(c, generator=g).cuda(), torch.randn(c, generator=g).cuda()
    mean, var = y.mean((0, 2, 3)), y.var((0, 2, 3), unbiased=False)
    stats = torch.cat([mean, torch.rsqrt(var + 1e-5)]).contiguous()
    m = n * h * w
    act = torch.empty_like(y)
    nat.check(lib.gc_cuda_bn_apply(y.data_ptr(), m, c, stats.data_ptr(), gamma.data_ptr(), beta.data_ptr(), None, 1, act.data_ptr(), st()), "a")
    pooled = torch.empty(n, c, h // 2, w // 2, device="cuda").contiguous(memory_format=torch.channels_last)
    nat.check(lib.gc_cuda_bn_apply_pool(y.data_ptr(), n, h, w, c, stats.data_ptr(), gamma.data_ptr(), beta.data_ptr(), 1,
                                        pooled.data_ptr(), st()), "b")
    ref_pool = F.max_pool2d(act, 2, 2)
    assert torch.equal(pooled, ref_pool)
    # backward: route dpool with torch's pooling backward, then the plain kernels
    dpool = _cl(torch.randn(n, c, h // 2, w // 2, generator=g).cuda())
    a = act.clone().requires_grad_(True)
    F.max_pool2d(a, 2, 2).backward(dpool)
    dfull = _cl(a.grad)
    scratch = bnmod._scratch_for(y.device, c)
    sums_a, sums_b = torch.empty(2 * c, device="cuda"), torch.empty(2 * c, device="cuda")
    dx_a, dx_b = torch.empty_like(y), torch.empty_like(y)
    nat.check(lib.gc_cuda_bn_bwd_reduce(dfull.data_ptr(), y.data_ptr(), None, m, c, stats.data_ptr(), gamma.data_ptr(), beta.data_ptr(), 1,
                                        scratch.data_ptr(), sums_a.data_ptr(), None, st()), "c")
    nat.check(lib.gc_cuda_bn_bwd_apply(dfull.data_ptr(), y.data_ptr(), None, m, c, stats.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                                       sums_a.data_ptr(), 1, dx_a.data_ptr(), None, st()), "d")
    nat.check(lib.gc_cuda_bn_bwd_reduce_pool(dpool.data_ptr(), y.data_ptr(), n, h, w, c, stats.data_ptr(), gamma.data_ptr(), beta.data_ptr(), 1,
                                             scratch.data_ptr(), sums_b.data_ptr(), st()), "e")
    nat.check(lib.gc_cuda_bn_bwd_apply_pool(dpool.data_ptr(), y.data_ptr(), n, h, w, c, stats.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                                            sums_b.data_ptr(), 1, dx_b.data_ptr(), st()), "f")
    assert torch.allclose(sums_a, sums_b, rtol=1e-5, atol=1e-4)
    assert torch.allclose(dx_a, dx_b, rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("m,n,k", [(131072, 64, 64), (4096, 256, 128), (2048, 2048, 512), (1000, 96, 64), (128 * 300, 512, 32)])
def test_gemm_finishes_batch_norm_statistics_itself(m, n, k):
    """The GEMM's own finalize (per-CTA column sums, atomics, last-ticket epilogue group) against the statistics of its
    output computed in float64; the scratch it uses must come back zeroed (two launches in a row)."""
    from gradient_compression_b200.ops import gemm

    g = torch.Generator().manual_seed(m + n + k)
    a = (torch.randn(m, k, generator=g) + 0.5).cuda()
    b = torch.randn(n, k, generator=g).cuda()
    out = torch.empty(m, n, device="cuda")
    for momentum in (0.1, 0.3):
        stats = torch.empty(2 * n, device="cuda")
        rm, rv = torch.zeros(n, device="cuda"), torch.ones(n, device="cuda")
        fin = gemm.bn_fin_args(a.device, stats, rm, rv, momentum, 1e-5)
        gemm.gemm_tf32(a, b, out=out, bn_fin=fin)
        gemm.check()
        o = out.double()
        mean, var = o.mean(0), o.var(0, unbiased=False)
        assert torch.allclose(stats[:n].double(), mean, rtol=1e-4, atol=1e-4)
        assert torch.allclose(stats[n:].double(), 1.0 / torch.sqrt(var + 1e-5), rtol=1e-4, atol=1e-6)
        assert torch.allclose(rm.double(), momentum * mean, rtol=1e-4, atol=1e-4)
        assert torch.allclose(rv.double(), (1 - momentum) + momentum * var * m / (m - 1), rtol=1e-4, atol=1e-5)
    assert int(gemm._fin_scratch[("cuda", a.device.index)].count_nonzero()) == 0
