"""tcgen05 TF32 GEMM against an fp32 PyTorch matmul (TF32 keeps 10 mantissa bits per operand)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("m,n,k", [(128, 128, 32), (128, 16, 64), (256, 64, 128), (1000, 256, 576), (131, 10, 2048),
                                   (4096, 512, 64), (300, 200, 100), (128, 128, 36), (1024, 256, 64), (333, 1000, 128),
                                   (2048, 2048, 512)])
def test_gemm_tf32_matches_fp32(m, n, k):
    from gradient_compression_b200.ops import gemm

    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randn(m, k, generator=g).cuda()
    b = torch.randn(n, k, generator=g).cuda()
    bias = torch.randn(n, generator=g).cuda()
    assert gemm.supported(a, b)
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = False
    try:
        ref = a @ b.t() + bias
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old
    out = gemm.gemm_tf32(a, b, bias)
    gemm.check()
    err = (out - ref).abs().max() / ref.abs().max()
    assert float(err) < 3e-3, float(err)
    out2 = gemm.gemm_tf32(a, b)                # no bias, second launch reuses the configured kernel
    gemm.check()
    assert float((out2 + bias - ref).abs().max() / ref.abs().max()) < 3e-3


def test_gemm_exact_on_tf32_representable_inputs():
    from gradient_compression_b200.ops import gemm

    g = torch.Generator().manual_seed(0)
    a = torch.randint(-8, 9, (256, 96), generator=g).float().cuda()       # small integers: exact in TF32 and in fp32 sums
    b = torch.randint(-8, 9, (48, 96), generator=g).float().cuda()
    out = gemm.gemm_tf32(a, b)
    gemm.check()
    assert torch.equal(out, a @ b.t())


def test_unsupported_shapes_fall_back():
    from gradient_compression_b200.ops import gemm

    a = torch.randn(64, 27, device="cuda")      # row stride 27 * 4 bytes is not a multiple of 16
    b = torch.randn(8, 27, device="cuda")
    assert not gemm.supported(a, b)
    assert torch.allclose(gemm.gemm_tf32(a, b), a @ b.t(), atol=1e-4)


def test_gemm_into_strided_and_unaligned_outputs():
    """C with a row stride that breaks the TMA store rules takes the plain-store epilogue; a wider aligned
    row stride takes the TMA store."""
    from gradient_compression_b200.ops import gemm

    g = torch.Generator().manual_seed(3)
    a = torch.randint(-4, 5, (200, 64), generator=g).float().cuda()
    b = torch.randint(-4, 5, (72, 64), generator=g).float().cuda()
    ref = a @ b.t()
    wide = torch.zeros(200, 80, device="cuda")
    gemm.gemm_tf32(a, b, out=wide[:, :72])
    assert torch.equal(wide[:, :72], ref) and float(wide[:, 72:].abs().max()) == 0.0
    odd = torch.zeros(200, 73, device="cuda")
    gemm.gemm_tf32(a, b, out=odd[:, :72])
    gemm.check()
    assert torch.equal(odd[:, :72], ref) and float(odd[:, 72:].abs().max()) == 0.0


@pytest.fixture
def gemm_choice():
    from gradient_compression_b200.ops import gemm

    yield gemm.configure
    gemm.configure("auto", 0)


@pytest.mark.parametrize("kernel,tile_n", [("tile", 64), ("tile", 128), ("tile", 256), ("persistent", 64), ("persistent", 128),
                                           ("persistent", 256)])
@pytest.mark.parametrize("m,n,k", [(128, 64, 32), (1000, 256, 576), (4096, 512, 64), (300, 200, 100), (20000, 320, 96),
                                   (131, 40, 2048), (38000, 64, 64)])
def test_both_kernels_every_tile_width(gemm_choice, kernel, tile_n, m, n, k):
    """Exact on small-integer inputs (TF32 represents them, fp32 sums are exact): any mix-up of tiles, accumulator
    buffers, staging slabs or pipeline phases shows as a wrong entry.  The larger cases give every CTA of the
    persistent kernel several tiles, so both TMEM buffers and the whole staging ring are reused."""
    from gradient_compression_b200.ops import gemm

    g = torch.Generator().manual_seed(m * 7 + n * 3 + k)
    a = torch.randint(-4, 5, (m, k), generator=g).float().cuda()
    b = torch.randint(-4, 5, (n, k), generator=g).float().cuda()
    bias = torch.randint(-9, 10, (n,), generator=g).float().cuda()
    ref = a.double() @ b.double().t() + bias.double()
    gemm_choice(kernel, tile_n)
    out = torch.full((m, n), float("nan"), device="cuda")
    gemm.gemm_tf32(a, b, bias, out=out)
    gemm.check()
    assert torch.equal(out.double(), ref)
    # column statistics of the same product
    parts = torch.full((gemm.m_tiles(m), 2, n), float("nan"), device="cuda")
    out2 = torch.empty(m, n, device="cuda")
    gemm.gemm_tf32(a, b, bias, out=out2, col_partials=parts)
    gemm.check()
    assert torch.equal(out2.double(), ref)
    assert torch.equal(parts[:, 0].double().sum(0), ref.sum(0))
    assert torch.allclose(parts[:, 1].double().sum(0), (ref * ref).sum(0), rtol=1e-5)


@pytest.mark.parametrize("kernel", ["tile", "persistent"])
def test_chosen_tile_width_random_inputs(gemm_choice, kernel):
    from gradient_compression_b200.ops import gemm

    gemm_choice(kernel, 0)
    for (m, n, k) in [(131072, 64, 64), (32768, 512, 128), (8192, 256, 1024), (2048, 2048, 512)]:
        a = torch.randn(m, k, device="cuda")
        b = torch.randn(n, k, device="cuda")
        ref = (a.double() @ b.double().t()).float()
        out = gemm.gemm_tf32(a, b)
        gemm.check()
        assert float((out - ref).abs().max() / ref.abs().max()) < 3e-3


@pytest.mark.parametrize("m,n,k", [(1000, 256, 96), (20000, 64, 64), (4096, 40, 200)])
def test_accumulate_adds_onto_the_output(m, n, k):
    """``accumulate=True``: C += A B^T through TMA reduce stores; exact on small integers, rows and columns outside the
    product untouched."""
    from gradient_compression_b200.ops import gemm

    g = torch.Generator().manual_seed(m + n + k)
    a = torch.randint(-4, 5, (m, k), generator=g).float().cuda()
    b = torch.randint(-4, 5, (n, k), generator=g).float().cuda()
    c0 = torch.randint(-100, 101, (m + 3, n + 8), generator=g).float().cuda()
    c = c0.clone()
    gemm.gemm_tf32(a, b, out=c[:m, :n], accumulate=True)
    gemm.check()
    ref = c0.clone()
    ref[:m, :n] += a @ b.t()
    assert torch.equal(c, ref)
    gemm.gemm_tf32(a, b, out=c[:m, :n], accumulate=True)          # twice: the reduce really reads what is there
    ref[:m, :n] += a @ b.t()
    assert torch.equal(c, ref)


@pytest.mark.parametrize("p,mo,no", [(64, 128, 64), (4096, 64, 256), (40000, 256, 64), (1000, 96, 160), (8192, 512, 128),
                                     (2048, 2048, 512), (33, 32, 32)])
def test_gemm_tn_weight_gradient_shape(p, mo, no):
    """out = A^T B with the contraction over the rows (both operands MN-major for the tensor core, split-K with TMA
    reduce stores).  Small integers: TF32 represents them and every partial sum is exact in fp32, so the result
    is exact whatever the order in which the splits land."""
    from gradient_compression_b200.ops import gemm

    g = torch.Generator().manual_seed(p + mo + no)
    a = torch.randint(-3, 4, (p, mo), generator=g).float().cuda()
    b = torch.randint(-3, 4, (p, no), generator=g).float().cuda()
    out = torch.full((mo, no), float("nan"), device="cuda")
    assert gemm.tn_supported(a, b, out)
    gemm.gemm_tn_tf32(a, b, out=out)
    gemm.check()
    ref = (a.double().t() @ b.double())
    assert torch.equal(out.double(), ref)
    gemm.gemm_tn_tf32(a, b, out=out, accumulate=True)
    gemm.check()
    assert torch.equal(out.double(), 2 * ref)


def test_gemm_tn_random_inputs_and_fallback():
    from gradient_compression_b200.ops import gemm

    a = torch.randn(20000, 128, device="cuda")
    b = torch.randn(20000, 96, device="cuda")
    ref = (a.double().t() @ b.double()).float()
    out = gemm.gemm_tn_tf32(a, b)
    gemm.check()
    assert float((out - ref).abs().max() / ref.abs().max()) < 3e-3
    a2, b2 = torch.randn(500, 20, device="cuda"), torch.randn(500, 12, device="cuda")      # not multiples of 32: plain matmul
    assert torch.allclose(gemm.gemm_tn_tf32(a2, b2), a2.t() @ b2, atol=1e-3)
