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
