"""Small single-GPU cases of each hot kernel: event-timed, with the algorithmic bytes and the achieved
fraction of the measured copy bandwidth.  Also the workloads used for the ``ncu`` captures under
``profiles/`` (a few hundred MB on the device, a handful of launches).

    python -m gradient_compression_b200.benchmarks.kernel_cases --case qsgd --n 33554432
"""
from __future__ import annotations

import argparse
import json
import os

import torch


def _peak():
    path = os.path.join(os.path.dirname(__file__), "..", "..", "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "of measured"
    except Exception:
        return 6650.0, "of fallback"


def _time(fn, warmup, iters, flush):
    times = []
    for i in range(warmup + iters):
        flush.add_(1.0)                   # 256 MB rewrite: L2 holds nothing of the case's tensors
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(s.elapsed_time(e) * 1e-3)
    times.sort()
    return times[len(times) // 2]


def case_qsgd(n, bits=8):
    from .. import reducers as R
    red = R.QSGDMaxNormReducer("cuda", quantization_level=bits, seed=1, backend="fused")
    x = torch.randn(n, device="cuda") * 1e-3
    out = [torch.empty_like(x)]
    return (lambda: red.reduce([x], out)), 4 * n * 3, "qsgd_fused_kernel (W=1): abs-max read + quantise read + dequantised write"


def case_absmax(n):
    from .. import ops
    x = torch.randn(n, device="cuda")
    out = torch.zeros(1, device="cuda")
    return (lambda: ops.absmax(x, out)), 4 * n, "absmax_kernel: one read"


def case_sgd(n):
    from .. import ops
    p, g, m = (torch.randn(n, device="cuda") for _ in range(3))
    hyper = torch.tensor([0.1, 0.9, 5e-4], device="cuda")
    return (lambda: ops.sgd_step(p, g, m, hyper=hyper)), 4 * n * 5, "sgd_kernel: read p, g, m; write p, m"


def case_pack(n, bits=4):
    from .. import ops
    x = torch.randn(n, device="cuda") * 1e-3
    norm = ops.absmax(x)
    mb, pb = ops.packed_sizes(n, bits)
    mags = torch.empty(mb, dtype=torch.uint8, device="cuda")
    signs = torch.empty(pb // 4, dtype=torch.int32, device="cuda")
    return (lambda: ops.qsgd_pack(x, norm, bits, 1, 1, 0, mags, signs)), 4 * n + mb + pb, "qsgd_pack_kernel: read fp32, write packed"


def _bn_tensors(n):
    c, hw = 256, 32 * 32
    batch = max(n // (c * hw), 1)
    x = torch.randn(batch, c, 32, 32, device="cuda").contiguous(memory_format=torch.channels_last)
    return x, torch.nn.BatchNorm2d(c).cuda()


def case_bn_fwd(n):
    from ..ops.bn import bn_act
    x, bn = _bn_tensors(n)
    with torch.no_grad():
        pass
    return (lambda: bn_act(bn, x)), 4 * x.numel() * 3, "bn_stats + bn_apply (+ReLU): 2 reads, 1 write"


def case_bn_bwd(n):
    from ..ops.bn import bn_act
    x, bn = _bn_tensors(n)
    x.requires_grad_(True)
    dy = torch.randn_like(x)

    def run():
        y = bn_act(bn, x)
        y.backward(dy)
        x.grad = None
    return run, 4 * x.numel() * (3 + 5), "bn fwd (3 passes) + bn_bwd_reduce + bn_bwd_apply (4 reads, 1 write)"


def case_topk(n):
    from ..ops.topk import TopKSelector
    g = torch.randn(n, device="cuda")
    e = torch.zeros(n, device="cuda")
    sel = TopKSelector([(0, n, max(n // 100, 1))], "cuda")
    return (lambda: sel.select(g, e)), 4 * n * 6, "topk: 3 histogram passes + compaction (pass 0 reads g, e and writes e)"


def case_psgd(n, rank=2):
    from .. import reducers as R
    shapes = [(512, 512, 3, 3)] * max(n // (512 * 512 * 9), 1) + [(512,)]
    grads = [torch.randn(s, device="cuda") * 1e-3 for s in shapes]
    red = R.RankKReducer("cuda", rank=rank, seed=1, backend="fused")
    tot = sum(g.numel() for g in grads)
    flat = torch.cat([g.reshape(-1) for g in grads])
    views, off = [], 0
    for g in grads:
        views.append(flat[off:off + g.numel()].view(g.shape))
        off += g.numel()
    return (lambda: red.reduce(views, views)), 4 * tot * 7, "psgd_p (2 reads, 1 write) + psgd_q (1 read) + psgd_out (1 read, 2 writes)"


def case_gemm(n):
    """1x1 convolution of ResNet-50's first stage as a GEMM: [131072, 64] x [256, 64]^T with BN statistics."""
    from ..ops import gemm
    m, k, nn = 131072, 64, 256
    a = torch.randn(m, k, device="cuda")
    b = torch.randn(nn, k, device="cuda")
    out = torch.empty(m, nn, device="cuda")
    part = torch.empty(gemm.m_tiles(m), 2, nn, device="cuda")
    return (lambda: gemm.gemm_tf32(a, b, out=out, col_partials=part)), 4 * (m * k + nn * k + m * nn), \
        "gemm_tf32_persistent_kernel<256>: TMA loads, tcgen05.mma kind::tf32, double-buffered TMEM accumulator, TMA store + column statistics"


def case_gemm_narrow(n):
    """[131072, 64] x [64, 64]^T: the narrowest 1x1 convolution of the first stage (67 MB of traffic, 1 GFLOP)."""
    from ..ops import gemm
    m, k, nn = 131072, 64, 64
    a = torch.randn(m, k, device="cuda")
    b = torch.randn(nn, k, device="cuda")
    out = torch.empty(m, nn, device="cuda")
    return (lambda: gemm.gemm_tf32(a, b, out=out)), 4 * (m * k + nn * k + m * nn), "gemm_tf32_persistent_kernel<64>"


def case_gemm_tn(n):
    """Weight gradient of a first-stage 1x1 convolution: dW[256, 64] = dY[131072, 256]^T X[131072, 64] (168 MB of reads)."""
    from ..ops import gemm
    p, mo, no = 131072, 256, 64
    a = torch.randn(p, mo, device="cuda")
    b = torch.randn(p, no, device="cuda")
    out = torch.zeros(mo, no, device="cuda")
    return (lambda: gemm.gemm_tn_tf32(a, b, out=out, accumulate=True)), 4 * (p * mo + p * no), \
        "gemm_tn_tf32_kernel<64>: MN-major tcgen05 operands, split-K over 148 CTAs, TMA reduce stores"


def case_gemm_deep(n):
    """Compute-heavier GEMM: [8192, 2048] x [2048, 2048]^T (69 GFLOP)."""
    from ..ops import gemm
    m, k, nn = 8192, 2048, 2048
    a = torch.randn(m, k, device="cuda")
    b = torch.randn(nn, k, device="cuda")
    out = torch.empty(m, nn, device="cuda")
    return (lambda: gemm.gemm_tf32(a, b, out=out)), 4 * (m * k + nn * k + m * nn), \
        f"gemm_tf32_kernel: {2 * m * nn * k / 1e9:.0f} GFLOP"


def _conv_tensors(hw=16, c=128, batch=128):
    cl = torch.channels_last
    x = torch.randn(batch, c, hw, hw, device="cuda").contiguous(memory_format=cl)
    w = torch.randn(c, c, 3, 3, device="cuda").contiguous(memory_format=cl)
    return x, w


def case_conv3x3(n):
    """3x3 convolution of ResNet-50's second stage, forward with BN statistics: 128 x 16 x 16 x 128 -> 128 channels."""
    from ..ops import conv, gemm
    x, w = _conv_tensors()
    out = torch.empty_like(x)
    m = x.shape[0] * 256
    part = torch.empty(gemm.m_tiles(m), 2, 128, device="cuda")
    return (lambda: conv.conv_forward(x, w, None, 1, 1, col_partials=part, out=out)), 4 * (2 * x.numel() + w.numel()), \
        f"gemm_tf32_persistent_kernel, A from shifted 4-D TMA boxes: {2 * m * 128 * 1152 / 1e9:.2f} GFLOP"


def case_conv3x3_wgrad(n):
    """Weight gradient of the same layer: dW[128, 9 * 128] from dY and shifted boxes of X."""
    from ..ops import conv
    x, w = _conv_tensors()
    dy = torch.randn_like(x)
    return (lambda: conv.conv_wgrad(dy, x, 3, 1, 1)), 4 * (2 * x.numel() + w.numel()), \
        f"gemm_tn_tf32_kernel, B from shifted 4-D TMA boxes: {2 * x.shape[0] * 256 * 128 * 1152 / 1e9:.2f} GFLOP"


CASES = {"conv3x3": case_conv3x3, "conv3x3_wgrad": case_conv3x3_wgrad, "qsgd": case_qsgd, "absmax": case_absmax, "sgd": case_sgd, "pack": case_pack, "bn_fwd": case_bn_fwd,
         "bn_bwd": case_bn_bwd, "topk": case_topk, "psgd": case_psgd, "gemm": case_gemm, "gemm_narrow": case_gemm_narrow, "gemm_tn": case_gemm_tn,
         "gemm_deep": case_gemm_deep}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--case", nargs="+", default=list(CASES))
    ap.add_argument("--n", type=int, default=1 << 25, help="elements (default 32 Mi = 128 MiB of fp32, above the L2 size)")
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    args = ap.parse_args(argv)
    torch.cuda.set_device(0)
    peak, src = _peak()
    flush = torch.zeros(64 << 20, device="cuda")
    for name in args.case:
        fn, nbytes, what = CASES[name](args.n)
        sec = _time(fn, args.warmup, args.iters, flush)
        gbs = nbytes / sec / 1e9
        print(json.dumps({"case": name, "n": args.n, "us": sec * 1e6, "algorithmic_bytes": nbytes, "GB_per_s": gbs,
                          "fraction_of_copy_peak": gbs / peak, "peak": f"{peak:.0f} GB/s {src}", "what": what}))


if __name__ == "__main__":
    main()
