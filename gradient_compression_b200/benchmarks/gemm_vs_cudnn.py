"""tcgen05 TF32 GEMM (``ops.gemm_tf32``) against cuDNN's 1x1 convolution on the ResNet-50 (CIFAR, batch 128) shapes.

    python -m gradient_compression_b200.benchmarks.gemm_vs_cudnn [--sweep]

One JSON line per shape: CUDA-event medians, L2 flushed between launches.
"""
import argparse
import json

import torch

from ..ops import gemm

# (M = N*H*W, K = Cin, N = Cout) of the 1x1 convolutions of the four stages
SHAPES = [(131072, 64, 64), (131072, 64, 256), (131072, 256, 64), (32768, 256, 128), (32768, 128, 512), (32768, 512, 128),
          (8192, 512, 256), (8192, 256, 1024), (8192, 1024, 256), (2048, 1024, 512), (2048, 512, 2048), (2048, 2048, 512)]


def _median_us(fn, flush, iters=10, warmup=3):
    times = []
    for i in range(iters + warmup):
        flush.add_(1.0)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda._sleep(300000)          # the host gets ahead: launch latency stays outside the timed interval
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        if i >= warmup:
            times.append(s.elapsed_time(e) * 1e3)
    times.sort()
    return times[len(times) // 2]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sweep", action="store_true", help="also time both kernels at every tile width")
    ap.add_argument("--wgrad", action="store_true", help="time the weight-gradient (TN, split-K) GEMM against cuDNN's wgrad")
    args = ap.parse_args()
    torch.backends.cudnn.benchmark = True
    flush = torch.zeros(64 << 20, device="cuda")
    for (m, k, n) in SHAPES:
        hw = {131072: 32, 32768: 16, 8192: 8, 2048: 4}[m]
        x = torch.randn(128, k, hw, hw, device="cuda").contiguous(memory_format=torch.channels_last)
        w = torch.randn(n, k, 1, 1, device="cuda").contiguous(memory_format=torch.channels_last)
        a = x.permute(0, 2, 3, 1).reshape(m, k)
        b = w.view(n, k)
        if args.wgrad:
            dy = torch.randn(128, n, hw, hw, device="cuda").contiguous(memory_format=torch.channels_last)
            dy2d = dy.permute(0, 2, 3, 1).reshape(m, n)
            dw = torch.zeros(n, k, device="cuda")
            res = {}
            for ctas, mink in ((2, 8), (1, 8), (4, 8), (2, 4), (2, 16)):
                gemm.configure_tn(ctas, mink)
                res[f"ctas{ctas}_min{mink}"] = round(_median_us(lambda: gemm.gemm_tn_tf32(dy2d, a, out=dw, accumulate=True), flush, iters=6), 1)
            gemm.configure_tn()
            t_cudnn = _median_us(lambda: torch.ops.aten.convolution_backward(dy, x, w, None, [1, 1], [0, 0], [1, 1], False, [0, 0], 1,
                                                                             [False, True, False]), flush, iters=6)
            nbytes = 4 * (m * k + m * n)
            print(json.dumps({"P": m, "Cin": k, "Cout": n, "ours_us": res, "cudnn_us": round(t_cudnn, 1),
                              "roofline_us": round(nbytes / 6566e3, 1)}))
            continue
        out = torch.empty(m, n, device="cuda")
        sweep = {}
        if args.sweep:                        # every kernel / tile width, to calibrate the choice
            for kernel in ("tile", "persistent"):
                for tile_n in (64, 128, 256):
                    if tile_n // 2 >= n:
                        continue
                    gemm.configure(kernel, tile_n)
                    sweep[f"{kernel}{tile_n}"] = round(_median_us(lambda: gemm.gemm_tf32(a, b, out=out), flush, iters=6), 1)
            gemm.configure("tile", 0)
            sweep["tile_auto"] = round(_median_us(lambda: gemm.gemm_tf32(a, b, out=out), flush, iters=6), 1)
        gemm.configure("auto", 0)
        t_ours = _median_us(lambda: gemm.gemm_tf32(a, b, out=out), flush)
        parts = torch.empty(gemm.m_tiles(m), 2, n, device="cuda")
        t_stats = _median_us(lambda: gemm.gemm_tf32(a, b, out=out, col_partials=parts), flush)
        t_cudnn = _median_us(lambda: torch.nn.functional.conv2d(x, w), flush)
        ref = torch.nn.functional.conv2d(x, w).permute(0, 2, 3, 1).reshape(m, n)
        err = float((out - ref).abs().max() / ref.abs().max())
        nbytes = 4 * (m * k + n * k + m * n)
        print(json.dumps({"M": m, "K": k, "N": n, "ours_us": round(t_ours, 1), "ours_with_bn_stats_us": round(t_stats, 1), "cudnn_us": round(t_cudnn, 1),
                          "ours_GBs": round(nbytes / t_ours / 1e3), "ours_TFLOPs": round(2 * m * n * k / t_ours / 1e6, 1),
                          "relerr_vs_cudnn": err, **({"sweep_us": sweep} if sweep else {})}))
    gemm.check()


if __name__ == "__main__":
    main()
