"""Implicit-GEMM convolutions on tcgen05 (``ops.conv``) against cuDNN on the 3x3 and strided layers of the CIFAR
ResNet-50 and VGG-16 at batch 128: forward (with the BN statistics epilogue), input gradient, weight gradient.

    python -m gradient_compression_b200.benchmarks.conv_vs_cudnn [--sweep] [--batch 128]

One JSON line per shape: CUDA-event medians in microseconds, L2 flushed between launches, cuDNN autotuned
(``cudnn.benchmark``) with TF32 allowed, as in the training step.
"""
import argparse
import json

import torch
import torch.nn.functional as F

from ..ops import conv, gemm
from .gemm_vs_cudnn import _median_us

# (H = W, Cin, Cout, R, stride): ResNet-50 3x3 stride 1, 3x3 stride 2, strided 1x1 shortcuts; VGG-16's other shapes
SHAPES = [(32, 64, 64, 3, 1), (16, 128, 128, 3, 1), (8, 256, 256, 3, 1), (4, 512, 512, 3, 1),
          (32, 128, 128, 3, 2), (16, 256, 256, 3, 2), (8, 512, 512, 3, 2),
          (32, 256, 512, 1, 2), (16, 512, 1024, 1, 2), (8, 1024, 2048, 1, 2),
          (16, 64, 128, 3, 1), (8, 128, 256, 3, 1), (4, 256, 512, 3, 1), (2, 512, 512, 3, 1)]


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--sweep", action="store_true", help="also time the forward kernel at every tile width")
    ap.add_argument("--batch", type=int, default=128)
    ap.add_argument("--no-split", action="store_true", help="never split the contraction of the forward / input-gradient kernel")
    args = ap.parse_args()
    if args.no_split:
        gemm.configure_split(1)
    torch.backends.cudnn.benchmark = True
    cl = torch.channels_last
    flush = torch.zeros(64 << 20, device="cuda")
    n = args.batch
    for (hw, cin, cout, r, stride) in SHAPES:
        pad = (r - 1) // 2
        x = torch.randn(n, cin, hw, hw, device="cuda").contiguous(memory_format=cl)
        w = torch.randn(cout, cin, r, r, device="cuda").contiguous(memory_format=cl)
        ho = (hw + 2 * pad - r) // stride + 1
        dy = torch.randn(n, cout, ho, ho, device="cuda").contiguous(memory_format=cl)
        m = n * ho * ho
        row = {"HW": hw, "Cin": cin, "Cout": cout, "R": r, "stride": stride, "GFLOP": round(2e-9 * m * cout * r * r * cin, 2)}
        out = torch.empty(n, cout, ho, ho, device="cuda").contiguous(memory_format=cl)
        parts = torch.empty(gemm.m_tiles(m), 2, cout, device="cuda")
        row["fwd_us"] = round(_median_us(lambda: conv.conv_forward(x, w, None, stride, pad, col_partials=parts, out=out), flush), 1)
        row["fwd_cudnn_us"] = round(_median_us(lambda: F.conv2d(x, w, None, stride, pad), flush), 1)
        splits = conv.nat.cuda().gc_cuda_conv_fwd_splits(n, hw, hw, cin, cout, r, stride, pad)
        if splits > 1 and not args.no_split:
            # what the layer runs instead: split contraction, then the statistics in a pass of their own
            from ..ops import bn
            stats = torch.empty(2 * cout, device="cuda")
            scratch = bn._scratch_for(x.device, cout)

            def split_fwd():
                conv.conv_forward(x, w, None, stride, pad, out=out)
                conv.nat.cuda().gc_cuda_bn_stats(out.data_ptr(), m, cout, scratch.data_ptr(), stats.data_ptr(), None, None, 0.1, 1e-5,
                                                 conv.nat.stream_ptr())
            row["fwd_split_plus_stats_us"] = round(_median_us(split_fwd, flush), 1)
        if args.sweep:
            sw = {}
            for tile_n in (64, 128, 256):
                if tile_n // 2 >= cout:
                    continue
                gemm.configure("auto", tile_n)
                sw[str(tile_n)] = round(_median_us(lambda: conv.conv_forward(x, w, None, stride, pad, out=out), flush, iters=6), 1)
            gemm.configure("auto", 0)
            row["fwd_sweep_us"] = sw
        if stride == 1:
            dx = torch.empty_like(x)
            lib1 = conv.nat.cuda()
            row["dgrad_us"] = round(_median_us(lambda: lib1.gc_cuda_conv_dgrad(
                dy.data_ptr(), w.data_ptr(), dx.data_ptr(), n, hw, hw, cin, cout, r, pad, 0, conv._err(x.device), conv.nat.stream_ptr()), flush), 1)
        elif conv.nat.cuda().gc_cuda_conv_dgrad_s2_supported(n, hw, hw, cin, cout, r, pad):
            dx = torch.empty_like(x)
            lib2 = conv.nat.cuda()
            row["dgrad_us"] = round(_median_us(lambda: lib2.gc_cuda_conv_dgrad_s2(
                dy.data_ptr(), w.data_ptr(), dx.data_ptr(), n, hw, hw, cin, cout, r, pad, conv._err(x.device), conv.nat.stream_ptr()), flush), 1)
        row["dgrad_cudnn_us"] = round(_median_us(lambda: torch.ops.aten.convolution_backward(
            dy, x, w, None, [stride, stride], [pad, pad], [1, 1], False, [0, 0], 1, [True, False, False]), flush), 1)
        row["wgrad_us"] = round(_median_us(lambda: conv.conv_wgrad(dy, x, r, stride, pad), flush), 1)
        row["wgrad_cudnn_us"] = round(_median_us(lambda: torch.ops.aten.convolution_backward(
            dy, x, w, None, [stride, stride], [pad, pad], [1, 1], False, [0, 0], 1, [False, True, False]), flush), 1)
        print(json.dumps(row), flush=True)
    # the 3-channel stem: gather + K = 32 GEMM against cuDNN
    x = torch.randn(n, 3, 32, 32, device="cuda").contiguous(memory_format=cl)
    w = torch.randn(64, 3, 3, 3, device="cuda").contiguous(memory_format=cl)
    a = torch.empty(n * 1024, conv.STEM_K, device="cuda")
    wpad = torch.empty(64, conv.STEM_K, device="cuda")
    out = torch.empty(n * 1024, 64, device="cuda")
    parts = torch.empty(gemm.m_tiles(n * 1024), 2, 64, device="cuda")
    lib = conv.nat.cuda()

    def stem():
        lib.gc_cuda_im2col_small(x.data_ptr(), a.data_ptr(), n, 32, 32, 3, 3, 1, conv.STEM_K, w.data_ptr(), wpad.data_ptr(), 64,
                                 conv.nat.stream_ptr())
        gemm.gemm_tf32(a, wpad, out=out, col_partials=parts)

    dy = torch.randn(n, 64, 32, 32, device="cuda").contiguous(memory_format=cl)
    dy2d = dy.permute(0, 2, 3, 1).reshape(n * 1024, 64)
    print(json.dumps({"stem": "3->64 3x3", "fwd_us": round(_median_us(stem, flush), 1),
                      "fwd_cudnn_us": round(_median_us(lambda: F.conv2d(x, w, None, 1, 1), flush), 1),
                      "wgrad_us": round(_median_us(lambda: gemm.gemm_tn_tf32(dy2d, a), flush), 1),
                      "wgrad_cudnn_us": round(_median_us(lambda: torch.ops.aten.convolution_backward(
                          dy, x, w, None, [1, 1], [1, 1], [1, 1], False, [0, 0], 1, [False, True, False]), flush), 1)}))
    gemm.check()


if __name__ == "__main__":
    main()
