"""1x1 convolution + batch norm (+ residual) (+ ReLU) with the convolution on the tcgen05 GEMM.

``conv_bn_act(conv, bn, x, residual=None, relu=True)`` is ``relu(bn(conv(x)) + residual)``.  For a 1x1,
stride-1, ungrouped convolution on channels-last fp32 CUDA tensors the convolution is the GEMM
``[N*H*W, Cin] x [Cout, Cin]^T`` (``ops.gemm_tf32``: TMA + tcgen05.mma kind::tf32 + TMEM), whose epilogue also
emits the per-channel sums the batch norm needs -- the normalisation statistics are fused into the producing
kernel, so the activation is written once and read once (by the apply pass) instead of written, read for the
statistics and read again.  Backward: fused BN backward kernels, input gradient on the same GEMM
(``dY x W``), weight gradient through cuDNN.  Every other convolution falls back to ``bn_act(bn, conv(x))``.
"""
from __future__ import annotations

import os

import torch

from . import _native as nat
from . import gemm
from .bn import _cl, _scratch_for, bn_act, kernel_path_ok

# Off by default: on the CIFAR ResNet-50 step the GEMM is still 15-25 % behind cuDNN's own sm_100 kernels on these
# shapes, which costs more than the saved statistics pass returns.  GCB200_TC_CONV=1 (or ``ENABLED = True``) turns it on.
ENABLED = os.environ.get("GCB200_TC_CONV", "0") == "1"


def _as_2d(t):
    n, c, h, w = t.shape
    return t.permute(0, 2, 3, 1).reshape(n * h * w, c)


class _Conv1x1BNAct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, cbias, gamma, beta, residual, running_mean, running_var, training, momentum, eps, relu):
        x = _cl(x)
        n, cin, h, wd = x.shape
        cout = w.shape[0]
        m = n * h * wd
        lib, st = nat.cuda(), nat.stream_ptr
        yconv = torch.empty((n, cout, h, wd), dtype=torch.float32, device=x.device, memory_format=torch.channels_last)
        stats = torch.empty(2 * cout, dtype=torch.float32, device=x.device)
        w2d = w.reshape(cout, cin)
        with torch.cuda.device(x.device):
            if training:
                tiles = gemm.m_tiles(m)
                partials = torch.empty(tiles, 2, cout, dtype=torch.float32, device=x.device)
                gemm.gemm_tf32(_as_2d(x), w2d, bias=cbias, out=_as_2d(yconv), col_partials=partials)
                nat.check(lib.gc_cuda_bn_finalize_partials(partials.data_ptr(), tiles, m, cout, stats.data_ptr(),
                                                           nat.ptr(running_mean), nat.ptr(running_var), float(momentum),
                                                           float(eps), st()), "bn_finalize_partials")
            else:
                gemm.gemm_tf32(_as_2d(x), w2d, bias=cbias, out=_as_2d(yconv))
                stats[:cout] = running_mean
                stats[cout:] = torch.rsqrt(running_var + eps)
            res = _cl(residual) if residual is not None else None
            out = torch.empty_like(yconv)
            nat.check(lib.gc_cuda_bn_apply(yconv.data_ptr(), m, cout, stats.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                                           nat.ptr(res), int(relu), out.data_ptr(), st()), "bn_apply")
        ctx.relu, ctx.has_res, ctx.has_cbias = bool(relu), residual is not None, cbias is not None
        ctx.save_for_backward(x, w, yconv, gamma, beta, stats, out if (residual is not None and relu) else None)
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w, yconv, gamma, beta, stats, out = ctx.saved_tensors
        dy = _cl(dy)
        n, cout, h, wd = yconv.shape
        cin = x.shape[1]
        m = n * h * wd
        lib, st = nat.cuda(), nat.stream_ptr
        sums = torch.empty(2 * cout, dtype=torch.float32, device=x.device)
        dconv = torch.empty_like(yconv)
        dres = torch.empty_like(yconv) if (ctx.has_res and ctx.needs_input_grad[5]) else None
        with torch.cuda.device(x.device):
            nat.check(lib.gc_cuda_bn_bwd_reduce(dy.data_ptr(), yconv.data_ptr(), nat.ptr(out), m, cout, stats.data_ptr(),
                                                gamma.data_ptr(), beta.data_ptr(), int(ctx.relu),
                                                _scratch_for(x.device, cout).data_ptr(), sums.data_ptr(), st()), "bn_bwd_reduce")
            nat.count_launch()
            nat.check(lib.gc_cuda_bn_bwd_apply(dy.data_ptr(), yconv.data_ptr(), nat.ptr(out), m, cout, stats.data_ptr(),
                                               gamma.data_ptr(), beta.data_ptr(), sums.data_ptr(), int(ctx.relu),
                                               dconv.data_ptr(), nat.ptr(dres), st()), "bn_bwd_apply")
            dx = None
            if ctx.needs_input_grad[0]:
                dx = torch.empty_like(x)
                wt = w.reshape(cout, cin).t().contiguous()                  # [Cin, Cout]: K-major for dX = dY x W
                gemm.gemm_tf32(_as_2d(dconv), wt, out=_as_2d(dx))
            dw = torch.ops.aten.convolution_backward(dconv, x, w, None, [1, 1], [0, 0], [1, 1], False, [0, 0], 1,
                                                     [False, True, False])[1]
            dcb = dconv.sum((0, 2, 3)) if ctx.has_cbias else None
        return dx, dw, dcb, sums[cout:], sums[:cout], dres, None, None, None, None, None, None


def _fusable(conv, bn, x):
    if not (ENABLED and x.is_cuda and x.dtype == torch.float32 and x.dim() == 4 and isinstance(conv, torch.nn.Conv2d)):
        return False
    if not torch.backends.cudnn.allow_tf32:       # the GEMM multiplies in TF32: only where TF32 convolutions are allowed
        return False
    if conv.kernel_size != (1, 1) or conv.stride != (1, 1) or conv.padding != (0, 0) or conv.groups != 1 or conv.dilation != (1, 1):
        return False
    if not bn.affine or (not (bn.training or bn.running_mean is None) and torch.is_grad_enabled() and
                         (x.requires_grad or conv.weight.requires_grad)):
        return False
    n, cin, h, w = x.shape
    if cin % 4 or conv.out_channels % 4:
        return False
    return bool(nat.cuda().gc_cuda_bn_supported(n * h * w, conv.out_channels))


def conv_bn_act(conv, bn, x, residual=None, relu=True):
    if not _fusable(conv, bn, x):
        return bn_act(bn, conv(x), residual=residual, relu=relu)
    training = bn.training or bn.running_mean is None
    momentum = 0.1 if bn.momentum is None else bn.momentum
    if training and bn.track_running_stats and bn.num_batches_tracked is not None:
        bn.num_batches_tracked.add_(1)
    rm = bn.running_mean if bn.track_running_stats else None
    rv = bn.running_var if bn.track_running_stats else None
    return _Conv1x1BNAct.apply(x, conv.weight, conv.bias, bn.weight, bn.bias, residual, rm, rv, training, momentum,
                               bn.eps, relu)
