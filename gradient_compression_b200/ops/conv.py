"""1x1 convolution + batch norm (+ residual) (+ ReLU) with the convolution on the tcgen05 GEMMs.

``conv_bn_act(conv, bn, x, residual=None, relu=True)`` is ``relu(bn(conv(x)) + residual)``.  For a 1x1,
stride-1, ungrouped convolution on channels-last fp32 CUDA tensors the convolution is the GEMM
``[N*H*W, Cin] x [Cout, Cin]^T`` (``ops.gemm_tf32``: TMA + tcgen05.mma kind::tf32 + TMEM), whose epilogue also
emits the per-channel sums the batch norm needs -- the normalisation statistics are fused into the producing
kernel, so the activation is written once and read once (by the apply pass) instead of written, read for the
statistics and read again.  Backward: fused BN backward kernels; input gradient ``dY x W`` on the same GEMM
(reading transposed weights that one batched kernel refreshes after every optimiser step, and, in identity
blocks, adding its result onto the skip connection's gradient: ``GradLink``); weight gradient ``dY^T X`` on the
split-K GEMM with MN-major operands (``ops.gemm_tn_tf32``).  Every other convolution (3x3, strided, grouped,
fewer than ``MIN_ROWS`` positions) falls back to ``bn_act(bn, conv(x))`` with cuDNN's convolution.

The reference builds the same layers from ``nn.Conv2d`` + ``nn.BatchNorm2d`` + ``F.relu`` module calls
(models/resnet.py:45-76 of the reference).
"""
from __future__ import annotations

import os
import weakref

import torch

from . import _native as nat
from . import gemm
from .bn import _cl, _scratch_for, bn_act, count_batch, own_grad, take_owned_grad

# On by default.  Measured on the CIFAR ResNet-50 step (batch 128, one B200, three back-to-back pairs of runs): 8.04 /
# 8.28 / 8.26 ms with this path against 8.34 / 8.37 / 8.40 ms with cuDNN convolutions everywhere.  GCB200_TC_CONV=0 (or
# ``ENABLED = False``) keeps every convolution on cuDNN.
ENABLED = os.environ.get("GCB200_TC_CONV", "1") == "1"


# GradLink (accumulating input-gradient GEMMs of identity blocks) on / off, for measurements.
LINK_ENABLED = os.environ.get("GCB200_GRAD_LINK", "1") == "1"

# Weight gradients of these convolutions on the split-K tcgen05 GEMM (off: cuDNN).
WGRAD_ENABLED = os.environ.get("GCB200_TC_WGRAD", "1") == "1"

# Below this many output positions (N*H*W) cuDNN's kernels win by more than the fused statistics return.
MIN_ROWS = int(os.environ.get("GCB200_TC_CONV_MIN_ROWS", "4096"))


class _TransposedWeights:
    """[Cin, Cout] copies of the 1x1 convolution weights: the K-major operand of the input-gradient GEMM.

    A copy is valid while the weight's version counter and storage are the ones it was made from; the backward of
    a layer redoes a stale copy on the spot.  Kernels that write parameters through raw pointers do not move
    version counters, so ``ops.sgd_step`` marks every copy stale, and ``FlatArena.sgd_step`` -- which knows the
    parameter list -- then re-transposes all of its registered weights in ONE launch (``refresh``), which is also
    what a captured step graph replays."""

    def __init__(self):
        self.entries = {}          # id(weight) -> [weakref, wt, version, data_ptr]

    def get(self, w):
        e = self.entries.get(id(w))
        if e is None or e[0]() is not w or e[3] != w.data_ptr() or e[1].device != w.device:
            e = [weakref.ref(w), torch.empty(w.shape[1], w.shape[0], dtype=torch.float32, device=w.device), -1, w.data_ptr()]
            self.entries[id(w)] = e
            if len(self.entries) % 64 == 0:
                self.entries = {k: v for k, v in self.entries.items() if v[0]() is not None}
        if e[2] != w._version:
            e[1].copy_(w.detach().reshape(w.shape[0], w.shape[1]).t())
            e[2] = w._version
        return e[1]

    def invalidate(self):
        for e in self.entries.values():
            e[2] = -1

    def refresh(self, owner, params):
        """One launch for every registered weight among ``params``; the pointer table and the buffers it names are
        kept on ``owner`` so that they live as long as a graph that replays the launch."""
        mine = [e for e in (self.entries.get(id(p)) for p in params) if e is not None and e[0]() is not None and e[0]().is_cuda]
        if not mine:
            return
        key = tuple((e[0]().data_ptr(), e[1].data_ptr()) for e in mine)
        state = getattr(owner, "_transposed_weight_table", None)
        if state is None or state[0] != key:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("the table of transposed 1x1 weights changed inside a CUDA graph capture: run one "
                                   "eager step (forward, backward, optimiser) before capturing")
            rows, tiles = [], 0
            for e in mine:
                w = e[0]()
                rows.append([w.data_ptr(), e[1].data_ptr(), w.shape[0], w.shape[1], tiles])
                tiles += ((w.shape[0] + 31) // 32) * ((w.shape[1] + 31) // 32)
            state = (key, torch.tensor(rows, dtype=torch.int64).to(mine[0][1].device), tiles, [e[1] for e in mine])
            owner._transposed_weight_table = state
        _, table, tiles, _ = state
        with torch.cuda.device(table.device):
            nat.check(nat.cuda().gc_cuda_batched_transpose(table.data_ptr(), table.shape[0], tiles, nat.stream_ptr()),
                      "batched_transpose")
        for e in mine:
            e[2] = e[0]()._version


_transposed = _TransposedWeights()


def weights_written_raw():
    """Called by kernels that rewrite parameters through raw pointers (version counters do not move)."""
    _transposed.invalidate()


def refresh_transposed(owner, params):
    """Called by the owner of a parameter list after it rewrote them: one batched re-transpose."""
    _transposed.refresh(owner, params)


def _as_2d(t):
    n, c, h, w = t.shape
    return t.permute(0, 2, 3, 1).reshape(n * h * w, c)


class GradLink:
    """Joins the two gradients that reach the input of a residual block: the identity branch's and the first
    convolution's.  When that convolution runs on the GEMM, its input-gradient GEMM adds its product straight onto the
    identity branch's gradient (``accumulate=True``: TMA reduce stores), instead of autograd writing both and summing
    them in a third pass.  Usage, inside a block's ``forward``::

        link = GradLink()
        y = conv_bn_act(conv1, bn1, x, link=link)
        ...
        out = conv_bn_act(conv3, bn3, y, residual=link.residual(x))

    ``link.residual(x)`` must be called after the convolution (autograd runs later-created nodes first, and the
    identity gradient has to be there when the convolution's backward runs); either order stays correct, only the
    saving is lost."""

    def __init__(self):
        self.armed = False          # the convolution took the GEMM path and will look for a stashed gradient
        self.conv_done = False      # its backward already ran (without finding one)
        self.stash, self.stash_owned = None, False

    def residual(self, x):
        if not (self.armed and torch.is_grad_enabled() and x.requires_grad):
            return x
        return _StashGrad.apply(x, self)


class _StashGrad(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, link):
        ctx.link = link
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        link = ctx.link
        if link.conv_done:              # the convolution's backward came first: ordinary accumulation by autograd
            return g, None
        link.stash, link.stash_owned = g, take_owned_grad(g)
        return None, None


class _Conv1x1BNAct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, cbias, gamma, beta, residual, running_mean, running_var, training, momentum, eps, relu, link):
        x = _cl(x)
        ctx.link = link
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
        dres = own_grad(torch.empty_like(yconv)) if (ctx.has_res and ctx.needs_input_grad[5]) else None
        with torch.cuda.device(x.device):
            nat.check(lib.gc_cuda_bn_bwd_reduce(dy.data_ptr(), yconv.data_ptr(), nat.ptr(out), m, cout, stats.data_ptr(),
                                                gamma.data_ptr(), beta.data_ptr(), int(ctx.relu),
                                                _scratch_for(x.device, cout).data_ptr(), sums.data_ptr(), st()), "bn_bwd_reduce")
            nat.count_launch()
            nat.check(lib.gc_cuda_bn_bwd_apply(dy.data_ptr(), yconv.data_ptr(), nat.ptr(out), m, cout, stats.data_ptr(),
                                               gamma.data_ptr(), beta.data_ptr(), sums.data_ptr(), int(ctx.relu),
                                               dconv.data_ptr(), nat.ptr(dres), st()), "bn_bwd_apply")
            dx = None
            link = ctx.link
            if ctx.needs_input_grad[0]:
                wt = _transposed.get(w)                                     # [Cin, Cout]: K-major for dX = dY x W
                acc = None
                if link is not None and link.stash is not None:
                    acc, link.stash = link.stash, None
                    if not (link.stash_owned and acc.shape == x.shape and acc.dtype == torch.float32
                            and acc.is_contiguous(memory_format=torch.channels_last)):
                        acc = acc.contiguous(memory_format=torch.channels_last).clone()     # not ours to write into
                if acc is not None and gemm.can_accumulate(_as_2d(acc)):
                    dx = acc                                                # dX = identity-branch gradient + dY x W, added in L2
                    gemm.gemm_tf32(_as_2d(dconv), wt, out=_as_2d(dx), accumulate=True)
                else:
                    dx = torch.empty_like(x)
                    gemm.gemm_tf32(_as_2d(dconv), wt, out=_as_2d(dx))
                    if acc is not None:
                        dx += acc
            if link is not None:
                link.conv_done = True
            dw = None
            if ctx.needs_input_grad[1]:
                if WGRAD_ENABLED and cout % 32 == 0 and cin % 32 == 0:
                    # dW[Cout, Cin] = dY^T X over all positions: split-K GEMM with MN-major tcgen05 operands
                    dw2d = gemm.gemm_tn_tf32(_as_2d(dconv), _as_2d(x))
                    dw = dw2d.view(cout, cin, 1, 1).contiguous(memory_format=torch.channels_last)
                else:
                    dw = torch.ops.aten.convolution_backward(dconv, x, w, None, [1, 1], [0, 0], [1, 1], False, [0, 0], 1,
                                                             [False, True, False])[1]
            dcb = dconv.sum((0, 2, 3)) if ctx.has_cbias else None
        return dx, dw, dcb, sums[cout:], sums[:cout], dres, None, None, None, None, None, None, None


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
    if cin % 4 or conv.out_channels % 4 or n * h * w < MIN_ROWS:
        return False
    return bool(nat.cuda().gc_cuda_bn_supported(n * h * w, conv.out_channels))


def conv_bn_act(conv, bn, x, residual=None, relu=True, link=None):
    if not _fusable(conv, bn, x):
        return bn_act(bn, conv(x), residual=residual, relu=relu)
    if link is not None:
        link.armed = LINK_ENABLED and torch.is_grad_enabled() and x.requires_grad
    training = bn.training or bn.running_mean is None
    momentum = 0.1 if bn.momentum is None else bn.momentum
    if training and bn.track_running_stats and bn.num_batches_tracked is not None:
        count_batch(bn)
    rm = bn.running_mean if bn.track_running_stats else None
    rv = bn.running_var if bn.track_running_stats else None
    return _Conv1x1BNAct.apply(x, conv.weight, conv.bias, bn.weight, bn.bias, residual, rm, rv, training, momentum,
                               bn.eps, relu, link if (link is not None and link.armed) else None)
