"""Convolution + batch norm (+ residual) (+ ReLU) with the convolution on the tcgen05 kernels.

``conv_bn_act(conv, bn, x, residual=None, relu=True)`` is ``relu(bn(conv(x)) + residual)`` for an ungrouped
``nn.Conv2d`` on channels-last fp32 CUDA tensors.  Three forward paths, all TMA + tcgen05.mma kind::tf32 + TMEM:

* ``gemm``  1x1, stride 1: the GEMM ``[N*H*W, Cin] x [Cout, Cin]^T`` (``ops.gemm_tf32``);
* ``conv``  R x R at stride 1 or 2 with Cin a multiple of 32 (3x3 layers, strided projection shortcuts): implicit GEMM,
  one shifted 4-D TMA box of the activation per filter tap and 32-channel block, zero fill as padding
  (``csrc/gc_conv_tc.cu``);
* ``stem``  few input channels (the 3-channel first layer): a gather kernel writes rows of 32 floats (27 taps + padding),
  then the GEMM with K = 32.

The epilogue of each emits the per-channel sums the batch norm needs, so the activation is written once and read once
(by the apply pass; ``pool=True`` folds a following 2x2 max-pool into that pass and its backward).  Backward: fused BN
backward kernels; input gradient on the same kernel run on dY, reading the forward filter in place as an MN-major operand
whose taps the kernel addresses rotated by 180 degrees (for shapes that path does not cover: a rotated / transposed copy
that one batched kernel refreshes after every optimiser step); in residual blocks the product is added straight onto the
skip connection's or projection shortcut's gradient (``GradLink``); weight gradient ``dY^T X`` on the split-K kernel with
MN-major operands, per filter tap from shifted boxes, added straight into the owner's flat gradient buffer.  The input
gradient of a stride-2 convolution is four launches of the forward kernel, one per parity class of input pixels, each
writing its pixels through a strided 4-D store map.  Grouped convolutions and shapes the tilings exclude use cuDNN
through ``bn_act(bn, conv(x))`` or ``aten.convolution_backward``.

The reference builds the same layers from ``nn.Conv2d`` + ``nn.BatchNorm2d`` + ``F.relu`` module calls
(models/resnet.py:45-76, models/vgg.py:96-110 of the reference).
"""
from __future__ import annotations

import os
import weakref

import torch

from . import _native as nat
from . import gemm
from .bn import _cl, _fin_ptr, _scratch_for, bn_act, count_batch, own_grad, take_owned_grad

# GCB200_TC_CONV=0 (or ``ENABLED = False``) keeps every convolution on cuDNN.
ENABLED = os.environ.get("GCB200_TC_CONV", "1") == "1"

# GradLink (accumulating input-gradient kernels of identity blocks) on / off, for measurements.
LINK_ENABLED = os.environ.get("GCB200_GRAD_LINK", "1") == "1"

# Weight gradients of these convolutions on the split-K tcgen05 kernel (off: cuDNN).
WGRAD_ENABLED = os.environ.get("GCB200_TC_WGRAD", "1") == "1"

# Convolutions with fewer output positions (N*Ho*Wo) than this stay on cuDNN.
MIN_ROWS = int(os.environ.get("GCB200_TC_CONV_MIN_ROWS", "0"))

# Batch-norm statistics finished inside the producing kernel (off: per-tile partial sums + a separate finalize kernel).
FUSED_FINALIZE = os.environ.get("GCB200_BN_FUSED_FINALIZE", "0") == "1"

# Which paths may be taken (for measurements): any subset of "gemm", "conv", "stem", "dgrad_s2" (own input gradient of
# stride-2 convolutions; without it cuDNN computes those).
# activations of at most 2048 rows (the 4x4 / 2x2 stages at batch 128): BN statistics + apply, and BN backward, in one launch each
SMALL_BN = os.environ.get("GCB200_BN_SMALL", "1") == "1"
# ... and at most this many values: measured on one B200, VGG-16 89.9 k img/s without, 90.7 k with a limit of 1 Mi, 91.1 k with
# 256 Ki; ResNet-50 17.22 k / 17.19 k / 17.22 k (its 2048-row x 2048-channel maps are better streamed row by row)
SMALL_BN_ELEMENTS = int(os.environ.get("GCB200_BN_SMALL_ELEMENTS", str(1 << 18)))
# stride-1 input gradients read the forward filter in place (MN-major B operand) instead of a rotated / transposed copy
DGRAD_IN_PLACE = os.environ.get("GCB200_DGRAD_IN_PLACE", "1") == "1"
PATHS = set(os.environ.get("GCB200_TC_CONV_PATHS", "gemm,conv,stem,dgrad_s2").split(","))


def _taps(w):
    return w.shape[2] * w.shape[3]


def _s2_classes(r, pad):
    """Parity classes (ph, pw) of the input pixels of a stride-2 convolution, in the order the kernel walks them, each with
    the filter taps that reach it: ``(taps_h, taps_w)`` where tap d of an axis is filter index ``par + pad - 2 d``."""
    def axis(par):
        return [par + pad - 2 * d for d in range(r + pad + 1) if 0 <= par + pad - 2 * d < r]

    return [(ph, pw, axis(ph), axis(pw)) for ph in (0, 1) for pw in (0, 1)]


class _DgradWeights:
    """The filter as the input-gradient kernels read it.

    Stride 1: ``[Cin, taps * Cout]`` with tap ``t`` holding the transpose of the forward filter's tap ``taps - 1 - t``
    (rotation by 180 degrees, channel axes swapped); for a 1x1 filter that is the plain transpose ``[Cin, Cout]``.
    Stride 2: one such matrix per parity class of input pixels, back to back, class ``(ph, pw)`` holding
    ``[Cin][fr][fs][Cout] = w[Cout][ph + pad - 2 fr][pw + pad - 2 fs][Cin]`` (``csrc/gc_conv_tc.cu``).

    A copy is valid while the weight's version counter and storage are the ones it was made from; the backward of
    a layer redoes a stale copy on the spot.  Kernels that write parameters through raw pointers do not move
    version counters, so ``ops.sgd_step`` marks every copy stale, and ``FlatArena.sgd_step`` -- which knows the
    parameter list -- then redoes all of its registered weights in ONE launch (``refresh``), which is also
    what a captured step graph replays."""

    def __init__(self):
        self.entries = {}          # (id(weight), stride) -> [weakref, wd, version, data_ptr, stride, pad]

    def get(self, w, stride=1, pad=None):
        key = (id(w), stride)
        e = self.entries.get(key)
        if e is None or e[0]() is not w or e[3] != w.data_ptr() or e[1].device != w.device:
            shape = (w.shape[1], _taps(w) * w.shape[0]) if stride == 1 else (_taps(w) * w.shape[0] * w.shape[1],)
            e = [weakref.ref(w), torch.empty(shape, dtype=torch.float32, device=w.device), -1, w.data_ptr(), stride, pad]
            self.entries[key] = e
            if len(self.entries) % 64 == 0:
                self.entries = {k: v for k, v in self.entries.items() if v[0]() is not None}
        if e[2] != w._version:
            cout, cin, r, s = w.shape
            if stride == 1:
                e[1].view(cin, r, s, cout).copy_(w.detach().flip(2, 3).permute(1, 2, 3, 0))
            else:
                off = 0
                for _, _, th, tw in _s2_classes(r, pad):
                    if th and tw:
                        n = cin * len(th) * len(tw) * cout
                        dst = e[1][off: off + n].view(cin, len(th), len(tw), cout)
                        for a, fr in enumerate(th):              # tap by tap: plain strided copies, fine inside a graph capture
                            for b, fs in enumerate(tw):
                                dst[:, a, b, :].copy_(w.detach()[:, :, fr, fs].t())
                        off += n
            e[2] = w._version
        return e[1]

    def invalidate(self, lo=None, hi=None):
        """Mark stale the copies of the weights stored in the address range [lo, hi) (all of them without a range)."""
        for e in self.entries.values():
            if lo is None or lo <= e[3] < hi:
                e[2] = -1

    @staticmethod
    def _rows(e, tiles):
        """Table rows {src, dst, rows, cols, first tile, src pitch, dst pitch} of the batched transpose for one entry."""
        w = e[0]()
        cout, cin, r, taps = w.shape[0], w.shape[1], w.shape[2], _taps(w)
        per = ((cout + 31) // 32) * ((cin + 31) // 32)
        rows = []
        if e[4] == 1:
            for t in range(taps):       # tap t of [Cout][taps][Cin] -> tap (taps - 1 - t) of [Cin][taps][Cout]
                rows.append([w.data_ptr() + 4 * t * cin, e[1].data_ptr() + 4 * (taps - 1 - t) * cout, cout, cin, tiles,
                             taps * cin, taps * cout])
                tiles += per
        else:
            off = 0
            for _, _, th, tw in _s2_classes(r, e[5]):
                nt = len(th) * len(tw)
                for a, fr in enumerate(th):
                    for b, fs in enumerate(tw):      # filter tap (fr, fs) -> tap (a, b) of this class's [Cin][th][tw][Cout]
                        rows.append([w.data_ptr() + 4 * (fr * w.shape[3] + fs) * cin, e[1].data_ptr() + 4 * (off + (a * len(tw) + b) * cout),
                                     cout, cin, tiles, taps * cin, nt * cout])
                        tiles += per
                off += cin * nt * cout
        return rows, tiles

    def refresh(self, owner, params):
        """One launch for every registered weight among ``params``; the pointer table and the buffers it names are
        kept on ``owner`` so that they live as long as a graph that replays the launch."""
        mine = [e for p in params for e in (self.entries.get((id(p), 1)), self.entries.get((id(p), 2)))
                if e is not None and e[0]() is not None and e[0]().is_cuda]
        if not mine:
            return
        key = tuple((e[0]().data_ptr(), e[1].data_ptr()) for e in mine)
        state = getattr(owner, "_dgrad_weight_table", None)
        if state is None or state[0] != key:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("the table of input-gradient filters changed inside a CUDA graph capture: run one "
                                   "eager step (forward, backward, optimiser) before capturing")
            rows, tiles = [], 0
            for e in mine:
                more, tiles = self._rows(e, tiles)
                rows += more
            state = (key, torch.tensor(rows, dtype=torch.int64).to(mine[0][1].device), tiles, [e[1] for e in mine])
            owner._dgrad_weight_table = state
        _, table, tiles, _ = state
        with torch.cuda.device(table.device):
            nat.check(nat.cuda().gc_cuda_batched_transpose(table.data_ptr(), table.shape[0], tiles, nat.stream_ptr()),
                      "batched_transpose")
        for e in mine:
            e[2] = e[0]()._version


_dgrad_weights = _DgradWeights()


def weights_written_raw(lo=None, hi=None):
    """Called by kernels that rewrite parameters through raw pointers (version counters do not move); ``[lo, hi)``: the
    address range they wrote, so that another model's copies stay valid."""
    _dgrad_weights.invalidate(lo, hi)


def refresh_transposed(owner, params):
    """Called by the owner of a parameter list after it rewrote them: one batched kernel redoes every registered
    input-gradient filter."""
    _dgrad_weights.refresh(owner, params)


# Gradient slots: where the weight-gradient kernels add their result when the weight's owner (a ``FlatArena``) has offered
# the weight's place in its flat gradient buffer.  id(weight) -> (weakref(weight), 2-D view [Cout, R*S*Cin] of the slot).
_grad_slots = {}


def offer_grad_slots(params, slots):
    """``slots[i]``: the contiguous gradient storage of the 4-D weight ``params[i]`` in its memory order (None: no offer).
    The split-K weight-gradient kernels then add dW straight into the slot (it must hold the value to add to: zeros at the
    start of a step) and the layer's autograd node returns no weight gradient, instead of allocating and zeroing a
    tensor per layer that is copied into the flat buffer afterwards."""
    for p, slot in zip(params, slots):
        if slot is None:
            _grad_slots.pop(id(p), None)
        elif p.dim() == 4:
            _grad_slots[id(p)] = (weakref.ref(p), slot.reshape(p.shape[0], -1))


def withdraw_grad_slots(params):
    for p in params:
        _grad_slots.pop(id(p), None)


def _slot_of(w):
    e = _grad_slots.get(id(w))
    if e is None or e[0]() is not w or e[1].device != w.device:
        return None
    return e[1]


def _filter_in_place_ok(w):
    """The filter can be read by the input-gradient kernels where it lies: [Cout][R][S][Cin] memory order, 16-byte aligned."""
    return (w.data_ptr() % 16 == 0 and (w.shape[2] * w.shape[3] == 1 and w.is_contiguous() or
                                        w.is_contiguous(memory_format=torch.channels_last)))


def _as_2d(t):
    n, c, h, w = t.shape
    return t.permute(0, 2, 3, 1).reshape(n * h * w, c)


def _w2d(w):
    """The channels-last filter ``[Cout][R][S][Cin]`` as the matrix ``[Cout, R*S*Cin]`` (no copy)."""
    return w.permute(0, 2, 3, 1).reshape(w.shape[0], -1)


class GradLink:
    """Joins the two gradients that reach the input of a residual block: the identity branch's and the first
    convolution's.  When that convolution runs on the tensor-core kernels, its input-gradient kernel adds its product
    straight onto the identity branch's gradient (``accumulate=True``: TMA reduce stores), instead of autograd writing
    both and summing them in a third pass.  Usage, inside a block's ``forward``::

        link = GradLink()
        y = conv_bn_act(conv1, bn1, x, link=link)
        ...
        out = conv_bn_act(conv3, bn3, y, residual=link.residual(x))

    ``link.residual(x)`` must be called after the convolution (autograd runs later-created nodes first, and the
    identity gradient has to be there when the convolution's backward runs); either order stays correct, only the
    saving is lost."""

    def __init__(self):
        self.armed = False          # the convolution took a tensor-core path and will look for a stashed gradient
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


def _err(device):
    return gemm._error_flag(device).data_ptr()


def conv_forward(x, w, bias=None, stride=1, pad=1, col_partials=None, out=None, accumulate=False, bn_fin=None):
    """``conv2d(x, w, bias, stride, pad)`` of a channels-last activation on the implicit-GEMM kernel; ``w`` is the
    filter in channels-last memory order ``(Cout, Cin, R, R)`` or already a matrix ``[Cout, R*R*Cin]`` together with
    ``x`` of ``Cin`` channels.  ``col_partials`` ([tiles, 2, Cout]) receives per-tile column sums / sums of squares; ``bn_fin`` (``gemm.bn_fin_args``)
    makes the kernel finish the batch-norm statistics itself instead."""
    n, cin, h, wd = x.shape
    w2 = _w2d(w) if w.dim() == 4 else w
    cout = w2.shape[0]
    r = int(round((w2.shape[1] // cin) ** 0.5))
    ho, wo = (h + 2 * pad - r) // stride + 1, (wd + 2 * pad - r) // stride + 1
    if out is None:
        assert not accumulate
        out = torch.empty((n, cout, ho, wo), dtype=torch.float32, device=x.device, memory_format=torch.channels_last)
    with torch.cuda.device(x.device):
        nat.check(nat.cuda().gc_cuda_conv_fwd(x.data_ptr(), w2.data_ptr(), out.data_ptr(), nat.ptr(bias), n, h, wd, cin, cout, r,
                                              stride, pad, int(bool(accumulate)), nat.ptr(col_partials), _err(x.device),
                                              nat.stream_ptr(), bn_fin[0] if bn_fin is not None else None), "conv_fwd")
    return out


def conv_wgrad(dy, x, r, stride, pad, out=None):
    """Weight gradient ``[Cout, R*R*Cin]`` (channels-last filter order) of ``conv2d(x, w, stride, pad)`` given the
    channels-last output gradient ``dy``; added onto ``out`` when given."""
    n, cin, h, wd = x.shape
    cout = dy.shape[1]
    dw = out if out is not None else torch.zeros(cout, r * r * cin, dtype=torch.float32, device=x.device)
    with torch.cuda.device(x.device):
        nat.check(nat.cuda().gc_cuda_conv_wgrad(dy.data_ptr(), x.data_ptr(), dw.data_ptr(), n, h, wd, cin, cout, r, stride, pad,
                                                _err(x.device), nat.stream_ptr()), "conv_wgrad")
    return dw


_SPLIT_PLAN = {}


def _split_forward(lib, mode, n, h, wd, cin, cout, r, stride, pad, m):
    """True when the forward kernel of this layer should run as a split contraction and leave the batch statistics to a
    separate pass (the kernels' own cost model decides; cached per shape)."""
    key = (mode, n, h, wd, cin, cout, r, stride, pad)
    hit = _SPLIT_PLAN.get(key)
    if hit is None:
        if mode == "gemm":
            hit = lib.gc_cuda_gemm_tf32_splits(m, cout, cin) > 1
        elif mode == "conv":
            hit = lib.gc_cuda_conv_fwd_splits(n, h, wd, cin, cout, r, stride, pad) > 1
        else:
            hit = False
        _SPLIT_PLAN[key] = hit
    return hit


STEM_K = 32      # row length of the gathered stem operand: R*R*Cin taps padded to one 128-byte row


class _ConvBNAct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, cbias, gamma, beta, residual, running_mean, running_var, training, momentum, eps, relu, link,
                mode, stride, pad, donate=None, pool=False):
        x = _cl(x)
        ctx.link, ctx.mode, ctx.stride, ctx.pad, ctx.donate, ctx.pool = link, mode, stride, pad, donate, bool(pool)
        n, cin, h, wd = x.shape
        cout, r = w.shape[0], w.shape[2]
        ho, wo = (h + 2 * pad - r) // stride + 1, (wd + 2 * pad - r) // stride + 1
        m = n * ho * wo
        lib, st = nat.cuda(), nat.stream_ptr
        yconv = torch.empty((n, cout, ho, wo), dtype=torch.float32, device=x.device, memory_format=torch.channels_last)
        stats = torch.empty(2 * cout, dtype=torch.float32, device=x.device)
        gathered = None
        with torch.cuda.device(x.device):
            # training: the kernel that writes yconv also finishes its batch statistics (mean, rstd, running stats)
            fin = partials = None
            if training:
                if FUSED_FINALIZE and cout <= gemm.FIN_MAX_CHANNELS and cout > 16:
                    fin = gemm.bn_fin_args(x.device, stats, running_mean, running_var, momentum, eps)
                elif not _split_forward(lib, mode, n, h, wd, cin, cout, r, stride, pad, m):
                    tiles = gemm.m_tiles(m)
                    partials = torch.empty(tiles, 2, cout, dtype=torch.float32, device=x.device)
            if mode == "gemm":
                gemm.gemm_tf32(_as_2d(x), w.reshape(cout, cin), bias=cbias, out=_as_2d(yconv), col_partials=partials, bn_fin=fin)
            elif mode == "conv":
                conv_forward(x, w, cbias, stride, pad, col_partials=partials, out=yconv, bn_fin=fin)
            else:
                gathered = torch.empty(m, STEM_K, dtype=torch.float32, device=x.device)
                wpad = torch.empty(cout, STEM_K, dtype=torch.float32, device=x.device)
                nat.check(lib.gc_cuda_im2col_small(x.data_ptr(), gathered.data_ptr(), n, h, wd, cin, r, pad, STEM_K,
                                                   w.data_ptr(), wpad.data_ptr(), cout, st()), "im2col_small")
                gemm.gemm_tf32(gathered, wpad, bias=cbias, out=_as_2d(yconv), col_partials=partials, bn_fin=fin)
            res = _cl(residual) if residual is not None else None
            small = (SMALL_BN and training and fin is None and not pool and m * cout <= SMALL_BN_ELEMENTS
                     and lib.gc_cuda_bn_small_supported(m, cout))
            if small:
                # a few hundred kilobytes of activation: statistics (from the convolution's partial sums, or from yconv after a
                # split contraction), running-statistics update and apply in ONE launch instead of two or three
                out = torch.empty_like(yconv)
                nat.check(lib.gc_cuda_bn_small_forward(yconv.data_ptr(), m, cout, nat.ptr(partials),
                                                       partials.shape[0] if partials is not None else 0, gamma.data_ptr(),
                                                       beta.data_ptr(), nat.ptr(res), int(relu), nat.ptr(running_mean),
                                                       nat.ptr(running_var), float(momentum), float(eps), stats.data_ptr(),
                                                       out.data_ptr(), st()), "bn_small_forward")
            else:
                if partials is not None:
                    nat.check(lib.gc_cuda_bn_finalize_partials(partials.data_ptr(), partials.shape[0], m, cout, stats.data_ptr(),
                                                               nat.ptr(running_mean), nat.ptr(running_var), float(momentum),
                                                               float(eps), st()), "bn_finalize_partials")
                elif training and fin is None:
                    # the convolution ran as a split contraction (few output tiles, long filters): its statistics take a pass
                    # of their own over the small output
                    nat.check(lib.gc_cuda_bn_stats(yconv.data_ptr(), m, cout, _scratch_for(x.device, cout).data_ptr(), stats.data_ptr(),
                                                   nat.ptr(running_mean), nat.ptr(running_var), float(momentum), float(eps), st()),
                              "bn_stats")
                    nat.count_launch()
                elif not training:
                    stats[:cout] = running_mean
                    stats[cout:] = torch.rsqrt(running_var + eps)
                if pool:
                    # act = relu(bn(yconv)) is never written: only its 2x2 max-pooled map is
                    assert res is None
                    out = torch.empty((n, cout, ho // 2, wo // 2), dtype=torch.float32, device=x.device, memory_format=torch.channels_last)
                    nat.check(lib.gc_cuda_bn_apply_pool(yconv.data_ptr(), n, ho, wo, cout, stats.data_ptr(), gamma.data_ptr(),
                                                        beta.data_ptr(), int(relu), out.data_ptr(), st()), "bn_apply_pool")
                else:
                    out = torch.empty_like(yconv)
                    nat.check(lib.gc_cuda_bn_apply(yconv.data_ptr(), m, cout, stats.data_ptr(), gamma.data_ptr(), beta.data_ptr(),
                                                   nat.ptr(res), int(relu), out.data_ptr(), st()), "bn_apply")
        ctx.relu, ctx.has_res, ctx.has_cbias = bool(relu), residual is not None, cbias is not None
        ctx.save_for_backward(x, w, yconv, gamma, beta, stats, out if (residual is not None and relu) else None, gathered)
        return out

    @staticmethod
    def backward(ctx, dy):
        x, w, yconv, gamma, beta, stats, out, gathered = ctx.saved_tensors
        dy = _cl(dy)
        mode, stride, pad = ctx.mode, ctx.stride, ctx.pad
        n, cout, ho, wo = yconv.shape
        cin, r = x.shape[1], w.shape[2]
        m = n * ho * wo
        lib, st = nat.cuda(), nat.stream_ptr
        sums = torch.empty(2 * cout, dtype=torch.float32, device=x.device)
        dconv = torch.empty_like(yconv)
        dres = own_grad(torch.empty_like(yconv)) if (ctx.has_res and ctx.needs_input_grad[5]) else None
        with torch.cuda.device(x.device):
            if ctx.pool:
                # dy is the gradient of the pooled map: both kernels find each window's winner again from yconv
                nat.check(lib.gc_cuda_bn_bwd_reduce_pool(dy.data_ptr(), yconv.data_ptr(), n, ho, wo, cout, stats.data_ptr(),
                                                         gamma.data_ptr(), beta.data_ptr(), int(ctx.relu),
                                                         _scratch_for(x.device, cout).data_ptr(), sums.data_ptr(), st()),
                          "bn_bwd_reduce_pool")
                nat.count_launch()
                nat.check(lib.gc_cuda_bn_bwd_apply_pool(dy.data_ptr(), yconv.data_ptr(), n, ho, wo, cout, stats.data_ptr(),
                                                        gamma.data_ptr(), beta.data_ptr(), sums.data_ptr(), int(ctx.relu),
                                                        dconv.data_ptr(), st()), "bn_bwd_apply_pool")
            elif SMALL_BN and m * cout <= SMALL_BN_ELEMENTS and lib.gc_cuda_bn_small_supported(m, cout):
                # small activation: the two gradient sums and the input gradient in one launch (a block owns its channels)
                nat.check(lib.gc_cuda_bn_small_backward(dy.data_ptr(), yconv.data_ptr(), nat.ptr(out), m, cout, stats.data_ptr(),
                                                        gamma.data_ptr(), beta.data_ptr(), int(ctx.relu), sums.data_ptr(),
                                                        dconv.data_ptr(), nat.ptr(dres), st()), "bn_small_backward")
            else:
                nat.check(lib.gc_cuda_bn_bwd_reduce(dy.data_ptr(), yconv.data_ptr(), nat.ptr(out), m, cout, stats.data_ptr(),
                                                    gamma.data_ptr(), beta.data_ptr(), int(ctx.relu),
                                                    _scratch_for(x.device, cout).data_ptr(), sums.data_ptr(), _fin_ptr(x.device, cout), st()), "bn_bwd_reduce")
                nat.count_launch()
                nat.check(lib.gc_cuda_bn_bwd_apply(dy.data_ptr(), yconv.data_ptr(), nat.ptr(out), m, cout, stats.data_ptr(),
                                                   gamma.data_ptr(), beta.data_ptr(), sums.data_ptr(), int(ctx.relu),
                                                   dconv.data_ptr(), nat.ptr(dres), st()), "bn_bwd_apply")
            dx = None
            link = ctx.link
            if ctx.needs_input_grad[0]:
                acc = None
                if link is not None and link.stash is not None:
                    acc, link.stash = link.stash, None
                    if not (link.stash_owned and acc.shape == x.shape and acc.dtype == torch.float32
                            and acc.is_contiguous(memory_format=torch.channels_last)):
                        acc = acc.contiguous(memory_format=torch.channels_last).clone()     # not ours to write into
                h_in, w_in = x.shape[2], x.shape[3]
                in_place = (stride == 1 and mode in ("gemm", "conv") and DGRAD_IN_PLACE and _filter_in_place_ok(w)
                            and lib.gc_cuda_conv_dgrad_supported(n, h_in, w_in, cin, cout, r, pad))
                tc_dgrad = mode == "gemm" or (mode == "conv" and stride == 1 and
                                              lib.gc_cuda_conv_fwd_supported(n, ho, wo, cout, cin, r, 1, r - 1 - pad))
                if in_place:
                    # dX = dY (*) rot(W) with the forward filter read in place as the MN-major operand: no transposed copy
                    accumulate = acc is not None and gemm.can_accumulate(_as_2d(acc))
                    dx = acc if accumulate else torch.empty_like(x)
                    nat.check(lib.gc_cuda_conv_dgrad(dconv.data_ptr(), w.data_ptr(), dx.data_ptr(), n, h_in, w_in, cin, cout, r, pad,
                                                     int(accumulate), _err(x.device), st()), "conv_dgrad")
                    if acc is not None and not accumulate:
                        dx += acc
                elif tc_dgrad:
                    wd_ = _dgrad_weights.get(w)           # [Cin, taps * Cout]: the K-major operand of dX = dY (*) rot(W)
                    accumulate = acc is not None and gemm.can_accumulate(_as_2d(acc))
                    dx = acc if accumulate else torch.empty_like(x)
                    if mode == "gemm":
                        gemm.gemm_tf32(_as_2d(dconv), wd_, out=_as_2d(dx), accumulate=accumulate)
                    else:
                        conv_forward(dconv, wd_, None, 1, r - 1 - pad, out=dx, accumulate=accumulate)
                    if acc is not None and not accumulate:
                        dx += acc
                elif (mode == "conv" and stride == 2 and "dgrad_s2" in PATHS and _filter_in_place_ok(w)
                      and lib.gc_cuda_conv_dgrad_s2_supported(n, x.shape[2], x.shape[3], cin, cout, r, pad)):
                    # one launch per parity class of input pixels, each a stride-1 convolution of dY written through a
                    # strided 4-D store map
                    dx = torch.empty_like(x)
                    nat.check(lib.gc_cuda_conv_dgrad_s2(dconv.data_ptr(), w.data_ptr(), dx.data_ptr(), n,
                                                        x.shape[2], x.shape[3], cin, cout, r, pad, _err(x.device), st()),
                              "conv_dgrad_s2")
                    if acc is not None:
                        dx += acc
                else:
                    dx = torch.ops.aten.convolution_backward(dconv, x, w, None, [stride, stride], [pad, pad], [1, 1], False,
                                                             [0, 0], 1, [True, False, False])[0]
                    if acc is not None:
                        dx = dx + acc
            if link is not None:
                link.conv_done = True
            donate = ctx.donate
            if donate is not None and dx is not None and not donate.conv_done and donate.stash is None:
                # this layer shares its input with the link's convolution, whose backward runs later: hand the gradient
                # over instead of returning it, so that that kernel adds onto it (autograd would sum the two in a pass)
                donate.stash, donate.stash_owned, dx = dx, True, None
            dw = None
            if ctx.needs_input_grad[1]:
                slot = _slot_of(w) if WGRAD_ENABLED else None       # the owner's gradient storage, or None: return a tensor
                if mode == "gemm" and WGRAD_ENABLED and cout % 32 == 0 and cin % 32 == 0:
                    # dW[Cout, Cin] = dY^T X over all positions: split-K GEMM with MN-major tcgen05 operands
                    dw2d = gemm.gemm_tn_tf32(_as_2d(dconv), _as_2d(x), out=slot, accumulate=slot is not None)
                    dw = None if slot is not None else dw2d.view(cout, cin, 1, 1).contiguous(memory_format=torch.channels_last)
                elif mode == "conv" and WGRAD_ENABLED and lib.gc_cuda_conv_wgrad_supported(n, x.shape[2], x.shape[3], cin, cout, r,
                                                                                           stride, pad):
                    dw2d = conv_wgrad(dconv, x, r, stride, pad, out=slot)
                    dw = None if slot is not None else dw2d.view(cout, r, r, cin).permute(0, 3, 1, 2)
                elif mode == "stem" and WGRAD_ENABLED and cout % 32 == 0:
                    dwp = gemm.gemm_tn_tf32(_as_2d(dconv), gathered)                       # [Cout, STEM_K]
                    dw = dwp[:, : r * r * cin].reshape(cout, r, r, cin).permute(0, 3, 1, 2)
                else:
                    dw = torch.ops.aten.convolution_backward(dconv, x, w, None, [stride, stride], [pad, pad], [1, 1], False,
                                                             [0, 0], 1, [False, True, False])[1]
            # a bias in front of a training-mode batch norm has no effect on the output: its gradient is the sum of
            # dconv over all positions, which the batch norm's backward makes zero up to rounding
            # (where the weight's owner keeps a zeroed flat gradient buffer -- the slot offer above -- the bias' place in it
            # already holds that zero, and returning nothing saves a fill and an accumulation per layer)
            dcb = (torch.zeros(cout, dtype=torch.float32, device=x.device)
                   if ctx.has_cbias and not (WGRAD_ENABLED and _slot_of(w) is not None) else None)
        return dx, dw, dcb, sums[cout:], sums[:cout], dres, None, None, None, None, None, None, None, None, None, None, None, None


def _mode(conv, bn, x):
    """Which tensor-core path runs ``conv`` on ``x`` ("gemm", "conv", "stem") or None for cuDNN."""
    if not (ENABLED and x.is_cuda and x.dtype == torch.float32 and x.dim() == 4 and isinstance(conv, torch.nn.Conv2d)):
        return None
    if not torch.backends.cudnn.allow_tf32:       # the kernels multiply in TF32: only where TF32 convolutions are allowed
        return None
    k, s, p = conv.kernel_size, conv.stride, conv.padding
    if conv.groups != 1 or conv.dilation != (1, 1) or k[0] != k[1] or s[0] != s[1] or isinstance(p, str) or p[0] != p[1]:
        return None
    if conv.padding_mode != "zeros":
        return None
    if not bn.affine or (not (bn.training or bn.running_mean is None) and torch.is_grad_enabled() and
                         (x.requires_grad or conv.weight.requires_grad)):
        return None
    n, cin, h, w = x.shape
    r, stride, pad = k[0], s[0], p[0]
    cout = conv.out_channels
    ho, wo = (h + 2 * pad - r) // stride + 1, (w + 2 * pad - r) // stride + 1
    if ho < 1 or wo < 1 or n * ho * wo < MIN_ROWS or cout % 4:
        return None
    lib = nat.cuda()
    if not lib.gc_cuda_bn_supported(n * ho * wo, cout):
        return None
    if r == 1 and stride == 1 and pad == 0:
        mode = "gemm" if cin % 4 == 0 else None
    elif (cin * r * r <= STEM_K and stride == 1 and 2 * pad == r - 1 and cout > 16 and not x.requires_grad
          and conv.weight.is_contiguous(memory_format=torch.channels_last)):
        mode = "stem"
    elif conv.weight.is_contiguous(memory_format=torch.channels_last) and lib.gc_cuda_conv_fwd_supported(n, h, w, cin, cout, r,
                                                                                                          stride, pad):
        mode = "conv"
    else:
        mode = None
    return mode if mode in PATHS else None


def conv_bn_act(conv, bn, x, residual=None, relu=True, link=None, donate=None, pool=False):
    """``act(bn(conv(x)) + residual)`` on the tensor-core kernels where the layer qualifies (cuDNN + the fused BN kernels
    otherwise).  ``link``: see ``GradLink``.  ``donate``: the ``GradLink`` of an earlier-created layer that reads the same
    ``x`` (a block's first convolution, when this layer is the projection shortcut): this layer's input gradient is then
    handed to that layer's input-gradient kernel to add onto.  ``pool=True``: a 2x2 / stride-2 max-pool of the result, folded
    into the BN kernels (no residual)."""
    mode = _mode(conv, bn, x)
    if mode is not None and pool:
        n, _, h, w = x.shape
        r, sd, pd = conv.kernel_size[0], conv.stride[0], conv.padding[0]
        ho, wo = (h + 2 * pd - r) // sd + 1, (w + 2 * pd - r) // sd + 1
        if residual is not None or not nat.cuda().gc_cuda_bn_pool_supported(n, ho, wo, conv.out_channels):
            return torch.nn.functional.max_pool2d(conv_bn_act(conv, bn, x, residual, relu, link, donate), 2, 2)
    if mode is None:
        y = bn_act(bn, conv(x), residual=residual, relu=relu)
        return torch.nn.functional.max_pool2d(y, 2, 2) if pool else y
    if link is not None:
        link.armed = LINK_ENABLED and torch.is_grad_enabled() and x.requires_grad
    training = bn.training or bn.running_mean is None
    momentum = 0.1 if bn.momentum is None else bn.momentum
    if training and bn.track_running_stats and bn.num_batches_tracked is not None:
        count_batch(bn)
    rm = bn.running_mean if bn.track_running_stats else None
    rv = bn.running_var if bn.track_running_stats else None
    return _ConvBNAct.apply(x, conv.weight, conv.bias, bn.weight, bn.bias, residual, rm, rv, training, momentum,
                            bn.eps, relu, link if (link is not None and link.armed) else None, mode, conv.stride[0],
                            conv.padding[0], donate if (donate is not None and donate.armed) else None, bool(pool))
