"""Fused batch-norm (+ residual add) (+ ReLU) for channels-last fp32 activations.

``bn_act(bn_module, x, residual=None, relu=True)`` computes ``relu(bn(x) + residual)`` -- the pattern
of every block of the zoo (reference: models/resnet.py:71-75, models/vgg.py:105-106) -- with the
kernels of ``csrc/gc_bn.cu`` on CUDA and with the equivalent torch ops on CPU.  The module stays a plain
``torch.nn.BatchNorm2d`` (same parameters, buffers and ``state_dict`` keys); only the arithmetic moves.
"""
from __future__ import annotations

import os
import weakref

import torch
import torch.nn.functional as F

from . import _native as nat

# Gradient tensors this library allocated itself and handed to autograd for a residual input: nobody else holds
# them, so a later kernel may accumulate into them in place (``ops.conv.GradLink``).  Keyed by address, checked by
# object identity through a weak reference, so a freed and re-used address never matches.
_owned_grads = {}


# ``num_batches_tracked`` of the batch norms of a model that called ``defer_batch_counters``: incremented together by
# one multi-tensor launch when the model's forward returns, instead of one tiny launch per layer (53 for ResNet-50).
_pending_counters = {}


def count_batch(bn):
    t = bn.num_batches_tracked
    if getattr(bn, "_gcb200_deferred_counter", False) and t.is_cuda:
        e = _pending_counters.get(id(t))
        if e is None:
            _pending_counters[id(t)] = [t, 1]
        else:
            e[1] += 1
        if len(_pending_counters) > 4096:
            flush_batch_counters()
    else:
        t.add_(1)


def flush_batch_counters():
    if _pending_counters:
        entries = list(_pending_counters.values())
        _pending_counters.clear()
        if all(n == 1 for _, n in entries):
            torch._foreach_add_([t for t, _ in entries], 1)
        else:
            for t, n in entries:
                t.add_(n)


def _flush_hook(module, inputs, output):
    flush_batch_counters()


def defer_batch_counters(model):
    """Batch the ``num_batches_tracked`` increments of every batch norm under ``model`` into one launch at the end of
    ``model``'s forward."""
    for m in model.modules():
        if isinstance(m, torch.nn.modules.batchnorm._BatchNorm):
            m._gcb200_deferred_counter = True
    model.register_forward_hook(_flush_hook)
    return model


def own_grad(t):
    if len(_owned_grads) >= 256:
        for k in [k for k, r in _owned_grads.items() if r() is None]:
            del _owned_grads[k]
        if len(_owned_grads) >= 256:
            _owned_grads.clear()
    _owned_grads[t.data_ptr()] = weakref.ref(t)
    return t


def take_owned_grad(t):
    """True exactly once for a tensor registered with ``own_grad``."""
    r = _owned_grads.pop(t.data_ptr(), None)
    return r is not None and r() is t

_scratch = {}
FUSED_BWD_FINALIZE = os.environ.get("GCB200_BN_FUSED_BWD_FINALIZE", "0") == "1"


def _scratch_for(device, channels):
    key = (device.type, device.index)
    cur = _scratch.get(key)
    need = nat.cuda().gc_cuda_bn_scratch_bytes(int(channels))
    if cur is None or cur.numel() < need:
        cur = torch.empty(max(need, nat.cuda().gc_cuda_bn_scratch_bytes(2048)), dtype=torch.uint8, device=device)
        _scratch[key] = cur
    return cur


def _fin_ptr(device, channels):
    """Scratch that lets the backward reduction finish its sums inside its own launch (None: separate finalize)."""
    from . import gemm

    if not FUSED_BWD_FINALIZE or channels > gemm.FIN_MAX_CHANNELS:
        return None
    return gemm.fin_scratch(device).data_ptr()


def _cl(t):
    return t if t.is_contiguous(memory_format=torch.channels_last) else t.contiguous(memory_format=torch.channels_last)


def kernel_path_ok(x):
    if not (x.is_cuda and x.dtype == torch.float32 and x.dim() == 4):
        return False
    n, c, h, w = x.shape
    return bool(nat.cuda().gc_cuda_bn_supported(n * h * w, c))


class _FusedBNAct(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, residual, running_mean, running_var, training, momentum, eps, relu):
        x = _cl(x)
        n, c, h, w = x.shape
        m = n * h * w
        lib, st = nat.cuda(), nat.stream_ptr()
        stats = torch.empty(2 * c, dtype=torch.float32, device=x.device)
        with torch.cuda.device(x.device):
            if training:
                nat.check(lib.gc_cuda_bn_stats(x.data_ptr(), m, c, _scratch_for(x.device, c).data_ptr(), stats.data_ptr(),
                                               nat.ptr(running_mean), nat.ptr(running_var), float(momentum), float(eps),
                                               st), "bn_stats")
                nat.count_launch()
            else:
                stats[:c] = running_mean
                stats[c:] = torch.rsqrt(running_var + eps)
            res = _cl(residual) if residual is not None else None
            y = torch.empty_like(x)
            nat.check(lib.gc_cuda_bn_apply(x.data_ptr(), m, c, stats.data_ptr(), weight.data_ptr(), bias.data_ptr(),
                                           nat.ptr(res), int(relu), y.data_ptr(), st), "bn_apply")
        ctx.relu, ctx.has_res, ctx.training = bool(relu), residual is not None, bool(training)
        ctx.save_for_backward(x, weight, bias, stats, y if (residual is not None and relu) else None)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, weight, bias, stats, y = ctx.saved_tensors
        dy = _cl(dy)
        n, c, h, w = x.shape
        m = n * h * w
        lib, st = nat.cuda(), nat.stream_ptr()
        if not ctx.training:
            raise RuntimeError("bn_act: backward through eval-mode statistics is not supported by the fused kernel")
        sums = torch.empty(2 * c, dtype=torch.float32, device=x.device)
        dx = torch.empty_like(x)
        dres = own_grad(torch.empty_like(x)) if (ctx.has_res and ctx.needs_input_grad[3]) else None
        with torch.cuda.device(x.device):
            nat.check(lib.gc_cuda_bn_bwd_reduce(dy.data_ptr(), x.data_ptr(), nat.ptr(y), m, c, stats.data_ptr(),
                                                weight.data_ptr(), bias.data_ptr(), int(ctx.relu),
                                                _scratch_for(x.device, c).data_ptr(), sums.data_ptr(), _fin_ptr(x.device, c), st),
                      "bn_bwd_reduce")
            nat.count_launch()
            nat.check(lib.gc_cuda_bn_bwd_apply(dy.data_ptr(), x.data_ptr(), nat.ptr(y), m, c, stats.data_ptr(),
                                               weight.data_ptr(), bias.data_ptr(), sums.data_ptr(), int(ctx.relu),
                                               dx.data_ptr(), nat.ptr(dres), st), "bn_bwd_apply")
        if ctx.has_res and dres is None and ctx.needs_input_grad[3]:
            dres = dy
        return dx, sums[c:], sums[:c], dres, None, None, None, None, None, None


def bn_act(bn, x, residual=None, relu=True):
    """``relu(bn(x) + residual)`` with ``bn`` a ``torch.nn.BatchNorm2d`` (affine, tracking running stats)."""
    training = bn.training or bn.running_mean is None
    use_kernel = kernel_path_ok(x) and bn.affine and not (not training and torch.is_grad_enabled() and x.requires_grad)
    if not use_kernel:
        y = bn(x)
        if residual is not None:
            y = y + residual
        return F.relu(y) if relu else y
    momentum = 0.1 if bn.momentum is None else bn.momentum
    if training and bn.track_running_stats and bn.num_batches_tracked is not None:
        count_batch(bn)
    rm = bn.running_mean if bn.track_running_stats else None
    rv = bn.running_var if bn.track_running_stats else None
    return _FusedBNAct.apply(x, bn.weight, bn.bias, residual, rm, rv, training, momentum, bn.eps, relu)
