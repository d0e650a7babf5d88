"""Classifier head: global average pool + linear + softmax cross-entropy + top-1 / top-5 of the batch
(``csrc/gc_head.cu``: one forward kernel, two backward kernels; the metrics never leave the device).

``head_loss(features, linear, labels)`` returns ``(loss, logits, metrics)`` where ``features`` is the last feature map
``[N, C, H, W]`` (averaged over all of H x W), ``loss`` the mean cross-entropy (differentiable), ``logits`` the class
scores and ``metrics`` a 3-element tensor ``[cross-entropy, top-1 rate, top-5 rate]``.  On CPU, and for shapes the
kernels do not cover, the same values come from torch ops.

The reference computes them with ``F.avg_pool2d`` + ``nn.Linear`` (models/resnet.py:106-108), ``CrossEntropyLoss`` twice
and ``topk`` / ``eq`` / ``sum`` followed by three ``.item()`` reads (model_dispatcher.py:127-128,140-164).
"""
from __future__ import annotations

import torch
import torch.nn.functional as F

from . import _native as nat

_scratch = {}


def _scratch_for(device, batch):
    key = (device.type, device.index)
    need = int(nat.cuda().gc_cuda_head_scratch_bytes(int(batch)))
    cur = _scratch.get(key)
    if cur is None or cur.numel() < need:
        cur = torch.zeros(max(need, int(nat.cuda().gc_cuda_head_scratch_bytes(4096))), dtype=torch.uint8, device=device)
        _scratch[key] = cur
    return cur


def supported(features, weight, labels):
    if not (features.is_cuda and features.dtype == torch.float32 and features.dim() == 4 and weight.dtype == torch.float32
            and labels.dtype == torch.int64):
        return False
    n, c, h, w = features.shape
    if weight.data_ptr() % 16 or not weight.is_contiguous():      # the kernels read W in 16-byte quads
        return False
    return bool(nat.cuda().gc_cuda_head_supported(n, h * w, c, weight.shape[0]))


class _HeadCE(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, labels):
        n, c, h, w = x.shape
        x = x if x.is_contiguous(memory_format=torch.channels_last) else x.contiguous(memory_format=torch.channels_last)
        k = weight.shape[0]
        dev = x.device
        pooled = torch.empty(n, c, dtype=torch.float32, device=dev)
        logits = torch.empty(n, k, dtype=torch.float32, device=dev)
        dlogits = torch.empty(n, k, dtype=torch.float32, device=dev)
        out3 = torch.empty(3, dtype=torch.float32, device=dev)
        wc = weight.contiguous()
        with torch.cuda.device(dev):
            nat.check(nat.cuda().gc_cuda_head_forward(x.data_ptr(), n, h * w, c, wc.data_ptr(), nat.ptr(bias), k, labels.data_ptr(),
                                                      pooled.data_ptr(), logits.data_ptr(), dlogits.data_ptr(),
                                                      _scratch_for(dev, n).data_ptr(), out3.data_ptr(), nat.stream_ptr()),
                      "head_forward")
        ctx.save_for_backward(pooled, dlogits, wc)
        ctx.shape, ctx.has_bias = (n, c, h, w), bias is not None
        ctx.mark_non_differentiable(logits, out3)
        return out3[0].clone(), logits, out3

    @staticmethod
    def backward(ctx, gloss, _glogits, _gmetrics):
        pooled, dlogits, wc = ctx.saved_tensors
        n, c, h, w = ctx.shape
        k = wc.shape[0]
        dev = pooled.device
        need_x, need_w = ctx.needs_input_grad[0], ctx.needs_input_grad[1]
        dx = torch.empty((n, c, h, w), dtype=torch.float32, device=dev, memory_format=torch.channels_last) if need_x else None
        dw = torch.empty(k, c, dtype=torch.float32, device=dev) if need_w else None
        db = torch.empty(k, dtype=torch.float32, device=dev) if (ctx.has_bias and need_w) else None
        g = gloss.contiguous().float()
        with torch.cuda.device(dev):
            nat.check(nat.cuda().gc_cuda_head_backward(dlogits.data_ptr(), pooled.data_ptr(), wc.data_ptr(), g.data_ptr(), n, h * w, c,
                                                       k, nat.ptr(dx), nat.ptr(dw), nat.ptr(db), nat.stream_ptr()), "head_backward")
            if need_x and need_w:
                nat.count_launch()
        return dx, dw, db, None


def head_loss(features, linear, labels):
    """``(mean cross-entropy, logits, [cross-entropy, top-1, top-5])`` of ``linear(mean over H, W of features)``."""
    if supported(features, linear.weight, labels):
        return _HeadCE.apply(features, linear.weight, linear.bias, labels)
    logits = linear(features.mean((2, 3)) if features.dim() == 4 else features)
    loss = F.cross_entropy(logits, labels)
    with torch.no_grad():
        top5 = logits.topk(min(5, logits.shape[1]), 1, True, True)[1]
        hit = top5.eq(labels.view(-1, 1))
        metrics = torch.stack([loss.detach(), hit[:, 0].float().mean(), hit.float().sum(1).clamp(max=1).mean()])
    return loss, logits, metrics
