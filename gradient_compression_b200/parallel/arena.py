"""Flat parameter / gradient / momentum arenas.

All parameters of a model are re-pointed into one contiguous fp32 buffer, and so are their ``.grad``
tensors and the optimiser's momentum.  Consequences: the reducer sees the gradient as one vector with
no ``torch.cat`` (reference: reducer.py:62) and no per-tensor "accumulate" copy (trainer.py:188-190);
the optimiser is ONE kernel over N elements (``ops.sgd_step``) instead of a per-tensor loop; zeroing
gradients is one memset.  Tensors are packed back to back (``align=1``) so that the parameter list
aliases the flat buffer exactly; ``align=4`` starts every tensor on a 16-byte boundary instead.
"""
from __future__ import annotations

import torch

from .. import ops


class FlatArena:
    def __init__(self, params, align=1, with_momentum=True):
        self.params = [p for p in params]
        dev = self.params[0].device
        self.offsets, off = [], 0
        for p in self.params:
            assert p.dtype == torch.float32, "the arena holds fp32 parameters"
            self.offsets.append(off)
            off += (p.numel() + align - 1) // align * align
        self.total = off
        self.numel = sum(p.numel() for p in self.params)
        self.flat_params = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.flat_grads = torch.zeros(self.total, dtype=torch.float32, device=dev)
        self.flat_momentum = torch.zeros(self.total, dtype=torch.float32, device=dev) if with_momentum else None
        # grad_views / param_views: contiguous views in PHYSICAL element order (what reducers and the optimiser see);
        # a parameter in channels-last layout keeps that layout -- its segment holds [Cout][kh][kw][Cin] and the tensor
        # autograd sees is a permuted view of it -- so cuDNN never has to re-lay-out a weight (25 convolutions x forward
        # and backward of ResNet-50 did, 0.2 ms per step, when the arena flattened everything to NCHW order)
        self.grad_views, self.param_views, self._logical_grads = [], [], []
        with torch.no_grad():
            for p, o in zip(self.params, self.offsets):
                pv, logical_p = self._views(self.flat_params[o: o + p.numel()], p)
                logical_p.copy_(p.data)
                p.data = logical_p
                gv, logical_g = self._views(self.flat_grads[o: o + p.numel()], p)
                p.grad = logical_g
                self.param_views.append(pv)
                self.grad_views.append(gv)
                self._logical_grads.append(logical_g)
        self.dense = self.total == self.numel   # no padding holes: the list aliases the flat buffer exactly
        self._direct = False                    # weight-gradient kernels add straight into flat_grads (see direct_grads)

    def direct_grads(self, on=True):
        """Offer every 4-D weight's place in ``flat_grads`` to the tensor-core weight-gradient kernels, which then add dW
        there and hand autograd nothing for that weight: no per-layer gradient tensor, no zero fill of it, no copy into the
        flat buffer.  The buffer is zeroed at the start of every step (``detach_grads`` / ``zero_grad``).  Gradient hooks
        do not fire for such weights, so reducers that are driven by hooks must not turn this on."""
        if not self.flat_grads.is_cuda:
            return self
        from ..ops import conv

        self._direct = bool(on)
        if on:
            conv.offer_grad_slots(self.params, [gv if p.dim() == 4 else None for p, gv in zip(self.params, self.grad_views)])
        else:
            conv.withdraw_grad_slots(self.params)
        return self

    @staticmethod
    def _views(segment, p):
        """(contiguous view in physical order, view with p's logical shape) of a flat segment."""
        if p.dim() == 4 and p.is_contiguous(memory_format=torch.channels_last) and not p.is_contiguous():
            n, c, h, w = p.shape
            physical = segment.view(n, h, w, c)
            return physical, physical.permute(0, 3, 1, 2)
        v = segment.view(p.shape)
        return v, v

    def zero_grad(self):
        self.flat_grads.zero_()
        for p, gv in zip(self.params, self._logical_grads):
            if p.grad is not gv:           # someone set .grad to None / a new tensor: re-attach
                p.grad = gv

    def grads(self):
        return self.grad_views

    def detach_grads(self):
        """Let autograd allocate fresh gradients in the next backward (no accumulate-into-view kernels)."""
        if self._direct:
            self.flat_grads.zero_()           # the weight-gradient kernels add onto their slots
        for p in self.params:
            p.grad = None

    def collect_grads(self):
        """Copy the gradients autograd produced into the flat buffer with one multi-tensor kernel and
        re-attach the views.  Together with ``detach_grads`` this replaces one memset plus one in-place
        add per parameter tensor (161 launches for ResNet-50) by a single launch."""
        src, dst = [], []
        for p, gv in zip(self.params, self._logical_grads):
            if p.grad is None:
                # direct mode: the whole buffer was zeroed when the step began, and whatever belongs here was added by the
                # weight-gradient kernels (or is zero: an unused parameter, a bias in front of a batch norm)
                if not self._direct:
                    gv.zero_()
            elif p.grad is not gv:
                src.append(p.grad)
                dst.append(gv)
        if src:
            torch._foreach_copy_(dst, src)
        for p, gv in zip(self.params, self._logical_grads):
            p.grad = gv
        return self.grad_views

    def sgd_step(self, hyper=None, lr=None, momentum=0.9, weight_decay=5e-4, nesterov=True):
        ops.sgd_step(self.flat_params, self.flat_grads, self.flat_momentum, lr=lr, momentum=momentum,
                     weight_decay=weight_decay, nesterov=nesterov, hyper=hyper)
        if self.flat_params.is_cuda:
            from ..ops import conv

            conv.refresh_transposed(self, self.params)        # transposed 1x1 weights for the input-gradient GEMMs

    def state_dict(self):
        return {"momentum": self.flat_momentum.clone() if self.flat_momentum is not None else None}

    def load_state_dict(self, sd):
        if sd.get("momentum") is not None and self.flat_momentum is not None:
            self.flat_momentum.copy_(sd["momentum"])


class FlatSGD:
    """SGD(momentum, Nesterov, weight decay) over a ``FlatArena`` with a scheduler-friendly ``lr``.

    Mirrors what the reference configures with ``optim.SGD(..., momentum=0.9, weight_decay=5e-4,
    nesterov=True)`` + ``CosineAnnealingLR`` (trainer.py:163-166), as one fused kernel.  The
    hyper-parameters live in a 3-float device tensor, so a captured CUDA graph sees new values."""

    def __init__(self, arena, lr=0.1, momentum=0.9, weight_decay=5e-4, nesterov=True):
        self.arena = arena
        self.base_lr = lr
        self.lr, self.momentum, self.weight_decay, self.nesterov = lr, momentum, weight_decay, nesterov
        self.hyper = torch.tensor([lr, momentum, weight_decay], dtype=torch.float32, device=arena.flat_params.device)

    def set_lr(self, lr):
        self.lr = float(lr)
        self.hyper[0] = self.lr

    def step(self):
        self.arena.sgd_step(hyper=self.hyper, nesterov=self.nesterov)

    def zero_grad(self):
        self.arena.zero_grad()

    def state_dict(self):
        return {"lr": self.lr, "base_lr": self.base_lr, "momentum_buf": self.arena.flat_momentum.clone()}

    def load_state_dict(self, sd):
        self.base_lr = sd["base_lr"]
        self.set_lr(sd["lr"])
        self.arena.flat_momentum.copy_(sd["momentum_buf"])


class CosineSchedule:
    """eta_t = eta_min + (base - eta_min) * (1 + cos(pi * t / T_max)) / 2, stepped once per epoch
    (``CosineAnnealingLR(T_max=num_epochs, eta_min=0)``, trainer.py:166,198)."""

    def __init__(self, optimizer, T_max, eta_min=0.0):
        self.opt, self.T_max, self.eta_min, self.epoch = optimizer, T_max, eta_min, 0

    def get_last_lr(self):
        return [self.opt.lr]

    def step(self):
        import math

        self.epoch += 1
        lr = self.eta_min + (self.opt.base_lr - self.eta_min) * (1 + math.cos(math.pi * self.epoch / self.T_max)) / 2
        self.opt.set_lr(lr)

    def state_dict(self):
        return {"epoch": self.epoch}

    def load_state_dict(self, sd):
        self.epoch = int(sd["epoch"])
