"""One training step (zero-grad, forward, loss, backward, compressed reduce, SGD update) as a single
callable, optionally replayed from a CUDA graph.

The reference's step is launch-bound on a fast GPU: ~500 small kernels for a CIFAR ResNet-50, ~20
device synchronisations from its timers, per-tensor Python loops in the reducer and the optimiser.
Captured once, the whole step replays with one graph launch; the fused reducer kernels keep working
under replay because their epoch and Philox step counters live in device memory.
"""
from __future__ import annotations

import torch

from ..ops import _native as nat


class GraphedStep:
    def __init__(self, task, reducer, optimizer, enabled=True, eager_warmup=3):
        self.task, self.reducer, self.opt = task, reducer, optimizer
        self.want_graph = bool(enabled) and task._device.type == "cuda"
        self.eager_warmup = eager_warmup
        self.calls = 0
        self.graph = None
        self.graphed = False
        self.kernels_per_step = 0
        self.static_x = self.static_y = self.static_loss = None
        self.bits_per_step = 0

    # -- one eager step -------------------------------------------------------------------
    def _eager(self, x, y):
        task = self.task
        task.arena.detach_grads()
        loss = task._criterion(task._model(x), y)
        loss.backward()
        grads = task.arena.collect_grads()
        self.bits_per_step = self.reducer.reduce(grads, grads)
        self.opt.step()
        return loss.detach()

    def _graph_safe(self):
        """Capture only when the reduce step itself is host-free (fused kernel or a single worker)."""
        r = self.reducer
        if r.n_workers == 1 and not r._use_fused():
            return False
        return bool(r._use_fused() and getattr(r, "_fused", None))

    def _capture(self, x, y):
        self.static_x = x.clone(memory_format=torch.preserve_format)
        self.static_y = y.clone()
        eng = self.reducer._fused
        for ctx in eng.ops.arena.ctxs:
            nat.cuda().gc_comm_set_step_from_device(ctx.handle, 1)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = nat.launches()
        try:
            with torch.cuda.graph(graph):
                self.static_loss = self._eager(self.static_x, self.static_y)
        except Exception as exc:   # capture refused (e.g. a launch kind the driver cannot capture): stay eager
            for ctx in eng.ops.arena.ctxs:
                nat.cuda().gc_comm_set_step_from_device(ctx.handle, 0)
            self.want_graph = False
            self.capture_error = repr(exc)
            torch.cuda.synchronize()
            return False
        self.kernels_per_step = nat.launches() - before
        self.graph, self.graphed = graph, True
        return True

    def __call__(self, batch):
        x, y = batch
        if not x.is_cuda:
            x, y = self.task._to_device(x, y)
        self.calls += 1
        if self.graphed:
            self.static_x.copy_(x, non_blocking=True)
            self.static_y.copy_(y, non_blocking=True)
            self.graph.replay()
            return self.static_loss
        if self.want_graph and self.calls > self.eager_warmup and self._graph_safe():
            if self._capture(x, y):
                self.graph.replay()
                return self.static_loss
        return self._eager(x, y)
