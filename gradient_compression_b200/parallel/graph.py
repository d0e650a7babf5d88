"""One training step (zero-grad, forward, loss, backward, compressed reduce, SGD update, batch metrics) as a single
callable, optionally replayed from a CUDA graph, optionally with the reduce cut into buckets that run on a side
stream while backward still computes earlier layers.

The reference's step (trainer.py:183-196 + model_dispatcher.py:122-138) is launch-bound on a fast GPU: ~500 small
kernels for a CIFAR ResNet-50, ~20 device synchronisations from its timers, three ``.item()`` reads in its evaluation,
per-tensor Python loops in the reducer and the optimiser.  Captured once, the whole step replays with one graph
launch; the fused reducer kernels keep working under replay because their epoch, Philox step and index-window
counters live in device memory.  The step does the same work as the reference's: cross-entropy, top-1 and top-5 of
the batch are evaluated inside it and returned as device scalars.

Failure handling: behind every step the status words of the reducer's arenas are copied to pinned host memory
(asynchronously, on the step's stream, outside the graph); the next call looks at that copy if it has landed -- no
synchronisation.  A bounded device-side wait that ran out shows up there one or two steps late as ``CollectiveTimeout``; with ``fallback="dist"`` the step
then clears the status, switches the reducer to its ``torch.distributed`` backend, drops the graph and carries on.
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import _native as nat
from . import comm


class _StatusMirror:
    """Pinned host copies of the arenas' (status, detail) words, refreshed by an async copy behind every step."""

    def __init__(self, device):
        self.device = device
        self.host = None
        self.event = None
        self.ctxs = []

    def watch(self, arenas):
        ctxs = [c for a in arenas for c in a.ctxs]
        if [c.handle.value for c in ctxs] != [c.handle.value for c in self.ctxs]:
            self.ctxs = ctxs
            self.host = torch.zeros(max(len(ctxs), 1), 2, dtype=torch.int32).pin_memory()
            self.event = None


    def check(self):
        """Raise for what the last completed copy shows (nothing is waited for: a copy still in flight is looked at by
        a later call)."""
        if self.event is None or not self.event.query():
            return
        self.event = None
        for i, c in enumerate(self.ctxs):
            status, detail = int(self.host[i, 0]) & 0xFFFFFFFF, int(self.host[i, 1]) & 0xFFFFFFFF
            if status == comm.STATUS_TIMEOUT:
                raise comm.CollectiveTimeout(c.rank, detail >> 16, detail & 0xFFFF)
            if status != comm.STATUS_OK:
                raise nat.NativeError(f"fused kernel reported status {status} (detail {detail})")

    def enqueue(self):
        """Copy the status words to the host behind everything already queued on the current stream."""
        if not self.ctxs:
            return
        lib = nat.cuda()
        with torch.cuda.device(self.device):
            for i, c in enumerate(self.ctxs):
                err = lib.gc_comm_status_async(c.handle, ctypes.c_void_p(self.host[i].data_ptr()), nat.stream_ptr())
                if err != 0:
                    raise nat.NativeError(f"comm_status_async: CUDA error {err}")
            self.event = torch.cuda.Event()
            self.event.record()

    def clear(self):
        for c in self.ctxs:
            c.clear_status()
        if self.host is not None:
            self.host.zero_()
        self.event = None


class GraphedStep:
    """``step(batch) -> loss`` (a device scalar); ``step.metrics`` holds the batch's cross-entropy / top-1 / top-5 as
    device scalars after every call.

    ``reducer``: a ``Reducer`` (one reduce after the whole backward: the reference's semantics, one global max-norm) or
    a ``BucketedReducer`` (each bucket reduced on a side stream as soon as its gradients exist).
    ``enabled``: capture the step in a CUDA graph after ``eager_warmup`` eager steps.
    ``fallback``: ``None`` = a device-side timeout raises ``CollectiveTimeout``; ``"dist"`` = it is reported once
    (``self.fallback_events``), the reducer continues on ``torch.distributed`` and the step stays eager."""

    def __init__(self, task, reducer, optimizer, enabled=True, eager_warmup=3, evaluate=True, check_status=True, fallback=None):
        self.task, self.reducer, self.opt = task, reducer, optimizer
        self.want_graph = bool(enabled) and task._device.type == "cuda"
        self.eager_warmup = eager_warmup
        self.evaluate = bool(evaluate)
        self.fallback = fallback
        self.calls = 0
        self.replays = 0
        self.graph = None
        self.graphed = False
        self.kernels_per_step = 0
        self.static_x = self.static_y = self.static_loss = None
        self.bits_per_step = 0
        self.metrics = None
        self.metrics_vec = None       # [cross-entropy, top-1, top-5] of the last batch, one device tensor
        self.fallback_events = []
        self.capture_error = None
        self._bucketed = hasattr(reducer, "buckets")
        if self._bucketed:
            reducer.bind_arena(task.arena)       # driven by gradient hooks: every weight gradient must reach autograd
            task.arena.direct_grads(False)
        else:
            task.arena.direct_grads(True)        # weight-gradient kernels add straight into the flat gradient buffer
        self._status = _StatusMirror(task._device) if (check_status and task._device.type == "cuda") else None

    # -- the reducers behind this step -------------------------------------------------------
    def _reducers(self):
        return list(self.reducer.reducers) if self._bucketed else [self.reducer]

    def _arenas(self):
        out = []
        for r in self._reducers():
            eng = getattr(r, "_fused", None)
            if eng:
                out += [a for a in eng.arenas() if a not in out]
        return out

    # -- one eager step -------------------------------------------------------------------
    def _eager(self, x, y):
        task = self.task
        task.arena.detach_grads()
        if self._bucketed:
            self.reducer.start_step()
        loss, pred, m = task.forward_loss(x, y)
        loss.backward()
        if self._bucketed:
            self.bits_per_step = self.reducer.finish()          # joins the side stream; gradients are back in the arena
        else:
            grads = task.arena.collect_grads()
            self.bits_per_step = self.reducer.reduce(grads, grads)
        self.opt.step()
        loss = loss.detach()
        if self.evaluate:
            if m is None:                         # no fused head: cross-entropy is the loss, top-1 / top-5 from torch ops
                m = task.evaluate_predictions(pred.detach(), y, loss)
            self.metrics = {k: (v if torch.is_tensor(v) else torch.as_tensor(v)) for k, v in m.items()}
            # the three scalars side by side: one device-to-host copy reads a step's result
            self.metrics_vec = torch.stack([self.metrics[k].reshape(()).float() for k in
                                            ("cross_entropy_loss", "top1_accuracy", "top5_accuracy")])
        return loss

    def _graph_safe(self):
        """Capture only when the reduce step itself is host-free: a fused kernel whose per-step state (epochs, Philox
        steps, index windows) is derived on the device."""
        for r in self._reducers():
            if not (r._use_fused() and getattr(r, "_fused", None)):
                return False
            safe = getattr(r, "graph_safe", None)
            if safe is not None and not safe():
                return False
        return True

    def _set_step_from_device(self, on):
        for a in self._arenas():
            for ctx in a.ctxs:
                nat.cuda().gc_comm_set_step_from_device(ctx.handle, int(on))

    def _capture(self, x, y):
        self.static_x = x.clone(memory_format=torch.preserve_format)
        self.static_y = y.clone()
        self._set_step_from_device(True)
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        before = nat.launches()
        try:
            with torch.cuda.graph(graph):
                self.static_loss = self._eager(self.static_x, self.static_y)
        except Exception as exc:   # capture refused (e.g. a launch kind the driver cannot capture): stay eager
            self._set_step_from_device(False)
            self.want_graph = False
            self.capture_error = repr(exc)
            torch.cuda.synchronize()
            return False
        self.kernels_per_step = nat.launches() - before
        self.graph, self.graphed = graph, True
        return True

    def _run(self, x, y):
        if self.graphed:
            self.static_x.copy_(x, non_blocking=True)
            self.static_y.copy_(y, non_blocking=True)
            self.graph.replay()
            self.replays += 1
            return self.static_loss
        if self.want_graph and self.calls > self.eager_warmup and self._graph_safe():
            if self._capture(x, y):
                self.graph.replay()
                self.replays += 1
                return self.static_loss
        return self._eager(x, y)

    def _fall_back(self, exc):
        """After a device-side timeout: clear the status words, leave the graph, continue on torch.distributed."""
        self.fallback_events.append(repr(exc))
        torch.cuda.synchronize(self.task._device)
        self._status.clear()
        if self.graphed:
            self._set_step_from_device(False)
        self.graph, self.graphed, self.want_graph = None, False, False
        for r in self._reducers():
            r.backend = "dist"
        self.task.arena.collect_grads()           # re-attach the gradient views a dropped graph may have left detached

    def __call__(self, batch):
        x, y = batch
        if not x.is_cuda and self.task._device.type == "cuda":
            x, y = self.task._to_device(x, y)
        self.calls += 1
        if self._status is not None:
            try:
                self._status.check()               # the copy enqueued behind the previous step, if it has landed
            except comm.CollectiveTimeout as exc:
                if self.fallback != "dist":
                    self._status.clear()
                    raise
                self._fall_back(exc)
        out = self._run(x, y)
        if self._status is not None:
            self._status.watch(self._arenas())
            self._status.enqueue()
        return out

    def check(self):
        """Synchronise and raise if any reduce so far recorded a failure (end of an epoch, before a checkpoint)."""
        if self.task._device.type == "cuda":
            torch.cuda.synchronize(self.task._device)
        for a in self._arenas():
            a.check()

    def sync_host_counters(self):
        """Bring host-side step counters up to what the replayed graph consumed on the device, so that a checkpoint
        taken now resumes with fresh rounding-noise streams (index windows and query steps are read back from the
        device by the reducers' own ``state_dict``)."""
        if self.replays:
            for r in self._reducers():
                noise = getattr(r, "_noise", None)
                if noise is not None:
                    noise.step += self.replays + self.eager_warmup + 1
            self.replays = 0
