"""Bucket-by-bucket gradient reduction overlapped with the backward pass.

The reference reduces once, after the whole backward, on one flat buffer (trainer.py:184-193,
reducer.py:62).  ``BucketedReducer`` cuts the parameter list into buckets (in the order autograd finishes
them: last layers first), gives every bucket its own reducer instance, and launches a bucket's reduce on a
side stream as soon as all of its gradients exist -- while backward keeps computing earlier layers on the
main stream.  ``finish()`` joins the side stream before the optimiser runs.  The fork (side stream waits for
the main stream at the bucket's last gradient) and the join are plain stream dependencies, so the whole
arrangement can be captured in a CUDA graph and replays as parallel branches.

Semantics: every bucket is an independent instance of the chosen compressor (``norm_scope = "bucket"``):
QSGD-MaxNorm normalises by the bucket's own global max-norm, which keeps the estimator unbiased and only
tightens its variance bound (a bucket's max is at most the whole gradient's max).  A single bucket
reproduces the reference's whole-gradient behaviour exactly.

The fused kernels of all buckets share one symmetric arena and therefore run one after another on the
side stream; they overlap with backward kernels, not with each other.  ``max_blocks`` caps the grid of each
fused launch: the cooperative kernel's blocks spin while they wait for their peers, so they are kept to a
small share of the SMs and the backward kernels they run beside keep the rest.
"""
from __future__ import annotations

import os

import torch

from ..reducers import make_reducer


class BucketedReducer:
    def __init__(self, params, reducer_name, device, timer=None, config=None, bucket_mb=25.0, overlap=True, max_blocks=32,
                 tail_mb=2.0):
        self.params = list(params)
        self.device = torch.device(device)
        cap = int(bucket_mb * (1 << 20) / 4)
        # The bucket that is reduced last holds the first parameters (their gradients are the last to exist) and its
        # reduce is the only one that nothing can hide: it is kept small (``tail_mb``) and gets the whole GPU.
        tail_cap, n_tail, acc = int(tail_mb * (1 << 20) / 4), 0, 0
        if tail_cap > 0 and sum(p.numel() for p in self.params) > cap:
            for p in self.params[:-1]:
                if acc + p.numel() > tail_cap:
                    break
                acc += p.numel()
                n_tail += 1
        # the other buckets in reverse parameter order (gradients of the last layers are ready first), each a
        # contiguous range of the parameter list so that it aliases a slice of a flat arena
        self.buckets, cur, cur_n = [], [], 0
        for idx in reversed(range(n_tail, len(self.params))):
            cur.append(idx)
            cur_n += self.params[idx].numel()
            if cur_n >= cap:
                self.buckets.append(sorted(cur))
                cur, cur_n = [], 0
        if cur:
            self.buckets.append(sorted(cur))
        if n_tail:
            self.buckets.append(list(range(n_tail)))
        cfg = dict(config or {})
        self.reducers = []
        for b, _ in enumerate(self.buckets):
            c = dict(cfg)
            c["seed"] = int(cfg.get("seed", 0)) * 1000003 + b          # independent noise / index streams per bucket
            self.reducers.append(make_reducer(reducer_name, device, timer, c))
        largest = max(sum(self.params[i].numel() for i in idxs) for idxs in self.buckets)
        for r in self.reducers:
            r.fused_arena_elements = largest       # all buckets share one arena: size it once, for the largest of them
        self._bucket_of = {}
        for b, idxs in enumerate(self.buckets):
            for i in idxs:
                self._bucket_of[i] = b
        self.overlap = bool(overlap) and self.device.type == "cuda"
        self.stream = torch.cuda.Stream(device=self.device, priority=-1) if self.overlap else None
        self.max_blocks = int(max_blocks) if self.overlap else 0
        if self.overlap and os.environ.get("GCB200_BUCKET_PLAIN_LAUNCH", "1") == "1":
            from ..ops import _native as nat

            nat.cuda().gc_fused_small_grid_plain_launch(1)     # small grids as ordinary launches: they may overlap backward
        self._pending = [0] * len(self.buckets)
        self._launched = [False] * len(self.buckets)
        self._hooks = []
        self._arena = None
        self.bits = 0
        self.n_workers = self.reducers[0].n_workers
        self.rank = self.reducers[0].rank

    # -- hook-driven mode -------------------------------------------------------------------
    def attach(self):
        """Register post-accumulate-grad hooks: a bucket is reduced the moment its last gradient lands."""
        if not self._hooks:
            for i, p in enumerate(self.params):
                self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(i)))
        return self

    def detach(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []

    def bind_arena(self, arena):
        """Reduce in place inside ``arena``'s flat gradient buffer: autograd hands fresh gradient tensors to the hooks
        (``arena.detach_grads()`` before backward), a bucket's gradients are copied into their arena slots with one
        multi-tensor launch on the side stream, reduced there, and ``finish()`` re-attaches the arena views as
        ``.grad``.  Parameters must be the arena's, in its order."""
        assert [id(p) for p in arena.params] == [id(p) for p in self.params], "the arena's parameter list, in its order"
        self._arena = arena
        return self.attach()

    def start_step(self):
        self._pending = [len(idxs) for idxs in self.buckets]
        self._launched = [False] * len(self.buckets)
        self.bits = 0

    def _make_hook(self, i):
        def hook(param):
            b = self._bucket_of[i]
            self._pending[b] -= 1
            if self._pending[b] == 0 and not self._launched[b]:
                self._launch(b)
        return hook

    def _reduce_bucket(self, b):
        idxs = self.buckets[b]
        if self._arena is not None:
            views = [self._arena.grad_views[i] for i in idxs]            # physical-order views of the flat buffer
            logical = [self._arena._logical_grads[i] for i in idxs]
            src, dst = [], []
            for i, lg in zip(idxs, logical):
                g = self.params[i].grad
                if g is None:
                    lg.zero_()
                elif g is not lg:
                    src.append(g)
                    dst.append(lg)
            if src:
                torch._foreach_copy_(dst, src)
            grads = views
        else:
            grads = [self.params[i].grad for i in idxs]
        red = self.reducers[b]
        # every bucket but the last runs beside backward kernels on a capped grid; the last one has the GPU to itself
        red.fused_max_blocks = self.max_blocks if b + 1 < len(self.buckets) else 0
        self.bits += red.reduce(grads, grads)

    def _launch(self, b):
        self._launched[b] = True
        if self.overlap:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                self._reduce_bucket(b)
        else:
            self._reduce_bucket(b)

    def finish(self):
        """Reduce whatever has not been launched (parameters whose hooks did not fire), join the side stream and, with
        an arena bound, make the arena views the parameters' ``.grad`` again."""
        for b in range(len(self.buckets)):
            if not self._launched[b]:
                if self._arena is not None or all(self.params[i].grad is not None for i in self.buckets[b]):
                    self._launch(b)
        if self.overlap:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
        if self._arena is not None:
            for p, gv in zip(self._arena.params, self._arena._logical_grads):
                p.grad = gv
        return self.bits

    # -- plain mode (same result, no hooks): reduce(grad_in, grad_out) over all buckets ---------------
    def reduce(self, grad_in, grad_out):
        bits = 0
        for b, idxs in enumerate(self.buckets):
            bits += self.reducers[b].reduce([grad_in[i] for i in idxs], [grad_out[i] for i in idxs])
        return bits

    def state_dict(self):
        return {"buckets": [r.state_dict() for r in self.reducers]}

    def load_state_dict(self, sd):
        for r, s in zip(self.reducers, sd["buckets"]):
            r.load_state_dict(s)
