"""Bucket-by-bucket gradient reduction overlapped with the backward pass.

The reference reduces once, after the whole backward, on one flat buffer (trainer.py:184-193,
reducer.py:62).  ``BucketedReducer`` cuts the parameter list into buckets (in the order autograd finishes
them: last layers first), gives every bucket its own reducer instance, and launches a bucket's reduce on a
side stream as soon as all of its gradients exist -- while backward keeps computing earlier layers on the
main stream.  ``finish()`` joins the side stream before the optimiser runs.

Semantics: every bucket is an independent instance of the chosen compressor (``norm_scope = "bucket"``):
QSGD-MaxNorm normalises by the bucket's own global max-norm, which keeps the estimator unbiased and only
tightens its variance bound (a bucket's max is at most the whole gradient's max).  A single bucket
reproduces the reference's whole-gradient behaviour exactly.

The fused kernels of all buckets share one symmetric arena and therefore run one after another on the
side stream; they overlap with backward kernels, not with each other.
"""
from __future__ import annotations

import torch

from ..reducers import make_reducer


class BucketedReducer:
    def __init__(self, params, reducer_name, device, timer=None, config=None, bucket_mb=25.0, overlap=True):
        self.params = list(params)
        self.device = torch.device(device)
        cap = int(bucket_mb * (1 << 20) / 4)
        # buckets in reverse parameter order (gradients of the last layers are ready first), each a
        # contiguous range of the parameter list so that it aliases a slice of a flat arena
        self.buckets, cur, cur_n = [], [], 0
        for idx in reversed(range(len(self.params))):
            cur.append(idx)
            cur_n += self.params[idx].numel()
            if cur_n >= cap:
                self.buckets.append(sorted(cur))
                cur, cur_n = [], 0
        if cur:
            self.buckets.append(sorted(cur))
        cfg = dict(config or {})
        self.reducers = []
        for b, _ in enumerate(self.buckets):
            c = dict(cfg)
            c["seed"] = int(cfg.get("seed", 0)) * 1000003 + b          # independent noise / index streams per bucket
            self.reducers.append(make_reducer(reducer_name, device, timer, c))
        self._bucket_of = {}
        for b, idxs in enumerate(self.buckets):
            for i in idxs:
                self._bucket_of[i] = b
        self.overlap = bool(overlap) and self.device.type == "cuda"
        self.stream = torch.cuda.Stream(device=self.device, priority=-1) if self.overlap else None
        self._pending = [0] * len(self.buckets)
        self._launched = [False] * len(self.buckets)
        self._hooks = []
        self.bits = 0
        self.n_workers = self.reducers[0].n_workers

    # -- hook-driven mode -------------------------------------------------------------------
    def attach(self):
        """Register post-accumulate-grad hooks: a bucket is reduced the moment its last gradient lands."""
        for i, p in enumerate(self.params):
            self._hooks.append(p.register_post_accumulate_grad_hook(self._make_hook(i)))
        return self

    def detach(self):
        for h in self._hooks:
            h.remove()
        self._hooks = []

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

    def _launch(self, b):
        grads = [self.params[i].grad for i in self.buckets[b]]
        self._launched[b] = True
        if self.overlap:
            self.stream.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(self.stream):
                self.bits += self.reducers[b].reduce(grads, grads)
        else:
            self.bits += self.reducers[b].reduce(grads, grads)

    def finish(self):
        """Reduce whatever has not been launched (parameters without gradient hooks firing) and join."""
        for b in range(len(self.buckets)):
            if not self._launched[b]:
                if all(self.params[i].grad is not None for i in self.buckets[b]):
                    self._launch(b)
        if self.overlap:
            torch.cuda.current_stream(self.device).wait_stream(self.stream)
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
