"""Top-K sparsifying reducers with error feedback (reference: reducer.py:1144-1451).

One implementation serves the four reference classes; they differ only in how the flat gradient is cut
into segments (one per tensor, or one for everything) and in how K is derived.  Per step:
``a = g + memory``; per segment the K largest |a| are selected; ``memory = a`` with the selected entries
zeroed; every worker's (index, value) list reaches every other worker and the mean of the scattered
contributions becomes the gradient.  On CUDA the selection is the batched radix select of ``ops.topk``
(7 launches for any number of tensors); with the fused backend the exchange + scatter-add is one kernel
over peer memory, otherwise two all-gathers and ``index_add_``.
"""
from __future__ import annotations

import torch

from ..ops.topk import TopKSelector
from .base import Reducer, TensorBuffer


class _TopKBase(Reducer):
    fused_capable = True
    layerwise = True
    position_bits = 32          # what the reference's position arrays cost per entry

    def __init__(self, device, timer=None, **kw):
        super().__init__(device, timer, **kw)
        self._memory = None
        self._selector = None
        self._selector_key = None

    def _top_size(self, numel):
        raise NotImplementedError

    def _get_selector(self, flat, grad_in):
        key = (tuple(tuple(t.shape) for t in grad_in), str(flat.buffer.device))
        if self._selector_key != key:
            if self.layerwise:
                segs = [(s, e - s, self._top_size(e - s)) for s, e in zip(flat._start_idx, flat._end_idx)]
            else:
                segs = [(0, flat.total, self._top_size(flat.total))]
            self._selector, self._selector_key = TopKSelector(segs, flat.buffer.device), key
        return self._selector

    def reduce(self, grad_in, grad_out):
        with self._timer("reduce.flat_pack"):
            flat = TensorBuffer(grad_in)
        if self._memory is None:
            self._memory = torch.zeros_like(flat.buffer)
        sel = self._get_selector(flat, grad_in)
        with self._timer("reduce.topk", verbosity=2):
            idx, vals = sel.select(flat.buffer, self._memory)       # also updates the memory
        bits = sel.total * (32 + self.position_bits)
        self.last_wire_bits = sel.total * 64
        if self._use_fused():
            from ..parallel import engine as fused
            if fused.sparse(self, flat, grad_out, idx, vals):
                return bits
        with self._timer("reduce.gather", verbosity=2):
            all_vals = self._all_gather(vals)
            all_idx = self._all_gather(idx)
        with self._timer("reduce.combine", verbosity=2):
            out = torch.zeros_like(flat.buffer)
            for i, v in zip(all_idx, all_vals):
                out.index_add_(0, i.long(), v, alpha=1.0 / self.n_workers)
            if flat.is_view:
                flat.buffer.copy_(out)
            else:
                flat.buffer = out
            flat.scatter_to(grad_out)
        return bits

    def state_dict(self):
        return {"memory": self._memory} if self._memory is not None else {}

    def load_state_dict(self, sd):
        if "memory" in sd:
            self._memory = sd["memory"].to(self._device).clone()


class TopKReducer(_TopKBase):
    """Layer-wise Top-K: per tensor the K largest |g + memory| (reducer.py:1144-1225)."""

    def __init__(self, device, timer=None, K=100, **kw):
        super().__init__(device, timer, **kw)
        self._K = K

    def _top_size(self, numel):
        return min(numel, self._K)


class TopKReducerRatio(_TopKBase):
    """Layer-wise Top-K with K_l = max(1, int(ratio * numel)) (reducer.py:1228-1309)."""

    def __init__(self, device, timer=None, compression=1 / 100, **kw):
        super().__init__(device, timer, **kw)
        self._compression = compression

    def _top_size(self, numel):
        return max(1, int(self._compression * numel))


class GlobalTopKReducer(_TopKBase):
    """Top-K over the whole flat gradient (reducer.py:1312-1380).

    Default result: mean of the workers' sparse contributions.  ``reference_compat=True`` reproduces the
    reference, which adds the gathered values onto the full local gradient and divides by W a second time
    (reducer.py:1366-1375)."""

    layerwise = False
    position_bits = 64          # the reference gathers int64 positions here

    def __init__(self, device, timer=None, K=10000, **kw):
        super().__init__(device, timer, **kw)
        self._K = K

    def _top_size(self, numel):
        return min(numel, self._K)

    def reduce(self, grad_in, grad_out):
        if not self._compat:
            return super().reduce(grad_in, grad_out)
        flat = TensorBuffer(grad_in)
        if self._memory is None:
            self._memory = torch.zeros_like(flat.buffer)
        a = flat.buffer + self._memory
        k = self._top_size(a.numel())
        positions = torch.topk(a.abs(), k, sorted=False)[1]
        values = a[positions].contiguous()
        self._memory.copy_(a)
        self._memory[positions] = 0.0
        out = a.clone()
        for pos, val in zip(self._all_gather(positions), self._all_gather(values)):
            out.index_add_(0, pos, val / self.n_workers)
        out.mul_(1.0 / self.n_workers)
        if flat.is_view:
            flat.buffer.copy_(out)
        else:
            flat.buffer = out
        flat.scatter_to(grad_out)
        return k * 96


class GlobalTopKReducerRatio(GlobalTopKReducer):
    """Global Top-K with K = max(1, int(ratio * N)) (reducer.py:1383-1451)."""

    def __init__(self, device, timer=None, compression=1 / 100, **kw):
        super().__init__(device, timer, K=0, **kw)
        self._compression = compression

    def _top_size(self, numel):
        return max(1, int(self._compression * numel))
