"""Top-K sparsifying reducers with error feedback (reference: reducer.py:1144-1451)."""
from __future__ import annotations

import torch

from .base import Reducer, TensorBuffer, n_bits


class TopKReducer(Reducer):
    """Layer-wise Top-K: per tensor keep the K largest |g + memory|, remember the rest, all-gather
    (value, position) lists and scatter-add their mean (reducer.py:1144-1225).

    Selection of all layers runs as one batched pass over the flat buffer when ``ops.topk`` has a
    device kernel; positions travel as int32 like in the reference."""

    def __init__(self, device, timer=None, K=100, **kw):
        super().__init__(device, timer, **kw)
        self._K = K
        self._memory = None

    def _top_size(self, numel):
        return min(numel, self._K)

    def reduce(self, grad_in, grad_out):
        with self._timer("reduce.memory", verbosity=2):
            flat = TensorBuffer(grad_in)
            if self._memory is None:
                self._memory = torch.zeros_like(flat.buffer)
            else:
                flat.buffer.add_(self._memory)
        sizes = [self._top_size(t.numel()) for t in grad_in]
        offs = [0]
        for s in sizes:
            offs.append(offs[-1] + s)
        total = offs[-1]
        dev = flat.buffer.device
        with self._timer("reduce.topk", verbosity=2):
            flat_values = torch.empty(total, device=dev)
            flat_positions = torch.empty(total, device=dev, dtype=torch.int32)
            for i, k in enumerate(sizes):
                t = flat[i].view(-1)
                _, pos = torch.topk(t.abs(), k, sorted=False)
                flat_values[offs[i]: offs[i + 1]] = t[pos]
                flat_positions[offs[i]: offs[i + 1]] = pos
        with self._timer("reduce.set_memory", verbosity=2):
            self._memory.copy_(flat.buffer)
            starts = torch.tensor(flat._start_idx, device=dev, dtype=torch.int64)
            seg = torch.repeat_interleave(starts, torch.tensor(sizes, device=dev))
            global_pos = seg + flat_positions.long()
            self._memory[global_pos] = 0.0
        with self._timer("reduce.gather", verbosity=2):
            all_values = self._all_gather(flat_values)
            all_positions = self._all_gather(flat_positions)
        bits = n_bits(flat_values) + n_bits(flat_positions)
        self.last_wire_bits = bits
        with self._timer("reduce.combine", verbosity=2):
            out = torch.zeros_like(flat.buffer)
            for pos, val in zip(all_positions, all_values):
                out.index_add_(0, seg + pos.long(), val / self.n_workers)
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


class TopKReducerRatio(TopKReducer):
    """Layer-wise Top-K with K_l = max(1, int(ratio * numel)) (reducer.py:1228-1309)."""

    def __init__(self, device, timer=None, compression=1 / 100, **kw):
        super().__init__(device, timer, K=0, **kw)
        self._compression = compression

    def _top_size(self, numel):
        return max(1, int(self._compression * numel))


class GlobalTopKReducer(Reducer):
    """Top-K over the whole flat gradient with error feedback (reducer.py:1312-1380).

    Default result: mean of the workers' sparse contributions.  ``reference_compat=True`` reproduces
    the reference, which adds the gathered values onto the full local gradient and divides by W again
    (reducer.py:1366-1375)."""

    def __init__(self, device, timer=None, K=10000, **kw):
        super().__init__(device, timer, **kw)
        self._K = K
        self._memory = None

    def _top_size(self, numel):
        return min(numel, self._K)

    def reduce(self, grad_in, grad_out):
        with self._timer("reduce.flat_pack"):
            flat = TensorBuffer(grad_in)
        if self._memory is None:
            self._memory = torch.zeros_like(flat.buffer)
        else:
            flat.buffer.add_(self._memory)
        k = self._top_size(flat.buffer.numel())
        with self._timer("reduce.topk", verbosity=2):
            _, positions = torch.topk(flat.buffer.abs(), k, sorted=False)
            values = flat.buffer[positions].contiguous()
        with self._timer("reduce.set_memory", verbosity=2):
            self._memory.copy_(flat.buffer)
            self._memory[positions] = 0.0
        with self._timer("reduce.gather", verbosity=2):
            all_values = self._all_gather(values)
            all_positions = self._all_gather(positions)
        bits = n_bits(values) + n_bits(positions)
        self.last_wire_bits = bits
        with self._timer("reduce.combine", verbosity=2):
            if self._compat:
                out = flat.buffer.clone()
                for pos, val in zip(all_positions, all_values):
                    out.index_add_(0, pos, val / self.n_workers)
                out.mul_(1.0 / self.n_workers)
            else:
                out = torch.zeros_like(flat.buffer)
                for pos, val in zip(all_positions, all_values):
                    out.index_add_(0, pos, val / self.n_workers)
        with self._timer("reduce.setgrad", verbosity=2):
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


class GlobalTopKReducerRatio(GlobalTopKReducer):
    """Global Top-K with K = max(1, int(ratio * N)) (reducer.py:1383-1451)."""

    def __init__(self, device, timer=None, compression=1 / 100, **kw):
        super().__init__(device, timer, K=0, **kw)
        self._compression = compression

    def _top_size(self, numel):
        return max(1, int(self._compression * numel))
