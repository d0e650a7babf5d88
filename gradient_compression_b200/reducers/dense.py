"""Uncompressed reducers (reference: reducer.py:71-173)."""
from __future__ import annotations

import torch

from .base import Reducer, TensorBuffer, n_bits


class NoneAllReducer(Reducer):
    """AllReduce-SGD: sum the flat fp32 gradient over workers and divide by W (reducer.py:140-173)."""

    fused_capable = True

    def reduce(self, grad_in, grad_out):
        with self._timer("reduce.flat_pack"):
            flat = TensorBuffer(grad_in)
        bits = n_bits(flat.buffer)
        self.last_wire_bits = bits
        with self._timer("reduce.allreduce", verbosity=2):
            if self._use_fused():
                from ..parallel import engine as fused
                if fused.allreduce_mean(self, flat, grad_out):
                    return bits
            self._all_reduce(flat.buffer)
            if self.n_workers > 1:
                flat.buffer.mul_(1.0 / self.n_workers)
        with self._timer("reduce.setgrad", verbosity=2):
            flat.scatter_to(grad_out)
        return bits


class NoneReducer(Reducer):
    """All-gather of the uncompressed gradients, then average (reducer.py:71-137).

    The reference stages floats through int64 buffers, which zeroes them; here the payload keeps its
    dtype.  The size exchange is kept so the wire pattern (size, then padded payload) is the same."""

    def reduce(self, grad_in, grad_out):
        with self._timer("reduce.flat_pack"):
            flat = TensorBuffer(grad_in)
        size = torch.tensor([flat.buffer.numel()], dtype=torch.int64, device=flat.buffer.device)
        with self._timer("reduce.gather", verbosity=2):
            sizes = self._all_gather(size)
            max_size = int(max(int(s) for s in sizes))
            payload = flat.buffer
            if payload.numel() < max_size:
                payload = torch.cat([payload, payload.new_zeros(max_size - payload.numel())])
            gathered = self._all_gather(payload)
        bits = n_bits(size) + n_bits(payload)
        self.last_wire_bits = bits
        with self._timer("reduce.average", verbosity=2):
            acc = torch.zeros_like(flat.buffer)
            for sz, g in zip(sizes, gathered):
                acc.add_(g[: int(sz)], alpha=1.0 / self.n_workers)
            if flat.is_view:
                flat.buffer.copy_(acc)
            else:
                flat.buffer = acc
        with self._timer("reduce.setgrad", verbosity=2):
            flat.scatter_to(grad_out)
        return bits
