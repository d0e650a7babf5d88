"""Two-scale and multi-scale QSGD-MaxNorm reducers (reference: reducer.py:1454-1531, 1636-1715)."""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import compressors as C
from .. import ops
from .base import Reducer, TensorBuffer, n_bits
from .qsgd import _write_flat


class QSGDMaxNormTwoScaleReducer(Reducer):
    """QSGD-MN-TS: both scales are rounded independently; a cross-worker AND of the "high-scale level
    fits the low range" mask picks per element which scale every worker sends; levels are summed."""

    fused_capable = True
    compressor_cls = C.QSGDMaxNormTwoScaleCompressor

    def __init__(self, device, timer=None, lower_quantization_level=6, higher_quantization_level=10, **kw):
        super().__init__(device, timer, **kw)
        self._lower_quantization_level = lower_quantization_level
        self._higher_quantization_level = higher_quantization_level
        self._noise = C.NoiseSource(self._seed, self.rank)
        self._compressor = self.compressor_cls(self._device, lower_quantization_level, higher_quantization_level,
                                               noise=self._noise)

    def _two_scale(self, values):
        """values: 1-D fp32 -> (mean over workers, bits) for this vector."""
        with self._timer("reduce.norm", verbosity=2):
            max_norm = self._global_max(ops.absmax(values))
        with self._timer("reduce.compress", verbosity=2):
            self._compressor.begin()
            lo = self._compressor.compress_lower(max_norm, values)
            hi, mask = self._compressor.compress_higher(max_norm, values)
            if self.n_workers > 1:
                # AND across workers; MIN equals the reference's PRODUCT on 0/1 masks
                dist.all_reduce(mask, op=dist.ReduceOp.MIN, group=self._group)
            levels = torch.where(mask.bool(), hi, lo)
        with self._timer("reduce.reduce.vector", verbosity=2):
            wire_levels, levels = levels, self._all_reduce_levels(levels)
        bits = 32 + n_bits(mask) + n_bits(wire_levels)
        mb, pb = ops.packed_sizes(values.numel(), self._lower_quantization_level)
        self.last_wire_bits = 32 + 8 * (mb + 2 * pb)
        with self._timer("reduce.decompress", verbosity=2):
            out = self._compressor.decompress(max_norm, levels, mask, self.n_workers)
        return out, bits

    def reduce(self, grad_in, grad_out):
        with self._timer("reduce.flat_pack"):
            flat = TensorBuffer(grad_in)
        if self._use_fused():
            from ..parallel import engine as fused
            bits = fused.qsgd_twoscale(self, flat, grad_out)
            if bits is not None:
                return bits
        values, bits = self._two_scale(flat.buffer)
        with self._timer("reduce.setgrad", verbosity=2):
            _write_flat(values, flat, grad_out)
        return bits

    def state_dict(self):
        return {"noise": self._noise.state_dict()}

    def load_state_dict(self, sd):
        self._noise.load_state_dict(sd["noise"])


class QSGDMaxNormMultiScaleReducer(Reducer):
    """L scales: per element the finest scale index that fits on every worker (MIN all-reduce of the
    int8 index array), then the agreed scale's levels are summed (reducer.py:1636-1715)."""

    fused_capable = True

    def __init__(self, device, timer=None, quantization_levels=None, **kw):
        super().__init__(device, timer, **kw)
        self._quantization_levels = sorted(quantization_levels or [6, 10])
        self._noise = C.NoiseSource(self._seed, self.rank)
        self._compressor = C.QSGDMaxNormMultiScaleCompressor(self._device, list(self._quantization_levels),
                                                             noise=self._noise)

    def reduce(self, grad_in, grad_out):
        with self._timer("reduce.flat_pack"):
            flat = TensorBuffer(grad_in)
        if self._use_fused():
            from ..parallel import engine as fused
            bits = fused.qsgd_multiscale(self, flat, grad_out)
            if bits is not None:
                return bits
        with self._timer("reduce.norm", verbosity=2):
            max_norm = self._global_max(ops.absmax(flat.buffer))
        with self._timer("reduce.compress", verbosity=2):
            mask = self._compressor.compress_mask(max_norm, flat.buffer)
            if self.n_workers > 1:
                dist.all_reduce(mask, op=dist.ReduceOp.MIN, group=self._group)
            levels = self._compressor.compress(mask)
        with self._timer("reduce.reduce.vector", verbosity=2):
            wire_levels, levels = levels, self._all_reduce_levels(levels)
        bits = 32 + n_bits(mask) + n_bits(wire_levels)
        self.last_wire_bits = bits
        with self._timer("reduce.decompress", verbosity=2):
            values = self._compressor.decompress(max_norm, levels, mask, self.n_workers)
        with self._timer("reduce.setgrad", verbosity=2):
            _write_flat(values, flat, grad_out)
        return bits

    def state_dict(self):
        return {"noise": self._noise.state_dict()}

    def load_state_dict(self, sd):
        self._noise.load_state_dict(sd["noise"])
