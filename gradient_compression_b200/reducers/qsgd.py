"""Quantised reducers (reference: reducer.py:176-554, 769-1141).

All-reduce-compatible family (QSGD-MaxNorm and relatives): every worker normalises by the same
global norm, so the signed integer levels can be *summed*.  All-gather family (QSGD, QSGD-WEC,
TernGrad, NUQSGD-Mod): each worker's own norm, payloads gathered and averaged after decoding.
"""
from __future__ import annotations

import torch

from .. import compressors as C
from .. import ops
from .base import Reducer, TensorBuffer, n_bits


def _write_flat(values, template, grad_out):
    """grad_out[i][:] = values[slice i] using the template's layout."""
    if template.is_view and values.data_ptr() != template.buffer.data_ptr():
        template.buffer.copy_(values)
    elif not template.is_view:
        template.buffer = values
    template.scatter_to(grad_out)


class _MaxNormReducer(Reducer):
    """Shared body of the all-reduce-compatible quantised reducers."""

    compressor_cls = C.QSGDMaxNormCompressor
    norm_kind = "absmax"      # or "l2"
    error_feedback = False
    fused_capable = False

    def __init__(self, device, timer=None, quantization_level=8, **kw):
        super().__init__(device, timer, **kw)
        self._quantization_level = quantization_level
        self._noise = C.NoiseSource(self._seed, self.rank)
        self._compressor = self.compressor_cls(self._device, quantization_level, noise=self._noise)
        self._memory = None

    def _local_norm(self, flat):
        if self.norm_kind == "l2":
            return torch.norm(flat).reshape(1)
        return ops.absmax(flat)

    def _wire_bits(self, n):
        mb, pb = ops.packed_sizes(n, self._quantization_level)
        return 32 + 8 * (mb + pb)

    def reduce(self, grad_in, grad_out):
        with self._timer("reduce.flat_pack"):
            flat = TensorBuffer(grad_in)
        if self.error_feedback:
            with self._timer("reduce.memory", verbosity=2):
                if self._memory is None:
                    self._memory = torch.zeros_like(flat.buffer)
                else:
                    flat.buffer.add_(self._memory)
        if self._use_fused() and not self.error_feedback:
            from ..parallel import engine as fused
            bits = fused.qsgd_maxnorm(self, flat, grad_out)
            if bits is not None:
                return bits
        with self._timer("reduce.norm", verbosity=2):
            max_norm = self._global_max(self._local_norm(flat.buffer))
        with self._timer("reduce.compress", verbosity=2):
            levels = self._compressor.compress(max_norm, flat.buffer)
        if self.error_feedback:
            with self._timer("reduce.set_memory", verbosity=2):
                local = self._compressor.decompress(max_norm, levels) if not self._compat else levels.float()
                torch.sub(flat.buffer, local, out=self._memory)
        with self._timer("reduce.reduce.vector", verbosity=2):
            wire_levels, levels = levels, self._all_reduce_levels(levels)
        bits = 32 + n_bits(wire_levels)
        self.last_wire_bits = self._wire_bits(flat.buffer.numel())
        with self._timer("reduce.decompress", verbosity=2):
            values = self._compressor.decompress(max_norm, levels, self.n_workers)
        with self._timer("reduce.setgrad", verbosity=2):
            _write_flat(values, flat, grad_out)
        return bits

    def state_dict(self):
        sd = {"noise": self._noise.state_dict()}
        if self._memory is not None:
            sd["memory"] = self._memory
        return sd

    def load_state_dict(self, sd):
        self._noise.load_state_dict(sd["noise"])
        if "memory" in sd:
            self._memory = sd["memory"].to(self._device).clone()


class QSGDMaxNormReducer(_MaxNormReducer):
    """QSGD-MN: global max-norm, stochastic b-bit levels, summed by all-reduce (reducer.py:498-554)."""

    fused_capable = True


class NUQSGDMaxNormReducer(_MaxNormReducer):
    """Power-of-two levels, shared maximum of the workers' L2 norms (reducer.py:829-885)."""

    compressor_cls = C.NUQSGDMaxNormCompressor
    norm_kind = "l2"


class QSGDMaxNormBiasedReducer(_MaxNormReducer):
    """Deterministic truncation (reducer.py:888-944)."""

    compressor_cls = C.QSGDMaxNormBiasedCompressor


class QSGDMaxNormBiasedMemoryReducer(_MaxNormReducer):
    """Truncation with error memory (reducer.py:947-1013).  memory = grad - dequantised(levels); with
    ``reference_compat`` the reference's ``grad - integer levels`` (reducer.py:987) is reproduced."""

    compressor_cls = C.QSGDMaxNormBiasedCompressor
    error_feedback = True


class NUQSGDMaxNormBiasedReducer(_MaxNormReducer):
    """Deterministic power-of-two floor (reducer.py:1016-1072)."""

    compressor_cls = C.NUQSGDMaxNormBiasedCompressor
    norm_kind = "l2"


class NUQSGDMaxNormBiasedMemoryReducer(_MaxNormReducer):
    """Same with error memory (reducer.py:1075-1141)."""

    compressor_cls = C.NUQSGDMaxNormBiasedCompressor
    norm_kind = "l2"
    error_feedback = True


# ------------------------------------------------------------------------- all-gather family
class _GatherReducer(Reducer):
    """Each worker encodes with its own norm; payload arrays are all-gathered and decoded."""

    compressor_cls = None
    takes_level = True

    def __init__(self, device, timer=None, quantization_level=8, **kw):
        super().__init__(device, timer, **kw)
        self._quantization_level = quantization_level
        self._noise = C.NoiseSource(self._seed, self.rank)
        args = (quantization_level,) if self.takes_level else ()
        self._compressor = self.compressor_cls(self._device, *args, noise=self._noise)

    def reduce(self, grad_in, grad_out):
        with self._timer("reduce.flat_pack"):
            flat = TensorBuffer(grad_in)
        with self._timer("reduce.compress", verbosity=2):
            parts = self._compressor.compress(flat.buffer)
            parts = [p if torch.is_tensor(p) else torch.tensor(p) for p in parts]
            parts = [p.reshape(1) if p.dim() == 0 else p for p in parts]
        with self._timer("reduce.gather", verbosity=2):
            gathered = [self._all_gather(p.to(flat.buffer.device)) for p in parts]
        bits = sum(n_bits(p) for p in parts)
        self.last_wire_bits = bits
        with self._timer("reduce.decompress", verbosity=2):
            acc = torch.zeros_like(flat.buffer)
            for w in range(self.n_workers):
                pw = [g[w] for g in gathered]
                pw = [p.reshape(()) if p.numel() == 1 and p.dtype.is_floating_point else p for p in pw]
                acc.add_(self._compressor.decompress(*pw).to(acc.dtype), alpha=1.0 / self.n_workers)
        with self._timer("reduce.setgrad", verbosity=2):
            _write_flat(acc, flat, grad_out)
        return bits


class QSGDWECReducer(_GatherReducer):
    """QSGD without Elias coding; norm, sign and xi gathered separately (reducer.py:246-308)."""

    compressor_cls = C.QSGDWECCompressor


class QSGDWECModReducer(_GatherReducer):
    """sign * xi fused into one array (reducer.py:311-368)."""

    compressor_cls = C.QSGDWECModCompressor


class TernGradReducer(_GatherReducer):
    """TernGrad (reducer.py:371-434)."""

    compressor_cls = C.TernGradCompressor
    takes_level = False

    def __init__(self, device, timer=None, **kw):
        super().__init__(device, timer, quantization_level=1, **kw)


class TernGradModReducer(TernGradReducer):
    """TernGrad with sign * b fused (reducer.py:437-495)."""

    compressor_cls = C.TernGradModCompressor


class NUQSGDModReducer(_GatherReducer):
    """Non-uniform QSGD with per-worker L2 norm (reducer.py:769-826)."""

    compressor_cls = C.NUQSGDModCompressor


class QSGDReducer(Reducer):
    """QSGD with Elias-omega coded, variable-length int64 payloads: size exchange, then a padded
    all-gather (reducer.py:176-243)."""

    def __init__(self, device, timer=None, quantization_level=8, **kw):
        super().__init__(device, timer, **kw)
        self._noise = C.NoiseSource(self._seed, self.rank)
        self._compressor = C.QSGDCompressor(self._device, quantization_level, noise=self._noise)

    def reduce(self, grad_in, grad_out):
        with self._timer("reduce.flat_pack"):
            flat = TensorBuffer(grad_in)
        dev = flat.buffer.device
        with self._timer("reduce.compress", verbosity=2):
            words, _ = self._compressor.compress(flat.buffer)
            words = words.to(dev)
            size = torch.tensor([words.numel()], dtype=torch.int64, device=dev)
        with self._timer("reduce.gather", verbosity=2):
            sizes = self._all_gather(size)
            max_size = max(int(s) for s in sizes)
            padded = torch.zeros(max_size, dtype=torch.int64, device=dev)
            padded[: words.numel()] = words
            gathered = self._all_gather(padded)
        bits = n_bits(size) + n_bits(padded)
        self.last_wire_bits = bits
        with self._timer("reduce.decompress", verbosity=2):
            acc = torch.zeros_like(flat.buffer)
            for sz, g in zip(sizes, gathered):
                acc.add_(self._compressor.decompress(g, int(sz)).to(dev), alpha=1.0 / self.n_workers)
        with self._timer("reduce.setgrad", verbosity=2):
            _write_flat(acc, flat, grad_out)
        return bits


class QSGDBPReducer(_GatherReducer):
    """QSGD + variable-width bit packing, all-gathered (reducer.py:557-623, commented out there)."""

    compressor_cls = C.QSGDBPCompressor

    def reduce(self, grad_in, grad_out):
        with self._timer("reduce.flat_pack"):
            flat = TensorBuffer(grad_in)
        dev, n = flat.buffer.device, flat.buffer.numel()
        norm, sign_p, xi_p, _ = self._compressor.compress(flat.buffer)
        sizes = torch.tensor([sign_p.numel(), xi_p.numel()], dtype=torch.int64, device=dev)
        all_sizes = self._all_gather(sizes)
        cap = [max(int(s[i]) for s in all_sizes) for i in (0, 1)]
        payload = torch.zeros(cap[0] + cap[1], dtype=torch.int32, device=dev)
        payload[: sign_p.numel()] = sign_p
        payload[cap[0]: cap[0] + xi_p.numel()] = xi_p
        norms = self._all_gather(norm.reshape(1).to(dev))
        gathered = self._all_gather(payload)
        bits = n_bits(sizes) + n_bits(payload) + 32
        self.last_wire_bits = bits
        acc = torch.zeros_like(flat.buffer)
        for nm, sz, g in zip(norms, all_sizes, gathered):
            dec = self._compressor.decompress(nm.reshape(()), g[: int(sz[0])], g[cap[0]: cap[0] + int(sz[1])], n)
            acc.add_(dec.to(dev), alpha=1.0 / self.n_workers)
        _write_flat(acc, flat, grad_out)
        return bits


class QSGDBPAllReducer(_MaxNormReducer):
    """QSGD-MaxNorm with byte-packed levels summed as int64 words (reducer.py:626-694, commented out
    there).  Byte lanes must not overflow: requires W * (2**b - 1) <= 127; checked at construction."""

    compressor_cls = C.QSGDBPAllReduceCompressor

    def __init__(self, device, timer=None, quantization_level=4, **kw):
        super().__init__(device, timer, quantization_level=quantization_level, **kw)
        if self.n_workers * ((1 << quantization_level) - 1) > 127:
            raise ValueError("byte-packed all-reduce would overflow: need W * (2**b - 1) <= 127")

    def reduce(self, grad_in, grad_out):
        flat = TensorBuffer(grad_in)
        max_norm = self._global_max(self._local_norm(flat.buffer))
        levels = C.QSGDMaxNormCompressor.compress(self._compressor, max_norm, flat.buffer).to(torch.int32)
        # bias every lane by +s*1 so lanes stay non-negative and carries never cross byte boundaries
        s = (1 << self._quantization_level) - 1
        packed = ops.bytepack(levels + s)
        self._all_reduce(packed)
        summed = ops.byteunpack(packed, levels.numel()) & 0xFF
        summed = summed - s * self.n_workers
        bits = 32 + n_bits(packed)
        self.last_wire_bits = bits
        values = ops.dequantize_levels(summed.to(torch.int32), max_norm, s, self.n_workers)
        _write_flat(values, flat, grad_out)
        return bits
