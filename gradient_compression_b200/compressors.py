"""Gradient codecs (reference: compressors.py).

Every class keeps the reference's name, constructor arguments and ``compress`` / ``decompress``
signatures, but is built on the native ops of this package: one fused kernel (or its C++ oracle on
CPU) per call instead of ~12 elementwise torch kernels, and counter-based Philox noise instead of
``torch.bernoulli`` so that a CPU run and a GPU run of the same (seed, rank, step) agree bit for bit.

Level containers follow the reference's dtype rule (int8 below 8 bits, int32 from 8 bits,
compressors.py:294-297) because these arrays are what ``torch.distributed`` all-reduces on the
collective backend.  The fused backend never materialises them: it moves the packed wire layout.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from . import ops
from .ops import philox


class NoiseSource:
    """(seed, rank, step) triple that names a Philox stream; ``next_step`` advances once per call."""

    def __init__(self, seed=0, rank=None):
        if rank is None:
            rank = dist.get_rank() if dist.is_available() and dist.is_initialized() else 0
        self.seed, self.rank, self.step = int(seed), int(rank), 0

    def next_step(self):
        s = self.step
        self.step += 1
        return s

    def stream(self, purpose):
        return philox.stream_id(self.rank, purpose)

    def state_dict(self):
        return {"seed": self.seed, "rank": self.rank, "step": self.step}

    def load_state_dict(self, sd):
        # the rank stays the live worker's: a state saved by another worker must not make two workers draw the same
        # rounding-noise stream
        self.seed, self.step = int(sd["seed"]), int(sd["step"])


def _container(bits, max_level=None):
    """int8 for codes of fewer than 8 bits whose largest level fits it (the non-uniform codecs reach 2**b = 128 at 7
    bits, one past int8; the reference stores that in int8 and wraps: compressors.py:466), int32 otherwise."""
    if max_level is None:
        max_level = _levels(bits)
    return torch.int8 if bits < 8 and max_level <= 127 else torch.int32


def _levels(s):
    return (1 << s) - 1


class _Codec:
    def __init__(self, device, noise=None):
        self._device = device
        self._noise = noise or NoiseSource()


class NoneCompressor(_Codec):
    """Identity codec (compressors.py:10-27)."""

    def compress(self, tensor):
        return tensor, torch.tensor(tensor.size(), device=self._device)

    def decompress(self, compressed_tensor, compressed_tensor_size):
        return compressed_tensor[: int(compressed_tensor_size)]


class QSGDCompressor(_Codec):
    """QSGD with L2 norm and Elias-omega coding into int64 words (compressors.py:30-149).

    The coder is native C++ (the reference builds Python strings per element).  Levels are coded as
    |q| + 1 so that zero survives a round trip.
    """

    def __init__(self, device, quantization_level=8, noise=None):
        super().__init__(device, noise)
        self._quantization_level = quantization_level

    def compress(self, tensor):
        s = _levels(self._quantization_level)
        flat = tensor.contiguous().view(-1).float()
        norm = torch.norm(flat)
        q = ops.quantize_levels(flat, norm, s, self._noise.seed, self._noise.stream(philox.PURPOSE_ROUND),
                                self._noise.next_step())
        words = ops.packing.elias_encode(q, float(norm) / s).to(self._device)
        return words, torch.tensor(words.size(), device=self._device)

    def decompress(self, compressed_tensor, compressed_tensor_size):
        norm_over_s, q = ops.packing.elias_decode(compressed_tensor[: int(compressed_tensor_size)])
        return norm_over_s * q.to(torch.float32)


class QSGDWECCompressor(_Codec):
    """QSGD without Elias coding: (norm / s, sign, xi) as three arrays (compressors.py:152-189)."""

    def __init__(self, device, quantization_level=8, noise=None):
        super().__init__(device, noise)
        self._quantization_level = quantization_level
        self._dtype = _container(quantization_level)

    def _q(self, tensor):
        s = _levels(self._quantization_level)
        flat = tensor.contiguous().view(-1)
        norm = ops.absmax(flat)
        q = ops.quantize_levels(flat, norm, s, self._noise.seed, self._noise.stream(philox.PURPOSE_ROUND),
                                self._noise.next_step())
        return norm.reshape(()) / s, q

    def compress(self, tensor):
        norm, q = self._q(tensor)
        return norm, torch.sign(q).to(torch.int8), q.abs().to(self._dtype)

    def decompress(self, norm, sign_array, xi_array):
        return norm * sign_array * xi_array


class QSGDWECModCompressor(QSGDWECCompressor):
    """Same with sign * xi fused into one array (compressors.py:192-230)."""

    def compress(self, tensor):
        norm, q = self._q(tensor)
        return norm, q.to(self._dtype)

    def decompress(self, norm, sign_xi_array):
        return norm * sign_xi_array


class TernGradCompressor(_Codec):
    """TernGrad: scaler = max |g|, b ~ Bernoulli(|g| / scaler) (compressors.py:233-254)."""

    def _q(self, tensor):
        flat = tensor.contiguous().view(-1)
        scaler = ops.absmax(flat)
        q = ops.quantize_levels(flat, scaler, 1, self._noise.seed, self._noise.stream(philox.PURPOSE_ROUND),
                                self._noise.next_step(), dtype=torch.int8)
        return scaler.reshape(()), q

    def compress(self, tensor):
        scaler, q = self._q(tensor)
        return scaler, torch.sign(q).to(torch.int8), q.abs()

    def decompress(self, scaler, sign_array, b_array):
        return scaler * sign_array * b_array


class TernGradModCompressor(TernGradCompressor):
    """TernGrad with sign * b fused (compressors.py:257-280)."""

    def compress(self, tensor):
        return self._q(tensor)

    def decompress(self, scaler, sign_b_array):
        return scaler * sign_b_array


class QSGDMaxNormCompressor(_Codec):
    """QSGD with a supplied (global max) norm: levels sum across workers (compressors.py:283-321)."""

    _mode = ops.MODE_STOCHASTIC

    def __init__(self, device, quantization_level=8, noise=None):
        super().__init__(device, noise)
        self._quantization_level = quantization_level
        self._dtype = _container(quantization_level)

    def _s(self):
        return _levels(self._quantization_level)

    def compress(self, norm, tensor):
        flat = tensor.contiguous().view(-1)
        return ops.quantize_levels(flat, norm, self._s(), self._noise.seed, self._noise.stream(philox.PURPOSE_ROUND),
                                   self._noise.next_step(), mode=self._mode, dtype=self._dtype)

    def decompress(self, norm, sign_xi_array, world=1):
        return ops.dequantize_levels(sign_xi_array, norm, self._s(), world)


class GlobalRandKMaxNormCompressor(QSGDMaxNormCompressor):
    """Identical codec applied to the K gathered coordinates (compressors.py:419-456)."""


class QSGDMaxNormBiasedCompressor(QSGDMaxNormCompressor):
    """Deterministic truncation toward zero, no random bits (compressors.py:546-573)."""

    _mode = ops.MODE_BIASED


class NUQSGDMaxNormCompressor(QSGDMaxNormCompressor):
    """Power-of-two levels with s = 2**b and a supplied norm (compressors.py:502-543)."""

    _mode = ops.MODE_NU

    def __init__(self, device, quantization_level=8, noise=None):
        super().__init__(device, quantization_level, noise)
        self._dtype = _container(quantization_level, 1 << quantization_level)

    def _s(self):
        return 1 << self._quantization_level


class NUQSGDMaxNormBiasedCompressor(NUQSGDMaxNormCompressor):
    """Deterministic floor to a power of two (compressors.py:576-609)."""

    _mode = ops.MODE_NU_BIASED


class NUQSGDModCompressor(_Codec):
    """Non-uniform QSGD with the tensor's own L2 norm (compressors.py:459-499)."""

    def __init__(self, device, quantization_level=8, noise=None):
        super().__init__(device, noise)
        self._quantization_level = quantization_level
        self._dtype = _container(quantization_level, 1 << quantization_level)

    def compress(self, tensor):
        s = 1 << self._quantization_level
        flat = tensor.contiguous().view(-1)
        norm = torch.norm(flat)
        q = ops.quantize_levels(flat, norm, s, self._noise.seed, self._noise.stream(philox.PURPOSE_ROUND),
                                self._noise.next_step(), mode=ops.MODE_NU, dtype=self._dtype)
        return norm / s, q

    def decompress(self, norm, sign_h_array):
        return norm * sign_h_array


class QSGDMaxNormTwoScaleCompressor(_Codec):
    """Two-scale QSGD-MaxNorm (compressors.py:612-680).

    ``compress_lower`` and ``compress_higher`` draw independent rounding noise (separate Philox
    streams of the same step); the mask says where the *rounded* high-scale level still fits the
    low-scale range, so after the cross-worker AND every transmitted value is bounded by s_lower.
    """

    def __init__(self, device, lower_quantization_level=6, higher_quantization_level=10, noise=None):
        super().__init__(device, noise)
        self._lower_quantization_level = lower_quantization_level
        self._higher_quantization_level = higher_quantization_level
        self._dtype = _container(lower_quantization_level)
        self._step = None

    def begin(self):
        """Pin both scales of one reduce() call to the same Philox step."""
        self._step = self._noise.next_step()
        return self._step

    def compress_lower(self, norm, tensor):
        step = self._step if self._step is not None else self._noise.next_step()
        return ops.quantize_levels(tensor.contiguous().view(-1), norm, _levels(self._lower_quantization_level),
                                   self._noise.seed, self._noise.stream(philox.PURPOSE_ROUND), step,
                                   dtype=self._dtype)

    def compress_higher(self, norm, tensor):
        step = self._step if self._step is not None else self._noise.next_step()
        s_lo = _levels(self._lower_quantization_level)
        q = ops.quantize_levels(tensor.contiguous().view(-1), norm, _levels(self._higher_quantization_level),
                                self._noise.seed, self._noise.stream(philox.PURPOSE_ROUND_HI), step,
                                dtype=torch.int32)
        mask = (q.abs() <= s_lo).to(torch.int8)
        return q.to(self._dtype), mask

    def decompress(self, norm, sign_xi_array, higher_resolution_mask, world=1):
        s_lo, s_hi = _levels(self._lower_quantization_level), _levels(self._higher_quantization_level)
        # both candidates come from the native dequantiser so CPU, GPU and the fused kernel agree bit for bit
        fine = ops.dequantize_levels(sign_xi_array, norm, s_hi, world)
        coarse = ops.dequantize_levels(sign_xi_array, norm, s_lo, world)
        return torch.where(higher_resolution_mask.bool(), fine, coarse)


class GlobalRandKMaxNormTwoScaleCompressor(QSGDMaxNormTwoScaleCompressor):
    """Identical two-scale codec for the K gathered coordinates (compressors.py:683-751)."""


class QSGDMaxNormMultiScaleCompressor(_Codec):
    """L-scale generalisation (compressors.py:754-826) without the reference's L x N fp32 cache:
    a level is recomputed from (norm, tensor, step) when needed -- Philox makes that deterministic."""

    def __init__(self, device, quantization_levels=None, noise=None):
        super().__init__(device, noise)
        levels = sorted(quantization_levels or [6, 10])
        self._quantization_levels = levels
        self._dtype = _container(levels[0])
        self._ctx = None

    def _level(self, ind):
        norm, flat, step = self._ctx
        return ops.quantize_levels(flat, norm, _levels(self._quantization_levels[ind]), self._noise.seed,
                                   self._noise.stream(philox.PURPOSE_LEVEL0 + ind), step)

    def compress_mask(self, norm, tensor):
        """int8 index of the finest scale whose rounded level fits into the coarsest scale's range."""
        flat = tensor.contiguous().view(-1)
        self._ctx = (norm, flat, self._noise.next_step())
        max_val = _levels(self._quantization_levels[0])
        mask = torch.zeros(flat.numel(), dtype=torch.int8, device=flat.device)
        for ind in range(1, len(self._quantization_levels)):
            mask[self._level(ind).abs() <= max_val] = ind
        return mask

    def compress(self, resolution_mask):
        out = torch.zeros(resolution_mask.numel(), dtype=torch.int32, device=resolution_mask.device)
        for ind in range(len(self._quantization_levels)):
            sel = resolution_mask == ind
            out[sel] = self._level(ind)[sel]
        return out.to(self._dtype)

    def decompress(self, norm, sign_xi_array, resolution_mask, world=1):
        out = ops.dequantize_levels(sign_xi_array, norm, _levels(self._quantization_levels[0]), world)
        for ind in range(1, len(self._quantization_levels)):
            cand = ops.dequantize_levels(sign_xi_array, norm, _levels(self._quantization_levels[ind]), world)
            out = torch.where(resolution_mask == ind, cand, out)
        return out


class QSGDBPCompressor(_Codec):
    """QSGD with the variable-width bit packer of the reference's extension (compressors.py:327-378,
    commented out there).  Sign is coded 0/1, both arrays go through ``ops.varpack``."""

    def __init__(self, device, quantization_level=8, noise=None):
        super().__init__(device, noise)
        self._quantization_level = quantization_level

    def compress(self, tensor):
        s = _levels(self._quantization_level)
        flat = tensor.contiguous().view(-1)
        norm = torch.norm(flat)
        q = ops.quantize_levels(flat, norm, s, self._noise.seed, self._noise.stream(philox.PURPOSE_ROUND),
                                self._noise.next_step())
        sign_packed = ops.varpack((q < 0).to(torch.int32))
        xi_packed = ops.varpack(q.abs())
        return norm / s, sign_packed, xi_packed, flat.numel()

    def decompress(self, norm, sign_packed, xi_packed, size):
        sign = 1 - 2 * ops.varunpack(sign_packed, size)
        return norm * (sign * ops.varunpack(xi_packed, size))


class QSGDBPAllReduceCompressor(QSGDMaxNormCompressor):
    """QSGD-MaxNorm levels byte-packed eight per int64 (compressors.py:381-416, commented out there).

    A sum of packed words only stays meaningful while no byte overflows; kept for API parity -- the
    fused backend's packed reduce with int32 accumulators is the supported way to do this."""

    def compress(self, norm, tensor):
        q = super().compress(norm, tensor)
        return ops.bytepack(q.to(torch.int32)), q.numel()

    def decompress(self, norm, packed, size, world=1):
        q = ops.byteunpack(packed, size)
        return ops.dequantize_levels(q, norm, self._s(), world)


__all__ = [name for name in dir() if name.endswith("Compressor")] + ["NoiseSource"]
