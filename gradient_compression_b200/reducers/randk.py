"""Global Rand-K reducers with a shared-seed index set (reference: reducer.py:697-766, 1534-1633).

Index sets come from a keyed point-wise permutation of [0, N) (``ops.randk_indices``): step t uses
positions [t*K, (t+1)*K) of the permutation, so every coordinate is visited exactly once per pass
and every worker derives the same K indices on its own device -- the reference builds a CPU
``randperm(N)`` (re-seeding every RNG of the process) and uploads K indices each step.

``unselected`` says what the coordinates outside the index set become: ``"local"`` = the worker's
own gradient / W (what the reference does, reducer.py:754-761), ``"zero"`` = 0.
"""
from __future__ import annotations

from .. import compressors as C
from .. import ops
from .base import Reducer, TensorBuffer, n_bits
from .multiscale import QSGDMaxNormTwoScaleReducer


class _IndexQueue:
    def __init__(self, seed, K, reshuffle_each_pass=False):
        self.seed, self.K, self.reshuffle = int(seed), int(K), reshuffle_each_pass
        self.position, self.npass = 0, 0

    def next_window(self, n):
        """-> (start, k, pass) of this step's window of the permutation of [0, n)."""
        if self.position >= n:
            self.position = 0
            self.npass += 1
        start = self.position
        k = min(self.K, n - start)
        self.position += k
        return start, k, (self.npass if self.reshuffle else 0)

    def state_dict(self):
        return {"position": self.position, "npass": self.npass}

    def load_state_dict(self, sd):
        self.position, self.npass = int(sd["position"]), int(sd["npass"])


class GlobalRandKMaxNormReducer(Reducer):
    """GRandK-MN: QSGD-MaxNorm on K shared random coordinates per step."""

    fused_capable = True

    def __init__(self, device, timer=None, seed=0, K=10000, quantization_level=8, unselected="local",
                 reshuffle_each_pass=False, **kw):
        super().__init__(device, timer, seed=seed, **kw)
        self._quantization_level = quantization_level
        self._K = K
        self._unselected = unselected
        self._queue = _IndexQueue(seed, K, reshuffle_each_pass)
        self._window = None       # device copy of the queue position, advanced by the fused kernel itself
        self._noise = C.NoiseSource(seed, self.rank)
        self._compressor = C.GlobalRandKMaxNormCompressor(self._device, quantization_level, noise=self._noise)

    def _reduce_selected(self, values):
        with self._timer("reduce.norm", verbosity=2):
            max_norm = self._global_max(ops.absmax(values))
        with self._timer("reduce.compress", verbosity=2):
            levels = self._compressor.compress(max_norm, values)
        with self._timer("reduce.reduce.vector", verbosity=2):
            wire_levels, levels = levels, self._all_reduce_levels(levels)
        bits = 32 + n_bits(wire_levels)
        mb, pb = ops.packed_sizes(values.numel(), self._quantization_level)
        self.last_wire_bits = 32 + 8 * (mb + pb)
        with self._timer("reduce.decompress", verbosity=2):
            out = self._compressor.decompress(max_norm, levels, self.n_workers)
        return out, bits

    def reduce(self, grad_in, grad_out):
        with self._timer("reduce.flat_pack"):
            flat = TensorBuffer(grad_in)
        n = flat.buffer.numel()
        start, k, npass = self._queue.next_window(n)
        if self._use_fused():
            from ..parallel import engine as fused
            bits = fused.randk(self, flat, grad_out, start, k, npass)
            if bits is not None:
                return bits
        with self._timer("reduce.gather", verbosity=2):
            values = ops.randk_gather(flat.buffer, self._queue.seed, start, k, npass)
        mean_sel, bits = self._reduce_selected(values)
        with self._timer("reduce.setgrad", verbosity=2):
            if self._unselected == "zero":
                flat.buffer.zero_()
            elif self.n_workers > 1:
                ops.scale_(flat.buffer, 1.0 / self.n_workers)
            ops.randk_scatter(flat.buffer, mean_sel, self._queue.seed, start, npass)
            flat.scatter_to(grad_out)
        return bits

    def _device_window(self, start):
        """The device-resident window start for the fused kernel (None when the permutation is re-keyed every pass: the
        key is built on the host).  Created from the host queue's position of the current step; from then on the kernel
        advances it, which is what keeps a replayed CUDA graph walking through the permutation."""
        if self._queue.reshuffle:
            return None
        if self._window is None:
            import torch

            self._window = torch.tensor([start], dtype=torch.int64, device=self._device)
        return self._window

    def graph_safe(self):
        """Replayable from a CUDA graph: every per-step quantity (window start, rounding step) is derived on the device."""
        return not self._queue.reshuffle

    def _sync_queue_from_device(self):
        if self._window is not None:
            self._queue.position = int(self._window.item())      # position of the NEXT window (0 = start of a pass)

    def state_dict(self):
        self._sync_queue_from_device()
        return {"noise": self._noise.state_dict(), "queue": self._queue.state_dict()}

    def load_state_dict(self, sd):
        self._noise.load_state_dict(sd["noise"])
        self._queue.load_state_dict(sd["queue"])
        if self._window is not None:
            self._window.fill_(self._queue.position)


class GlobalRandKMaxNormTwoScaleReducer(GlobalRandKMaxNormReducer):
    """GRandK-MN-TS: the two-scale codec on the K shared coordinates (reducer.py:1534-1633)."""

    def __init__(self, device, timer=None, seed=0, K=10000, lower_quantization_level=6,
                 higher_quantization_level=10, unselected="local", reshuffle_each_pass=False, **kw):
        super().__init__(device, timer, seed=seed, K=K, quantization_level=lower_quantization_level,
                         unselected=unselected, reshuffle_each_pass=reshuffle_each_pass, **kw)
        self._lower_quantization_level = lower_quantization_level
        self._higher_quantization_level = higher_quantization_level
        self._ts = QSGDMaxNormTwoScaleReducer(device, self._timer, lower_quantization_level,
                                              higher_quantization_level, seed=seed, backend="dist",
                                              group=self._group)
        self._ts._noise = self._noise
        self._ts._compressor._noise = self._noise

    def _reduce_selected(self, values):
        out, bits = self._ts._two_scale(values)
        self.last_wire_bits = self._ts.last_wire_bits
        return out, bits
