"""Cross-worker metric averaging (reference: metrics.py:5-40)."""
from __future__ import annotations

import torch
import torch.distributed as dist


class AverageMeter:
    """Running mean of scalar metrics, averaged over workers by ``reduce()``.

    Default: a true running mean accumulated in fp32 and reduced with ONE all-reduce
    of ``1 + n_keys`` floats.  ``reference_compat=True`` reproduces the reference's
    behaviour instead (metrics.py:18-22,33-38): ``add`` keeps only the latest value,
    and the cross-worker mean is taken in fp16 with one all-reduce per key.

    Values may be python floats or 0-dim tensors; tensors stay on the device until
    ``values()`` is read, so the training step needs no ``.item()`` sync.
    """

    def __init__(self, device=None, reference_compat=False):
        self._device = device
        self._compat = reference_compat
        self._sum = {}
        self._average = {}
        self._counter = 0
        self._dirty = False

    def add(self, metric_data):
        self._counter += 1
        for key, value in metric_data.items():
            if self._compat:
                self._sum[key] = value
            elif key in self._sum:
                self._sum[key] = self._sum[key] + value
            else:
                self._sum[key] = value if not torch.is_tensor(value) else value.clone()
        self._dirty = True

    def _local_means(self):
        out = {}
        for key, value in self._sum.items():
            v = float(value)
            out[key] = v if self._compat else v / max(self._counter, 1)
        return out

    def values(self):
        if self._dirty:
            self._average = self._local_means()
            self._dirty = False
        return self._average

    def reduce(self):
        means = self._local_means()
        self._dirty = False
        if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
            self._average = means
            return
        keys = sorted(means)
        if self._compat:
            total = torch.tensor(self._counter, dtype=torch.int32, device=self._device)
            dist.all_reduce(total)
            for key in keys:
                t = torch.tensor(means[key], dtype=torch.float16, device=self._device)
                t.mul_(self._counter)
                dist.all_reduce(t)
                means[key] = (t / total).item()
            self._average = means
            self._counter = int(total.item())
            return
        payload = torch.tensor([float(self._counter)] + [means[k] * self._counter for k in keys],
                               dtype=torch.float32, device=self._device)
        dist.all_reduce(payload)
        payload = payload.cpu()
        total = max(payload[0].item(), 1.0)
        self._average = {k: payload[i + 1].item() / total for i, k in enumerate(keys)}
        self._counter = int(payload[0].item())
