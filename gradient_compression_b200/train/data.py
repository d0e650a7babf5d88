"""Datasets and loaders of the CIFAR task (reference: model_dispatcher.py:33-107).

* ``"cifar10"``: torchvision CIFAR-10 with the reference's augmentation (random crop 32 / pad 4,
  horizontal flip, normalisation by the fixed channel mean / std) behind a ``DistributedSampler``;
  persistent worker processes instead of a new pool per epoch.
* ``"synthetic"``: N(0, 1) images and uniform labels from a seeded generator, held in pinned host
  memory; batches are sliced per rank like a ``DistributedSampler`` without shuffling overhead.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

MEAN = (0.4914, 0.4822, 0.4465)
STD = (0.247, 0.243, 0.261)


def _world():
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


class SyntheticCIFAR:
    """In-memory synthetic dataset of ``size`` 3x32x32 fp32 images and labels in 0..9."""

    def __init__(self, size, seed, pin=True):
        g = torch.Generator().manual_seed(int(seed))
        self.images = torch.randn(size, 3, 32, 32, generator=g)
        self.labels = torch.randint(0, 10, (size,), generator=g)
        if pin and torch.cuda.is_available():
            self.images, self.labels = self.images.pin_memory(), self.labels.pin_memory()

    def __len__(self):
        return self.images.shape[0]

    def loader(self, batch_size, epoch=0, shuffle=True, drop_last=True):
        world, rank = _world()
        n = len(self)
        per_rank = n // world
        if shuffle:
            g = torch.Generator().manual_seed(epoch)
            order = torch.randperm(n, generator=g)[rank::world][:per_rank]
        else:
            order = torch.arange(rank, n, world)[:per_rank]
        nb = per_rank // batch_size if drop_last else (per_rank + batch_size - 1) // batch_size
        return _SyntheticLoader(self, order, batch_size, nb, contiguous=not shuffle and world == 1)


class _SyntheticLoader:
    def __init__(self, ds, order, batch_size, nb, contiguous):
        self.ds, self.order, self.bs, self.nb, self.contiguous = ds, order, batch_size, nb, contiguous

    def __len__(self):
        return self.nb

    def __iter__(self):
        for b in range(self.nb):
            idx = self.order[b * self.bs: (b + 1) * self.bs]
            if self.contiguous:
                lo = int(idx[0])
                yield self.ds.images[lo: lo + len(idx)], self.ds.labels[lo: lo + len(idx)]
            else:
                imgs, labels = self.ds.images[idx], self.ds.labels[idx]
                if self.ds.images.is_pinned():
                    imgs, labels = imgs.pin_memory(), labels.pin_memory()
                yield imgs, labels


def load_cifar10(data_path="./data"):
    import torchvision
    import torchvision.transforms as T

    train_tf = T.Compose([T.RandomCrop(32, padding=4), T.RandomHorizontalFlip(), T.ToTensor(), T.Normalize(MEAN, STD)])
    test_tf = T.Compose([T.ToTensor(), T.Normalize(MEAN, STD)])
    try:
        train = torchvision.datasets.CIFAR10(root=data_path, train=True, download=False, transform=train_tf)
        test = torchvision.datasets.CIFAR10(root=data_path, train=False, download=False, transform=test_tf)
    except RuntimeError:
        train = torchvision.datasets.CIFAR10(root=data_path, train=True, download=True, transform=train_tf)
        test = torchvision.datasets.CIFAR10(root=data_path, train=False, download=True, transform=test_tf)
    return train, test


class TorchvisionLoaders:
    """DistributedSampler + DataLoader pair with workers kept alive across epochs."""

    def __init__(self, dataset, shuffle):
        from torch.utils.data import DistributedSampler

        world, rank = _world()
        self.dataset = dataset
        self.sampler = DistributedSampler(dataset, num_replicas=world, rank=rank, shuffle=shuffle)
        self._loader, self._bs = None, None

    def loader(self, batch_size, epoch=0):
        from torch.utils.data import DataLoader

        world, _ = _world()
        self.sampler.set_epoch(epoch)
        if self._loader is None or self._bs != batch_size:
            self._loader = DataLoader(self.dataset, batch_size=batch_size, sampler=self.sampler, pin_memory=True,
                                      drop_last=True, num_workers=max(world, 2), persistent_workers=True)
            self._bs = batch_size
        return self._loader


class DevicePrefetcher:
    """Iterates over (images, labels) host batches and yields device batches, with the host-to-device copy of the next
    ``depth`` batches already in flight on a side stream while the caller computes on the current one (pinned host
    memory makes the copies asynchronous).  ``convert`` maps the copied pair to what the model wants (for example
    channels-last images); it runs on the side stream too.  The reference copies every batch in line with
    ``.to(device)`` inside its loader generator (model_dispatcher.py:80-84)."""

    def __init__(self, batches, device, convert=None, depth=2):
        self._it = iter(batches)
        self._device = torch.device(device)
        self._convert = convert
        self._depth = max(1, int(depth))
        self._stream = torch.cuda.Stream(self._device) if self._device.type == "cuda" else None
        self._queue = []

    def _issue(self):
        try:
            imgs, labels = next(self._it)
        except StopIteration:
            return False
        if self._stream is None:
            out = (imgs.to(self._device), labels.to(self._device))
            self._queue.append((self._convert(*out) if self._convert else out, None))
            return True
        with torch.cuda.stream(self._stream):
            out = (imgs.to(self._device, non_blocking=True), labels.to(self._device, non_blocking=True))
            if self._convert:
                out = self._convert(*out)
            ev = torch.cuda.Event()
            ev.record(self._stream)
        self._queue.append((out, ev))
        return True

    def __iter__(self):
        while len(self._queue) < self._depth and self._issue():
            pass
        while self._queue:
            out, ev = self._queue.pop(0)
            if ev is not None:
                torch.cuda.current_stream(self._device).wait_event(ev)
                for t in out:
                    t.record_stream(torch.cuda.current_stream(self._device))
            self._issue()                       # keep the pipeline full before handing the batch out
            yield out


class LaggedReadback:
    """Device scalars (or short vectors) read on the host one step late: ``push(t)`` starts an asynchronous copy of ``t``
    into pinned host memory and returns the value pushed ``lag`` calls earlier (``None`` until there is one; a float for
    one element, a list of floats otherwise), so that reading the loss and metrics of every step never stalls the
    stream that is computing the next one.  ``drain()`` returns what is still pending.
    (The reference reads metrics with ``.item()`` inside the step: model_dispatcher.py:140-164.)"""

    def __init__(self, device, lag=1):
        self._device = torch.device(device)
        self._lag = max(1, int(lag))
        self._pending = []
        self._free = []

    def push(self, t):
        n = t.numel()
        if self._device.type != "cuda":
            flat = t.detach().reshape(-1).float()
            self._pending.append((float(flat[0]) if n == 1 else [float(v) for v in flat], None, None))
        else:
            buf = next((b for b in self._free if b.numel() == n), None)
            if buf is not None:
                self._free.remove(buf)
            else:
                buf = torch.empty(n, dtype=torch.float32).pin_memory()
            buf.copy_(t.detach().reshape(n).float(), non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self._device))
            self._pending.append((None, buf, ev))
        if len(self._pending) > self._lag:
            return self._take()
        return None

    def _take(self):
        val, buf, ev = self._pending.pop(0)
        if buf is None:
            return val
        ev.synchronize()
        val = float(buf[0]) if buf.numel() == 1 else [float(v) for v in buf]
        self._free.append(buf)
        return val

    def drain(self):
        out = []
        while self._pending:
            out.append(self._take())
        return out
