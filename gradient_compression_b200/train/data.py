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
