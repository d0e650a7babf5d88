"""Device-resident CIFAR input pipeline (``csrc/gc_augment.cu``).

The reference builds a new ``DataLoader`` (with worker processes) every epoch and copies each batch host ->
device (trainer.py:178, model_dispatcher.py:66-85).  Here the whole uint8 dataset (50 000 x 32 x 32 x 3 = 150 MB)
is uploaded once; each step ONE kernel draws the rank's batch from a keyed permutation of the epoch, applies
random crop (padding 4) + horizontal flip + normalisation with the reference's mean / std, and writes the fp32
channels-last batch.  ``DistributedSampler`` semantics: rank r takes slots r, r + W, r + 2W, ... of the epoch's
permutation; ``drop_last`` batches.  The CPU path runs the identical C++ oracle (bit-identical batches).
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist

from ..ops import _native as nat
from .data import MEAN, STD


class DeviceCIFAR:
    def __init__(self, images_u8, labels, device, seed=0, train=True):
        """images_u8: uint8 tensor [N, 32, 32, 3] (HWC, as stored by CIFAR-10); labels: int64 [N]."""
        assert images_u8.dtype == torch.uint8 and tuple(images_u8.shape[1:]) == (32, 32, 3)
        self.device = torch.device(device)
        self.images = images_u8.contiguous().to(self.device)
        self.labels = labels.to(torch.int64).contiguous().to(self.device)
        self.n = self.images.shape[0]
        self.seed, self.train = int(seed), bool(train)
        self._mean = (ctypes.c_float * 3)(*MEAN)
        self._inv_std = (ctypes.c_float * 3)(*[1.0 / s for s in STD])
        if dist.is_available() and dist.is_initialized():
            self.world, self.rank = dist.get_world_size(), dist.get_rank()
        else:
            self.world, self.rank = 1, 0

    @classmethod
    def from_torchvision(cls, dataset, device, seed=0, train=True):
        import numpy as np
        return cls(torch.from_numpy(np.asarray(dataset.data)), torch.tensor(dataset.targets), device, seed, train)

    @classmethod
    def synthetic(cls, n, device, seed=0, train=True):
        g = torch.Generator().manual_seed(seed)
        return cls(torch.randint(0, 256, (n, 32, 32, 3), generator=g, dtype=torch.uint8),
                   torch.randint(0, 10, (n,), generator=g), device, seed, train)

    def __len__(self):
        return self.n

    def num_batches(self, batch_size):
        return (self.n // self.world) // batch_size

    def batch(self, batch_size, epoch, index, shuffle=None):
        """Batch ``index`` of ``epoch`` for this rank -> (images [B, 3, 32, 32] channels-last fp32, labels [B])."""
        shuffle = self.train if shuffle is None else shuffle
        out = torch.empty(batch_size, 32, 32, 3, dtype=torch.float32, device=self.device)
        lab = torch.empty(batch_size, dtype=torch.int64, device=self.device)
        first = (index * batch_size) * self.world + self.rank
        args = (self.images.data_ptr(), self.labels.data_ptr(), self.n, self.seed, int(epoch), first, self.world, batch_size,
                int(self.train), int(shuffle), self._mean, self._inv_std, out.data_ptr(), lab.data_ptr())
        if self.device.type == "cuda":
            with torch.cuda.device(self.device):
                nat.check(nat.cuda().gc_cuda_augment(*args, nat.stream_ptr()), "augment")
        else:
            nat.host().gc_host_augment(*args)
        return out.permute(0, 3, 1, 2), lab          # NCHW view of NHWC memory = channels-last

    def loader(self, batch_size, epoch=0, shuffle=None, drop_last=True):
        return _DeviceLoader(self, batch_size, epoch, shuffle, drop_last)


class _DeviceLoader:
    def __init__(self, ds, batch_size, epoch, shuffle, drop_last=True):
        self.ds, self.bs, self.epoch, self.shuffle = ds, batch_size, epoch, shuffle
        per_rank = ds.n // ds.world
        self.full = per_rank // batch_size
        self.tail = 0 if drop_last else per_rank - self.full * batch_size

    def __len__(self):
        return self.full + (1 if self.tail else 0)

    def __iter__(self):
        for i in range(self.full):
            yield self.ds.batch(self.bs, self.epoch, i, self.shuffle)
        if self.tail:        # the last, shorter batch starts where the full ones ended
            ds = self.ds
            out = torch.empty(self.tail, 32, 32, 3, dtype=torch.float32, device=ds.device)
            lab = torch.empty(self.tail, dtype=torch.int64, device=ds.device)
            first = (self.full * self.bs) * ds.world + ds.rank
            shuffle = ds.train if self.shuffle is None else self.shuffle
            args = (ds.images.data_ptr(), ds.labels.data_ptr(), ds.n, ds.seed, int(self.epoch), first, ds.world, self.tail,
                    int(ds.train), int(shuffle), ds._mean, ds._inv_std, out.data_ptr(), lab.data_ptr())
            if ds.device.type == "cuda":
                with torch.cuda.device(ds.device):
                    nat.check(nat.cuda().gc_cuda_augment(*args, nat.stream_ptr()), "augment")
            else:
                nat.host().gc_host_augment(*args)
            yield out.permute(0, 3, 1, 2), lab
