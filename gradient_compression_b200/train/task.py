"""The CIFAR task: model + data + loss + metrics (reference: model_dispatcher.py:11-187).

Same public interface as the reference's ``CIFAR`` (``parameters``, ``train_dataloader``,
``test_dataloader``, ``batch_loss``, ``batch_loss_with_gradients``, ``evaluate_predictions``,
``state_dict``, ``test``, ``len_train_loader``).  Additions: parameters, gradients and momentum live
in one ``FlatArena``; metrics are returned as device tensors (no ``.item()`` sync inside the step)
unless ``sync_metrics=True``; data may be synthetic or fully device-resident (``data="cifar10_device"`` /
``"synthetic_device"``: one augmentation kernel per batch); host->device copies are non-blocking from pinned memory.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from .. import models
from ..parallel.arena import FlatArena
from ..utils.metrics import AverageMeter
from ..utils.timer import NullTimer
from . import data as D


class CIFAR:
    def __init__(self, device, timer=None, architecture="ResNet50", seed=0, data="cifar10", data_path="./data",
                 synthetic_train_size=50000, synthetic_test_size=10000, flat_arena=True, sync_metrics=False,
                 broadcast_parameters=False, channels_last=None, reference_compat=False):
        self._device = torch.device(device)
        self._timer = timer if timer is not None else NullTimer()
        self._architecture = architecture
        self._seed = seed
        self._epoch = 0
        self._sync_metrics = sync_metrics
        self._compat = reference_compat
        self._channels_last = (self._device.type == "cuda") if channels_last is None else channels_last
        self._model = self._create_model()
        if broadcast_parameters and dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
            for t in list(self._model.parameters()) + list(self._model.buffers()):
                dist.broadcast(t.data, src=0)
        self.parameters = [p for p in self._model.parameters()]
        self.arena = FlatArena(self.parameters) if flat_arena else None
        self._data_kind = data
        self._train_set, self._test_set = self._load_dataset(data, data_path, synthetic_train_size,
                                                             synthetic_test_size)
        self.len_train_loader = None
        self.len_aux_train_loader = None
        self.len_test_loader = None
        self._criterion = torch.nn.CrossEntropyLoss().to(self._device)

    # ------------------------------------------------------------------ construction
    def _create_model(self):
        torch.random.manual_seed(self._seed)
        model = getattr(models, self._architecture)()
        model.to(self._device)
        if self._channels_last:
            model.to(memory_format=torch.channels_last)
        model.train()
        return model

    def _load_dataset(self, kind, data_path, n_train, n_test):
        if kind == "synthetic":
            return D.SyntheticCIFAR(n_train, self._seed * 2 + 1), D.SyntheticCIFAR(n_test, self._seed * 2 + 2)
        if kind in ("synthetic_device", "cifar10_device"):
            # whole dataset resident on the device; one augmentation kernel per batch, no loader workers
            from .gpu_data import DeviceCIFAR
            if kind == "synthetic_device":
                return (DeviceCIFAR.synthetic(n_train, self._device, self._seed * 2 + 1, train=True),
                        DeviceCIFAR.synthetic(n_test, self._device, self._seed * 2 + 2, train=False))
            import torchvision
            tr = torchvision.datasets.CIFAR10(root=data_path, train=True, download=False)
            te = torchvision.datasets.CIFAR10(root=data_path, train=False, download=False)
            return (DeviceCIFAR.from_torchvision(tr, self._device, self._seed, train=True),
                    DeviceCIFAR.from_torchvision(te, self._device, self._seed, train=False))
        train, test = D.load_cifar10(data_path)
        return D.TorchvisionLoaders(train, shuffle=True), D.TorchvisionLoaders(test, shuffle=True)

    @property
    def model(self):
        return self._model

    # ------------------------------------------------------------------ loaders
    def _to_device(self, imgs, labels):
        imgs = imgs.to(self._device, non_blocking=True)
        labels = labels.to(self._device, non_blocking=True)
        if self._channels_last:
            imgs = imgs.contiguous(memory_format=torch.channels_last)
        return imgs, labels

    def _convert(self, imgs, labels):
        if self._channels_last:
            imgs = imgs.contiguous(memory_format=torch.channels_last)
        return imgs, labels

    def train_dataloader(self, batch_size=32, prefetch=None):
        """Device batches of one epoch.  ``prefetch`` (default: on for host-resident data and a CUDA device): the copy of
        the next batches runs on a side stream while the current step computes (``DevicePrefetcher``)."""
        loader = self._train_set.loader(batch_size, self._epoch)
        self.len_train_loader = len(loader)
        if prefetch is None:
            prefetch = self._device.type == "cuda" and self._data_kind in ("synthetic", "cifar10")
        if prefetch:
            from .data import DevicePrefetcher

            yield from DevicePrefetcher(loader, self._device, convert=self._convert, depth=2)
        else:
            for imgs, labels in loader:
                yield self._to_device(imgs, labels)
        self._epoch += 1

    def test_dataloader(self, batch_size=32):
        loader = (self._test_set.loader(batch_size, 0, shuffle=False, drop_last=False)
                  if self._data_kind in ("synthetic", "synthetic_device", "cifar10_device") else self._test_set.loader(batch_size, 0))
        self.len_test_loader = len(loader)
        for imgs, labels in loader:
            yield self._to_device(imgs, labels)

    # ------------------------------------------------------------------ steps
    def batch_loss(self, batch):
        with torch.no_grad():
            imgs, labels = batch
            with self._timer("batch.forward", float(self._epoch)):
                prediction = self._model(imgs)
                loss = self._criterion(prediction, labels)
            with self._timer("batch.evaluate", float(self._epoch)):
                metrics = self.evaluate_predictions(prediction, labels, loss)
        return (loss.item() if self._sync_metrics else loss), metrics

    def zero_grad(self):
        if self.arena is not None:
            self.arena.zero_grad()
        else:
            self._model.zero_grad()

    def forward_loss(self, imgs, labels):
        """``(loss, logits, metrics)`` of a batch, the metrics as device scalars.  Models with a fused head (pooling, linear
        layer, cross-entropy and top-1 / top-5 in one kernel: ``ops.head``) provide all three at once; for the others the
        loss comes from the criterion and the metrics from ``evaluate_predictions``."""
        fused = getattr(self._model, "forward_loss", None)
        if fused is not None and labels.dtype == torch.int64:
            loss, prediction, m = fused(imgs, labels)
            metrics = {"cross_entropy_loss": m[0], "top1_accuracy": m[1], "top5_accuracy": m[2]}
            return loss, prediction, metrics
        prediction = self._model(imgs)
        loss = self._criterion(prediction, labels)
        return loss, prediction, None

    def batch_loss_with_gradients(self, batch):
        self.zero_grad()
        imgs, labels = batch
        with self._timer("batch.forward", float(self._epoch)):
            loss, prediction, metrics = self.forward_loss(imgs, labels)
        with self._timer("batch.backward", float(self._epoch)):
            loss.backward()
        with self._timer("batch.evaluate", float(self._epoch)):
            if metrics is None:
                metrics = self.evaluate_predictions(prediction.detach(), labels, loss.detach())
            elif self._sync_metrics:
                metrics = {k: v.item() for k, v in metrics.items()}
        grads = self.arena.grads() if self.arena is not None else [p.grad for p in self.parameters]
        return loss.detach(), grads, metrics

    def evaluate_predictions(self, pred_labels, true_labels, loss=None):
        """cross-entropy, top-1 and top-5 accuracy of a batch.  The loss computed by the forward pass
        is reused when given (the reference evaluates it a second time, model_dispatcher.py:157)."""
        with torch.no_grad():
            ce = self._criterion(pred_labels, true_labels) if loss is None else loss
            top5 = pred_labels.topk(5, 1, True, True)[1]
            hit = top5.eq(true_labels.view(-1, 1))
            bs = true_labels.shape[0]
            top1 = hit[:, 0].float().sum() / bs
            top5 = hit.float().sum() / bs
        out = {"cross_entropy_loss": ce, "top1_accuracy": top1, "top5_accuracy": top5}
        if self._sync_metrics:
            out = {k: v.item() for k, v in out.items()}
        return out

    def state_dict(self):
        return self._model.state_dict()

    def load_state_dict(self, sd):
        self._model.load_state_dict(sd)

    def test(self, batch_size=256):
        mean_metrics = AverageMeter(self._device, reference_compat=self._compat)
        self._model.eval()
        with torch.no_grad():
            for imgs, labels in self.test_dataloader(batch_size):
                prediction = self._model(imgs)
                mean_metrics.add(self.evaluate_predictions(prediction, labels))
        mean_metrics.reduce()
        self._model.train()
        return mean_metrics
