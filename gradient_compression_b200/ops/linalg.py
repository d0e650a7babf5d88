"""Small dense helpers used by PowerSGD and Top-K (CPU oracle side; CUDA kernels are bound in
``ops.powersgd`` / ``ops.topk``)."""
from __future__ import annotations

import torch

from . import _native as nat


def gram_schmidt_(p, eps=1e-8):
    """In-place classical Gram-Schmidt on the columns of a row-major (n, r) fp32 matrix.

    Same order of operations as the reference's ``orthogonalize`` (reducer.py:1847-1855).
    """
    assert p.dim() == 2 and p.dtype == torch.float32
    if p.is_cuda or not p.is_contiguous():
        n, r = p.shape
        for i in range(r):
            col = p[:, i:i + 1]
            col /= torch.sqrt(torch.sum(col * col)) + eps
            if i + 1 < r:
                rest = p[:, i + 1:]
                rest -= torch.sum(col * rest, dim=0) * col
        return p
    nat.host().gc_host_gram_schmidt(p.data_ptr(), p.shape[0], p.shape[1], float(eps))
    return p


def topk_abs_indices(x, k):
    """Indices of the k largest |x| (ties toward the lower index), sorted ascending; CPU oracle."""
    x = x.contiguous().view(-1)
    if x.is_cuda:
        return torch.topk(x.abs(), k, sorted=False)[1]
    out = torch.empty(k, dtype=torch.int64)
    nat.host().gc_host_topk_abs(x.data_ptr(), x.numel(), int(k), out.data_ptr())
    return out
