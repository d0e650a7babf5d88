"""Counter-based Philox4x32-10 streams shared by the CPU oracle and the sm_100a kernels.

``stream_id(rank, purpose)`` builds the 32-bit stream word: rounding noise uses the caller's rank
(independent across workers), index sets and PowerSGD queries use rank 0 on every worker (identical
across workers).  Replaces ``torch.bernoulli`` (reference: compressors.py:310) and ``q.normal_()``
(reducer.py:1784), whose generator state cannot be reproduced outside torch.
"""
from __future__ import annotations

import torch

from . import _native as nat

PURPOSE_ROUND, PURPOSE_ROUND_HI, PURPOSE_INDEX, PURPOSE_QINIT, PURPOSE_LEVEL0, PURPOSE_USER = 1, 2, 3, 4, 16, 64
_KIND = {"uniform": 0, "normal": 1, "u32": 2}


def stream_id(rank: int, purpose: int) -> int:
    return ((int(rank) & 0xFFFFFF) << 8) | (int(purpose) & 0xFF)


def _fill(kind, n, seed, stream, step, device, out=None, step_offset=None):
    device = torch.device(device)
    dtype = torch.int32 if kind == "u32" else torch.float32
    if out is None:
        out = torch.empty(n, dtype=dtype, device=device)
    assert out.is_contiguous() and out.numel() >= n
    seed, stream, step = int(seed) & (2 ** 64 - 1), int(stream) & 0xFFFFFFFF, int(step) & 0xFFFFFFFF
    if out.is_cuda:
        with torch.cuda.device(out.device):
            assert step_offset is None or (step_offset.is_cuda and step_offset.dtype == torch.int32)
            nat.check(nat.cuda().gc_cuda_philox_fill(_KIND[kind], seed, stream, step, nat.ptr(step_offset), n, out.data_ptr(),
                                                     nat.stream_ptr()), "philox_fill")
    else:
        if step_offset is not None:
            step = (step + int(step_offset.item())) & 0xFFFFFFFF
        fn = {"uniform": nat.host().gc_host_philox_uniform, "normal": nat.host().gc_host_philox_normal,
              "u32": nat.host().gc_host_philox_u32}[kind]
        fn(seed, stream, step, n, out.data_ptr())
    return out


def uniform(n, seed, stream, step=0, device="cpu", out=None):
    """n floats in [0, 1): element i is word i%4 of Philox block i//4, as ``(w >> 8) * 2**-24``."""
    return _fill("uniform", n, seed, stream, step, device, out)


def normal(n, seed, stream, step=0, device="cpu", out=None, step_offset=None):
    """n standard normals (Box-Muller on word pairs of each block).  ``step_offset`` (one int32 on ``out``'s device) is
    added to ``step`` when the fill runs, so a launch replayed from a CUDA graph draws a new stream each time its
    owner advances the counter."""
    return _fill("normal", n, seed, stream, step, device, out, step_offset)


def u32(n, seed, stream, step=0, device="cpu", out=None):
    """n raw 32-bit words (returned as int32 bit patterns)."""
    return _fill("u32", n, seed, stream, step, device, out)


def philox_reference_u32(n, seed, stream, step=0):
    """Pure-python Philox4x32-10 used by the tests as a third, independent implementation."""
    M0, M1, W0, W1, MASK = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85, 0xFFFFFFFF
    out = []
    for blk in range((n + 3) // 4):
        c = [blk & MASK, (blk >> 32) & MASK, step & MASK, stream & MASK]
        k0, k1 = seed & MASK, (seed >> 32) & MASK
        for _ in range(10):
            p0, p1 = M0 * c[0], M1 * c[2]
            c = [((p1 >> 32) ^ c[1] ^ k0) & MASK, p1 & MASK, ((p0 >> 32) ^ c[3] ^ k1) & MASK, p0 & MASK]
            k0, k1 = (k0 + W0) & MASK, (k1 + W1) & MASK
        out.extend(c)
    return out[:n]
