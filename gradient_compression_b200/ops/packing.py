"""Packers with the bit layouts of the reference's C++ extensions.

``varpack`` / ``varunpack``: greedy variable-width packing of non-negative ints < 256 into 32-bit
words, ``mode << 30 | payload`` with 15x2 / 7x4 / 4x7 / 3x8-bit payloads
(extensions/Extension CPU/bitpacking.cpp:19-52, Extension GPU/gpu_bitpacking.cpp:19-53).
``bytepack`` / ``byteunpack``: eight 8-bit values per int64, element j in byte 7-j
(extensions/Extension CPU BP/bytepacking.cpp:21-24).  Out-of-range inputs raise instead of looping.
"""
from __future__ import annotations

import torch

from . import _native as nat


def varpack(src):
    dev = src.device
    s = src.contiguous().view(-1).to(torch.int32)
    if s.is_cuda and hasattr(nat.cuda(), "gc_cuda_varpack"):
        return _varpack_cuda(s)
    s = s.cpu()
    n = s.numel()
    words = nat.host().gc_host_varpack(s.data_ptr(), n, None)
    if words < 0:
        raise ValueError("varpack accepts values in [0, 255] only")
    out = torch.empty(words, dtype=torch.int32)
    nat.host().gc_host_varpack(s.data_ptr(), n, out.data_ptr())
    return out.to(dev)


def varunpack(words, n=None):
    dev = words.device
    w = words.contiguous().view(-1).to(torch.int32).cpu()
    cnt = nat.host().gc_host_varunpack(w.data_ptr(), w.numel(), None)
    out = torch.empty(cnt, dtype=torch.int32)
    nat.host().gc_host_varunpack(w.data_ptr(), w.numel(), out.data_ptr())
    if n is not None:
        out = out[:n]
    return out.to(dev)


def _varpack_cuda(s):  # filled in by the CUDA packer when present
    raise NotImplementedError


def bytepack(src):
    dev = src.device
    s = src.contiguous().view(-1).to(torch.int32).cpu()
    n = s.numel()
    out = torch.empty((n + 7) // 8, dtype=torch.int64)
    nat.host().gc_host_bytepack(s.data_ptr(), n, out.data_ptr())
    return out.to(dev)


def byteunpack(words, n=None):
    dev = words.device
    w = words.contiguous().view(-1).to(torch.int64).cpu()
    out = torch.empty(w.numel() * 8, dtype=torch.int32)
    nat.host().gc_host_byteunpack(w.data_ptr(), w.numel(), out.data_ptr())
    if n is not None:
        out = out[:n]
    return out.to(dev)


def elias_encode(levels, norm_over_s):
    """Elias-omega coded QSGD stream as int64 words (format: see csrc/host_oracle.cpp)."""
    dev = levels.device
    q = levels.contiguous().view(-1).to(torch.int32).cpu()
    n = q.numel()
    nw = nat.host().gc_host_elias_encode(q.data_ptr(), n, float(norm_over_s), None, 0)
    out = torch.empty(nw, dtype=torch.int64)
    nat.host().gc_host_elias_encode(q.data_ptr(), n, float(norm_over_s), out.data_ptr(), nw)
    return out.to(dev)


def elias_decode(words):
    """-> (norm_over_s: float, levels: int32 tensor)."""
    import ctypes

    dev = words.device
    w = words.contiguous().view(-1).to(torch.int64).cpu()
    norm = ctypes.c_float(0.0)
    cnt = nat.host().gc_host_elias_decode(w.data_ptr(), w.numel(), ctypes.addressof(norm), None, 0)
    if cnt < 0:
        raise ValueError("malformed Elias stream")
    out = torch.empty(cnt, dtype=torch.int32)
    nat.host().gc_host_elias_decode(w.data_ptr(), w.numel(), ctypes.addressof(norm), out.data_ptr(), cnt)
    return norm.value, out.to(dev)


# names used by the reference's extension modules
packing = varpack
unpacking = varunpack
