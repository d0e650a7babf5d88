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
    if s.is_cuda:
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
    if words.is_cuda:
        return _varunpack_cuda(words.contiguous().view(-1).to(torch.int32), n)
    w = words.contiguous().view(-1).to(torch.int32).cpu()
    cnt = nat.host().gc_host_varunpack(w.data_ptr(), w.numel(), None)
    out = torch.empty(cnt, dtype=torch.int32)
    nat.host().gc_host_varunpack(w.data_ptr(), w.numel(), out.data_ptr())
    if n is not None:
        out = out[:n]
    return out.to(dev)


def _varpack_cuda(s):
    """Parallel greedy packer on the device (csrc/gc_varpack.cu); one host read-back for the word count."""
    n = s.numel()
    if n == 0:
        return torch.empty(0, dtype=torch.int32, device=s.device)
    lib = nat.cuda()
    ws = torch.empty(lib.gc_cuda_varpack_workspace_bytes(n), dtype=torch.uint8, device=s.device)
    total = torch.zeros(1, dtype=torch.int64, device=s.device)
    bad = torch.zeros(1, dtype=torch.int32, device=s.device)
    with torch.cuda.device(s.device):
        nat.check(lib.gc_cuda_varpack_plan(s.data_ptr(), n, ws.data_ptr(), total.data_ptr(), bad.data_ptr(), nat.stream_ptr()),
                  "varpack_plan")
        nat.count_launch(4)
        n_words, is_bad = int(total.item()), int(bad.item())
        if is_bad:
            raise ValueError("varpack accepts values in [0, 255] only")
        out = torch.empty(n_words, dtype=torch.int32, device=s.device)
        nat.check(lib.gc_cuda_varpack_emit(s.data_ptr(), n, ws.data_ptr(), out.data_ptr(), nat.stream_ptr()), "varpack_emit")
    return out


def _varunpack_cuda(w, n=None):
    nw = w.numel()
    if nw == 0:
        return torch.empty(0, dtype=torch.int32, device=w.device)
    lib = nat.cuda()
    counts = torch.empty(nw, dtype=torch.int64, device=w.device)
    with torch.cuda.device(w.device):
        nat.check(lib.gc_cuda_varunpack_counts(w.data_ptr(), nw, counts.data_ptr(), nat.stream_ptr()), "varunpack_counts")
        ends = torch.cumsum(counts, 0)
        offsets = ends - counts
        out = torch.empty(int(ends[-1].item()), dtype=torch.int32, device=w.device)
        nat.check(lib.gc_cuda_varunpack_emit(w.data_ptr(), nw, offsets.data_ptr(), out.data_ptr(), nat.stream_ptr()),
                  "varunpack_emit")
    return out[:n] if n is not None else out


def bytepack(src):
    dev = src.device
    if src.is_cuda:
        s = src.contiguous().view(-1).to(torch.int32)
        out = torch.empty((s.numel() + 7) // 8, dtype=torch.int64, device=dev)
        with torch.cuda.device(dev):
            nat.check(nat.cuda().gc_cuda_bytepack(s.data_ptr(), s.numel(), out.data_ptr(), nat.stream_ptr()), "bytepack")
        return out
    s = src.contiguous().view(-1).to(torch.int32).cpu()
    n = s.numel()
    out = torch.empty((n + 7) // 8, dtype=torch.int64)
    nat.host().gc_host_bytepack(s.data_ptr(), n, out.data_ptr())
    return out.to(dev)


def byteunpack(words, n=None):
    dev = words.device
    if words.is_cuda:
        w = words.contiguous().view(-1).to(torch.int64)
        out = torch.empty(w.numel() * 8, dtype=torch.int32, device=dev)
        with torch.cuda.device(dev):
            nat.check(nat.cuda().gc_cuda_byteunpack(w.data_ptr(), w.numel(), out.data_ptr(), nat.stream_ptr()), "byteunpack")
        return out[:n] if n is not None else out
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
