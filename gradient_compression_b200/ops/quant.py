"""Quantisation, packing and selection ops: one Python entry per native kernel, CPU tensors go to
the C++ oracle and CUDA tensors to the sm_100a kernel of the same name (bit-identical results)."""
from __future__ import annotations

import torch

from . import _native as nat

MODE_STOCHASTIC, MODE_BIASED, MODE_NU, MODE_NU_BIASED = 0, 1, 2, 3
_scratch = {}


def mag_width(bits: int) -> int:
    w = 1
    while w < bits:
        w <<= 1
    return w


def pad128(n: int) -> int:
    return (n + 127) // 128 * 128


def sum_container_dtype(s: int, world: int):
    m = s * world
    return torch.int8 if m <= 127 else (torch.int16 if m <= 32767 else torch.int32)


def _flat32(x):
    assert x.dtype == torch.float32 and x.is_contiguous(), "expected a contiguous fp32 tensor"
    return x.view(-1)


def _absmax_scratch(device):
    key = (device.type, device.index)
    if key not in _scratch:
        nbytes = nat.cuda().gc_cuda_absmax_scratch_bytes()
        _scratch[key] = torch.zeros(nbytes, dtype=torch.uint8, device=device)
    return _scratch[key]


def absmax(x, out=None):
    """max |x| as a 1-element fp32 tensor on x's device (NaN inputs give +inf).

    Reference: ``flat_grad.buffer.abs().max()`` (reducer.py:516) -- two kernels and a temporary there.
    """
    x = _flat32(x)
    if out is None:
        out = torch.zeros(1, dtype=torch.float32, device=x.device)
    if x.numel() == 0:
        out.zero_()
        return out
    if x.is_cuda:
        with torch.cuda.device(x.device):
            nat.check(nat.cuda().gc_cuda_absmax(x.data_ptr(), x.numel(), _absmax_scratch(x.device).data_ptr(),
                                                out.data_ptr(), nat.stream_ptr()), "absmax")
    else:
        out[0] = nat.host().gc_host_absmax(x.data_ptr(), x.numel())
    return out


def _norm_tensor(norm, device):
    if torch.is_tensor(norm):
        return norm.to(device=device, dtype=torch.float32).reshape(1).contiguous()
    return torch.tensor([float(norm)], dtype=torch.float32, device=device)


def quantize_levels(x, norm, s, seed=0, stream=0, step=0, mode=MODE_STOCHASTIC, dtype=torch.int32, out=None):
    """Signed integer levels q in [-s, s] of x / norm * s (stochastic or truncating rounding).

    ``mode`` 0/1: uniform levels (compressors.py:299-316 / :562-568), 2/3: power-of-two levels with
    s = 2**b (compressors.py:520-541 / :593-603).  ``dtype`` is the container (int8/int16/int32).
    """
    x = _flat32(x)
    n = x.numel()
    if out is None:
        out = torch.empty(n, dtype=dtype, device=x.device)
    if n == 0:
        return out
    if x.is_cuda:
        nt = _norm_tensor(norm, x.device)
        with torch.cuda.device(x.device):
            nat.check(nat.cuda().gc_cuda_quantize_levels(x.data_ptr(), n, nt.data_ptr(), int(s), int(mode),
                                                         int(seed), int(stream), int(step), out.data_ptr(),
                                                         out.element_size(), nat.stream_ptr()), "quantize_levels")
    else:
        tmp = out if out.dtype == torch.int32 else torch.empty(n, dtype=torch.int32)
        nat.host().gc_host_quantize_levels(x.data_ptr(), n, float(norm), int(s), int(mode), int(seed), int(stream),
                                           int(step), tmp.data_ptr())
        if tmp is not out:
            out.copy_(tmp)
    return out


def dequantize_levels(q, norm, s, world=1, out=None):
    """fp32 ``norm / (s * world) * q`` (compressors.py:318-321 with the 1/W average folded in)."""
    q = q.contiguous().view(-1)
    n = q.numel()
    if out is None:
        out = torch.empty(n, dtype=torch.float32, device=q.device)
    if n == 0:
        return out
    if q.is_cuda:
        nt = _norm_tensor(norm, q.device)
        with torch.cuda.device(q.device):
            nat.check(nat.cuda().gc_cuda_dequantize_levels(q.data_ptr(), q.element_size(), n, nt.data_ptr(), int(s),
                                                           int(world), out.data_ptr(), nat.stream_ptr()),
                      "dequantize_levels")
    else:
        q32 = q if q.dtype == torch.int32 else q.to(torch.int32)
        nat.host().gc_host_dequantize_levels(q32.data_ptr(), n, float(norm), int(s), int(world), out.data_ptr())
    return out


def packed_sizes(n, bits):
    """(bytes of the magnitude stream, bytes of one bit plane) of the packed wire layout."""
    npad = pad128(n)
    return npad * mag_width(bits) // 8, npad // 8


def pack_levels(q, bits, mags=None, signs=None):
    """Pack int32 levels (|q| < 2**mag_width(bits)) into the wire layout -> (mags uint8, signs int32)."""
    q = q.contiguous().view(-1).to(torch.int32)
    n = q.numel()
    mb, pb = packed_sizes(n, bits)
    mags = torch.empty(mb, dtype=torch.uint8, device=q.device) if mags is None else mags
    signs = torch.empty(pb // 4, dtype=torch.int32, device=q.device) if signs is None else signs
    if q.is_cuda:
        with torch.cuda.device(q.device):
            nat.check(nat.cuda().gc_cuda_pack_levels(q.data_ptr(), n, mag_width(bits), mags.data_ptr(),
                                                     signs.data_ptr(), nat.stream_ptr()), "pack_levels")
    else:
        nat.host().gc_host_pack(q.data_ptr(), n, mag_width(bits), mags.data_ptr(), signs.data_ptr())
    return mags, signs


def unpack_levels(mags, signs, n, bits, out=None):
    out = torch.empty(n, dtype=torch.int32, device=mags.device) if out is None else out
    if mags.is_cuda:
        with torch.cuda.device(mags.device):
            nat.check(nat.cuda().gc_cuda_unpack_levels(mags.data_ptr(), signs.data_ptr(), n, mag_width(bits),
                                                       out.data_ptr(), nat.stream_ptr()), "unpack_levels")
    else:
        nat.host().gc_host_unpack(mags.data_ptr(), signs.data_ptr(), n, mag_width(bits), out.data_ptr())
    return out


def qsgd_pack(x, norm, bits, seed=0, stream=0, step=0, mags=None, signs=None):
    """Fused stochastic quantise + pack: one pass over x, (b+1)/8-ish bytes out per element."""
    x = _flat32(x)
    n = x.numel()
    mb, pb = packed_sizes(n, bits)
    mags = torch.empty(mb, dtype=torch.uint8, device=x.device) if mags is None else mags
    signs = torch.empty(pb // 4, dtype=torch.int32, device=x.device) if signs is None else signs
    if x.is_cuda:
        nt = _norm_tensor(norm, x.device)
        with torch.cuda.device(x.device):
            nat.check(nat.cuda().gc_cuda_qsgd_pack(x.data_ptr(), n, nt.data_ptr(), int(bits), int(seed), int(stream),
                                                   int(step), mags.data_ptr(), signs.data_ptr(), nat.stream_ptr()),
                      "qsgd_pack")
    else:
        q = quantize_levels(x, norm, (1 << bits) - 1, seed, stream, step)
        pack_levels(q, bits, mags, signs)
    return mags, signs


def qsgd_unpack_dequant(mags, signs, n, norm, bits, world=1, out=None):
    out = torch.empty(n, dtype=torch.float32, device=mags.device) if out is None else out
    if mags.is_cuda:
        nt = _norm_tensor(norm, mags.device)
        with torch.cuda.device(mags.device):
            nat.check(nat.cuda().gc_cuda_qsgd_unpack_dequant(mags.data_ptr(), signs.data_ptr(), n, nt.data_ptr(),
                                                             int(bits), int(world), out.data_ptr(),
                                                             nat.stream_ptr()), "qsgd_unpack_dequant")
    else:
        q = unpack_levels(mags, signs, n, bits)
        dequantize_levels(q, norm, (1 << bits) - 1, world, out)
    return out


def plane_pack(bits01):
    """Pack a 0/1 uint8 vector into the ballot-word bit-plane layout (CPU oracle only)."""
    b = bits01.contiguous().view(-1).to(torch.uint8).cpu()
    n = b.numel()
    words = torch.empty(pad128(n) // 32, dtype=torch.int32)
    nat.host().gc_host_plane_pack(b.data_ptr(), n, words.data_ptr())
    return words


def plane_unpack(words, n):
    out = torch.empty(n, dtype=torch.uint8)
    nat.host().gc_host_plane_unpack(words.contiguous().cpu().data_ptr(), n, out.data_ptr())
    return out


# --------------------------------------------------------------------------------------- RandK
def randk_indices(seed, n, start, k, npass=0, device="cpu"):
    """perm(start) .. perm(start+k-1) of the keyed permutation of [0, n): the shared index set."""
    out = torch.empty(k, dtype=torch.int64)
    nat.host().gc_host_randk_indices(int(seed), int(npass), int(n), int(start), int(k), out.data_ptr())
    return out.to(device)


def randk_gather(x, seed, start, k, npass=0, want_indices=False):
    """x[perm(start+i)] for i < k, with the indices computed on the device (no index upload)."""
    x = _flat32(x)
    if not x.is_cuda:
        idx = randk_indices(seed, x.numel(), start, k, npass)
        return (x[idx], idx) if want_indices else x[idx]
    vals = torch.empty(k, dtype=torch.float32, device=x.device)
    idx = torch.empty(k, dtype=torch.int64, device=x.device) if want_indices else None
    with torch.cuda.device(x.device):
        nat.check(nat.cuda().gc_cuda_randk_gather(x.data_ptr(), x.numel(), int(seed), int(npass), int(start), int(k),
                                                  vals.data_ptr(), nat.ptr(idx), nat.stream_ptr()), "randk_gather")
    return (vals, idx) if want_indices else vals


def randk_scatter(x, vals, seed, start, npass=0, alpha=1.0):
    """x[perm(start+i)] = alpha * vals[i]."""
    x = _flat32(x)
    k = vals.numel()
    if not x.is_cuda:
        idx = randk_indices(seed, x.numel(), start, k, npass)
        x[idx] = vals * alpha
        return x
    with torch.cuda.device(x.device):
        nat.check(nat.cuda().gc_cuda_randk_scatter(x.data_ptr(), x.numel(), int(seed), int(npass), int(start), k,
                                                   vals.contiguous().data_ptr(), float(alpha), nat.stream_ptr()),
                  "randk_scatter")
    return x


def scale_(x, alpha):
    x = _flat32(x)
    if x.is_cuda:
        with torch.cuda.device(x.device):
            nat.check(nat.cuda().gc_cuda_scale(x.data_ptr(), x.numel(), float(alpha), nat.stream_ptr()), "scale")
    else:
        x.mul_(alpha)
    return x


# --------------------------------------------------------------------------------------- SGD
def sgd_step(p, g, m, lr=None, momentum=0.9, weight_decay=0.0, nesterov=True, hyper=None):
    """In-place SGD over flat fp32 arrays: d = g + wd*p; m = mu*m + d; p -= lr*(d + mu*m | m).

    One kernel for the whole model instead of per-tensor launches (reference: ``optim.SGD``,
    trainer.py:163,196).  ``hyper`` is an optional device tensor [lr, momentum, weight_decay]; passing
    it keeps the launch arguments constant so the step can live inside a CUDA graph.
    """
    p, g, m = _flat32(p), _flat32(g), _flat32(m)
    n = p.numel()
    if p.is_cuda:
        if hyper is None:
            hyper = torch.tensor([lr, momentum, weight_decay], dtype=torch.float32, device=p.device)
        with torch.cuda.device(p.device):
            nat.check(nat.cuda().gc_cuda_sgd_step(p.data_ptr(), g.data_ptr(), m.data_ptr(), n, hyper.data_ptr(),
                                                  int(bool(nesterov)), nat.stream_ptr()), "sgd_step")
        from . import conv                     # raw-pointer write: cached transposes of these weights are stale

        conv.weights_written_raw(p.data_ptr(), p.data_ptr() + 4 * n)
    else:
        if hyper is not None:
            lr, momentum, weight_decay = (float(v) for v in hyper.tolist())
        nat.host().gc_host_sgd_step(p.data_ptr(), g.data_ptr(), m.data_ptr(), n, float(lr), float(momentum),
                                    float(weight_decay), int(bool(nesterov)))
    return p
