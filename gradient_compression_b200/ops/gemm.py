"""TF32 tensor-core GEMM (``csrc/gc_gemm_tc.cu``: TMA -> shared memory -> tcgen05.mma -> TMEM -> epilogue).

``gemm_tf32(a, b_nk, bias=None)`` returns ``a @ b_nk.T (+ bias)`` for row-major fp32 ``a [M, K]`` and
``b_nk [N, K]`` (optionally accumulating onto ``out`` and emitting column statistics);
``gemm_tn_tf32(a_pm, b_pn)`` returns ``a_pm.T @ b_pn`` with the contraction over the rows (weight gradients).
On CPU (and for shapes the TMA rules exclude) both are plain fp32 matmuls.
"""
from __future__ import annotations

import torch

from . import _native as nat

_err = {}


class TensorCoreTimeout(RuntimeError):
    pass


def _error_flag(device):
    key = (device.type, device.index)
    if key not in _err:
        _err[key] = torch.zeros(1, dtype=torch.int32, device=device)
    return _err[key]


def supported(a, b_nk):
    if not (a.is_cuda and b_nk.is_cuda and a.dtype == torch.float32 and b_nk.dtype == torch.float32):
        return False
    if a.dim() != 2 or b_nk.dim() != 2 or a.shape[1] != b_nk.shape[1] or a.stride(1) != 1 or b_nk.stride(1) != 1:
        return False
    return bool(nat.cuda().gc_cuda_gemm_tf32_supported(a.data_ptr(), b_nk.data_ptr(), a.shape[0], b_nk.shape[0], a.shape[1],
                                                       a.stride(0), b_nk.stride(0)))


def can_accumulate(out):
    """``accumulate=True`` needs an output the TMA store rules accept and more than 16 columns."""
    return (out.is_cuda and out.dtype == torch.float32 and out.dim() == 2 and out.stride(1) == 1 and out.shape[1] > 16
            and out.data_ptr() % 16 == 0 and out.stride(0) % 4 == 0)


_fin_scratch = {}
FIN_MAX_CHANNELS = 4096


def fin_scratch(device):
    """The per-device zero-initialised scratch (ticket + double accumulators) of the kernels that finish a reduction
    inside the producing launch; every such launch leaves it zeroed."""
    key = (device.type, device.index)
    if key not in _fin_scratch:
        n = int(nat.cuda().gc_cuda_bn_fin_scratch_bytes(FIN_MAX_CHANNELS))
        _fin_scratch[key] = torch.zeros(n, dtype=torch.uint8, device=device)
    return _fin_scratch[key]


def bn_fin_args(device, stats, running_mean, running_var, momentum, eps):
    """Argument block that makes a GEMM / convolution launch finish the batch-norm statistics of its output itself: mean and
    1 / sqrt(var + eps) land in ``stats`` ([2N] floats), the running statistics are updated in place.  The kernel's CTAs
    add their column sums into a per-device scratch with atomics and the last one to finish does the rest, so no
    separate finalize kernel runs.  Launches that use it must not overlap on the device (one stream)."""
    import ctypes

    a = nat.BnFinArgs(fin_scratch(device).data_ptr(), stats.data_ptr(), nat.ptr(running_mean), nat.ptr(running_var),
                      float(momentum), float(eps))
    return ctypes.byref(a), a


def gemm_tf32(a, b_nk, bias=None, out=None, col_partials=None, accumulate=False, bn_fin=None):
    """``col_partials`` (optional, fp32 [m_tiles, 2, N]): receives per 128-row tile the column sums and sums of
    squares of the product -- batch-norm statistics of a 1x1 convolution's output for free.
    ``accumulate=True``: ``out += a @ b_nk.T`` with the additions done by TMA reduce stores (in L2), so the old
    contents of ``out`` never travel to an SM."""
    assert not accumulate or out is not None, "accumulate needs the tensor to add to"
    if not supported(a, b_nk) or (accumulate and not can_accumulate(out)):
        assert col_partials is None and bn_fin is None, "column statistics need the tensor-core path"
        y = a @ b_nk.t()
        if bias is not None:
            y = y + bias
        if out is not None:
            if accumulate:
                out.add_(y)
            else:
                out.copy_(y)
            return out
        return y
    m, k = a.shape
    n = b_nk.shape[0]
    if out is None:
        out = torch.empty(m, n, dtype=torch.float32, device=a.device)
    assert out.stride(1) == 1
    with torch.cuda.device(a.device):
        nat.check(nat.cuda().gc_cuda_gemm_tf32(a.data_ptr(), b_nk.data_ptr(), out.data_ptr(), nat.ptr(bias), m, n, k,
                                               a.stride(0), b_nk.stride(0), out.stride(0), int(bool(accumulate)),
                                               nat.ptr(col_partials),
                                               _error_flag(a.device).data_ptr(), nat.stream_ptr(),
                                               bn_fin[0] if bn_fin is not None else None), "gemm_tf32")
    return out


def tn_supported(a_pm, b_pn, out):
    ok = all(t.is_cuda and t.dtype == torch.float32 and t.dim() == 2 and t.stride(1) == 1 for t in (a_pm, b_pn, out))
    if not ok or a_pm.shape[0] != b_pn.shape[0] or out.shape != (a_pm.shape[1], b_pn.shape[1]):
        return False
    return bool(nat.cuda().gc_cuda_gemm_tn_tf32_supported(a_pm.data_ptr(), b_pn.data_ptr(), out.data_ptr(), a_pm.shape[0],
                                                          a_pm.shape[1], b_pn.shape[1], a_pm.stride(0), b_pn.stride(0), out.stride(0)))


def gemm_tn_tf32(a_pm, b_pn, out=None, accumulate=False):
    """``out[Mo, No] (+)= a_pm[P, Mo].T @ b_pn[P, No]``: the contraction runs over the rows, which is the weight gradient
    of a 1x1 convolution (``a_pm`` = output gradient, ``b_pn`` = input, rows = positions).  On the tensor-core path both
    operands are MN-major tcgen05 operands and the contraction is split over CTAs whose partial tiles are added onto
    ``out`` by TMA reduce stores (so the summation order of the partials is not fixed)."""
    if out is None:
        assert not accumulate
        out = torch.zeros(a_pm.shape[1], b_pn.shape[1], dtype=torch.float32, device=a_pm.device)
    elif not accumulate:
        out.zero_()
    if not tn_supported(a_pm, b_pn, out):
        out.add_(a_pm.t() @ b_pn)
        return out
    with torch.cuda.device(a_pm.device):
        nat.check(nat.cuda().gc_cuda_gemm_tn_tf32(a_pm.data_ptr(), b_pn.data_ptr(), out.data_ptr(), a_pm.shape[0], a_pm.shape[1],
                                                  b_pn.shape[1], a_pm.stride(0), b_pn.stride(0), out.stride(0),
                                                  _error_flag(a_pm.device).data_ptr(), nat.stream_ptr()), "gemm_tn_tf32")
    return out


KERNELS = {"auto": 0, "tile": 1, "persistent": 2}


def configure(kernel="auto", tile_n=0):
    """Pin the kernel ("tile": one output tile per CTA; "persistent": one CTA per SM with a double-buffered TMEM
    accumulator) and the tile width (64 / 128 / 256; 0 = choose) -- for measurements and tests."""
    nat.cuda().gc_cuda_gemm_tf32_config(KERNELS[kernel], int(tile_n))


def configure_split(splits=0):
    """Contraction splits of the persistent kernel where a product allows them (no statistics, plain 2-D output):
    0 = the kernels' cost model decides, 1 = never, n = n -- for measurements and tests."""
    nat.cuda().gc_cuda_tc_split_config(int(splits))


def configure_tn(ctas_per_sm=1, min_kblocks=4):
    """Split-K policy of ``gemm_tn_tf32`` (for measurements)."""
    nat.cuda().gc_cuda_gemm_tn_config(int(ctas_per_sm), int(min_kblocks))


def m_tiles(m):
    return int(nat.cuda().gc_cuda_gemm_tf32_m_tiles(int(m)))


def check(device="cuda"):
    """Raise if any GEMM since the last check gave up on a wait (synchronises)."""
    flag = _error_flag(torch.device(device) if not isinstance(device, torch.device) else device)
    if int(flag.item()) != 0:
        flag.zero_()
        raise TensorCoreTimeout("a tcgen05 GEMM abandoned a tile after a bounded wait ran out")
