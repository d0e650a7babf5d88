"""ctypes bindings to the in-tree native libraries.

The host library is always available (built on first import when missing).  The CUDA library is
required whenever a CUDA device is visible: ops never fall back to PyTorch on a GPU box, they raise.
"""
from __future__ import annotations

import ctypes
import os

import torch

from .. import build as _build

c_void_p, c_int, c_i64, c_u64, c_u32, c_float = (ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_uint64,
                                                 ctypes.c_uint32, ctypes.c_float)

_host = None
_cuda = None


class NativeError(RuntimeError):
    pass


class BnFinArgs(ctypes.Structure):
    """Host-side argument block of the GEMM / convolution kernels that finish batch-norm statistics themselves
    (``BnFinHost`` in ``csrc/gc_tc.cuh``)."""

    _fields_ = [("scratch", ctypes.c_void_p), ("stats", ctypes.c_void_p), ("running_mean", ctypes.c_void_p),
                ("running_var", ctypes.c_void_p), ("momentum", ctypes.c_float), ("eps", ctypes.c_float)]


def _declare(lib, name, restype, argtypes):
    fn = getattr(lib, name)
    fn.restype = restype
    fn.argtypes = argtypes
    return fn


def host():
    global _host
    if _host is None:
        path = _build.host_lib_path()
        override = os.environ.get("GCB200_HOST_LIB")           # e.g. the sanitizer build (build.py --sanitize)
        if override:
            path = override
        elif not os.path.exists(path) or os.environ.get("GCB200_REBUILD"):
            path = _build.build_host()
        else:
            try:
                path = _build.build_host()  # no-op when the stamp matches the sources
            except Exception:
                pass
        lib = ctypes.CDLL(path)
        P = c_void_p
        _declare(lib, "gc_host_abi_version", c_int, [])
        _declare(lib, "gc_host_philox_u32", None, [c_u64, c_u32, c_u32, c_i64, P])
        _declare(lib, "gc_host_philox_uniform", None, [c_u64, c_u32, c_u32, c_i64, P])
        _declare(lib, "gc_host_philox_normal", None, [c_u64, c_u32, c_u32, c_i64, P])
        _declare(lib, "gc_host_absmax", c_float, [P, c_i64])
        _declare(lib, "gc_host_quantize_levels", None, [P, c_i64, c_float, c_int, c_int, c_u64, c_u32, c_u32, P])
        _declare(lib, "gc_host_dequantize_levels", None, [P, c_i64, c_float, c_int, c_int, P])
        _declare(lib, "gc_host_pack", None, [P, c_i64, c_int, P, P])
        _declare(lib, "gc_host_unpack", None, [P, P, c_i64, c_int, P])
        _declare(lib, "gc_host_plane_pack", None, [P, c_i64, P])
        _declare(lib, "gc_host_plane_unpack", None, [P, c_i64, P])
        _declare(lib, "gc_host_varpack", c_i64, [P, c_i64, P])
        _declare(lib, "gc_host_varunpack", c_i64, [P, c_i64, P])
        _declare(lib, "gc_host_bytepack", None, [P, c_i64, P])
        _declare(lib, "gc_host_byteunpack", None, [P, c_i64, P])
        _declare(lib, "gc_host_randk_indices", None, [c_u64, c_u32, c_i64, c_i64, c_i64, P])
        _declare(lib, "gc_host_gram_schmidt", None, [P, c_i64, c_int, c_float])
        _declare(lib, "gc_host_topk_abs", None, [P, c_i64, c_i64, P])
        _declare(lib, "gc_host_sgd_step", None, [P, P, P, c_i64, c_float, c_float, c_float, c_int])
        _declare(lib, "gc_host_conv3x3_geom", c_int, [c_int, c_int, c_int, c_int, P])
        _declare(lib, "gc_host_conv3x3_box", c_int, [c_int, c_int, c_int, c_int, c_int, c_int, P])
        _declare(lib, "gc_host_augment", None, [P, P, c_i64, c_u64, c_u32, c_i64, c_i64, c_int, c_int, c_int, P, P, P, P])
        _declare(lib, "gc_host_elias_encode", c_i64, [P, c_i64, c_float, P, c_i64])
        _declare(lib, "gc_host_elias_decode", c_i64, [P, c_i64, P, P, c_i64])
        _host = lib
    return _host


def cuda_available():
    return torch.cuda.is_available()


def cuda():
    """The CUDA kernel library.  Raises when it cannot be loaded: there is no eager fallback."""
    global _cuda
    if _cuda is None:
        debug = os.environ.get("GCB200_DEBUG_BOUNDS") == "1"      # the build whose gather / scatter indices are checked
        path = _build.cuda_lib_path(debug)
        try:
            path = _build.build_cuda(debug_bounds=debug)  # no-op when up to date
        except Exception as exc:
            if not os.path.exists(path):
                raise NativeError(f"libgcb200_cuda.so is missing and could not be built: {exc}") from exc
        try:
            lib = ctypes.CDLL(path)
        except OSError as exc:
            raise NativeError(f"cannot load {path}: {exc}") from exc
        P = c_void_p
        _declare(lib, "gc_cuda_abi_version", c_int, [])
        _declare(lib, "gc_cuda_sm_count", c_int, [])
        _declare(lib, "gc_cuda_philox_fill", c_int, [c_int, c_u64, c_u32, c_u32, P, c_i64, P, P])
        _declare(lib, "gc_cuda_absmax_scratch_bytes", c_i64, [])
        _declare(lib, "gc_cuda_absmax", c_int, [P, c_i64, P, P, P])
        _declare(lib, "gc_cuda_quantize_levels", c_int, [P, c_i64, P, c_int, c_int, c_u64, c_u32, c_u32, P, c_int, P])
        _declare(lib, "gc_cuda_dequantize_levels", c_int, [P, c_int, c_i64, P, c_int, c_int, P, P])
        _declare(lib, "gc_cuda_qsgd_pack", c_int, [P, c_i64, P, c_int, c_u64, c_u32, c_u32, P, P, P])
        _declare(lib, "gc_cuda_qsgd_unpack_dequant", c_int, [P, P, c_i64, P, c_int, c_int, P, P])
        _declare(lib, "gc_cuda_pack_levels", c_int, [P, c_i64, c_int, P, P, P])
        _declare(lib, "gc_cuda_unpack_levels", c_int, [P, P, c_i64, c_int, P, P])
        _declare(lib, "gc_cuda_randk_gather", c_int, [P, c_i64, c_u64, c_u32, c_i64, c_i64, P, P, P])
        _declare(lib, "gc_cuda_randk_scatter", c_int, [P, c_i64, c_u64, c_u32, c_i64, c_i64, P, c_float, P])
        _declare(lib, "gc_cuda_scale", c_int, [P, c_i64, c_float, P])
        _declare(lib, "gc_cuda_sgd_step", c_int, [P, P, P, c_i64, P, c_int, P])
        _declare(lib, "gc_cuda_bn_scratch_bytes", c_i64, [c_int])
        _declare(lib, "gc_cuda_bn_supported", c_int, [c_i64, c_int])
        _declare(lib, "gc_cuda_bn_stats", c_int, [P, c_i64, c_int, P, P, P, P, c_float, c_float, P])
        _declare(lib, "gc_cuda_bn_apply", c_int, [P, c_i64, c_int, P, P, P, P, c_int, P, P])
        _declare(lib, "gc_cuda_bn_bwd_reduce", c_int, [P, P, P, c_i64, c_int, P, P, P, c_int, P, P, P, P])
        _declare(lib, "gc_cuda_bn_bwd_fused_limit", None, [c_i64])
        _declare(lib, "gc_cuda_bn_bwd_apply", c_int, [P, P, P, c_i64, c_int, P, P, P, P, c_int, P, P, P])
        _declare(lib, "gc_cuda_bn_bwd_reduce_interleave", None, [c_int])
        _declare(lib, "gc_cuda_bn_small_supported", c_int, [c_i64, c_int])
        _declare(lib, "gc_cuda_bn_small_forward", c_int, [P, c_i64, c_int, P, c_int, P, P, P, c_int, P, P, c_float, c_float, P, P, P])
        _declare(lib, "gc_cuda_bn_small_backward", c_int, [P, P, P, c_i64, c_int, P, P, P, c_int, P, P, P, P])
        _declare(lib, "gc_cuda_bn_pool_supported", c_int, [c_int] * 4)
        _declare(lib, "gc_cuda_bn_apply_pool", c_int, [P, c_int, c_int, c_int, c_int, P, P, P, c_int, P, P])
        _declare(lib, "gc_cuda_bn_bwd_reduce_pool", c_int, [P, P, c_int, c_int, c_int, c_int, P, P, P, c_int, P, P, P])
        _declare(lib, "gc_cuda_bn_bwd_apply_pool", c_int, [P, P, c_int, c_int, c_int, c_int, P, P, P, P, c_int, P, P])
        _declare(lib, "gc_cuda_head_supported", c_int, [c_int, c_int, c_int, c_int])
        _declare(lib, "gc_cuda_head_scratch_bytes", c_i64, [c_int])
        _declare(lib, "gc_cuda_head_forward", c_int, [P, c_int, c_int, c_int, P, P, c_int, P, P, P, P, P, P, P])
        _declare(lib, "gc_cuda_head_backward", c_int, [P, P, P, P, c_int, c_int, c_int, c_int, P, P, P, P])
        _declare(lib, "gc_cuda_psgd_max_rank", c_int, [])
        _declare(lib, "gc_cuda_psgd_p", c_int, [P, P, P, c_int, c_i64, P, P, P, c_int, c_i64, P])
        _declare(lib, "gc_cuda_psgd_gs", c_int, [P, P, c_int, c_float, P])
        _declare(lib, "gc_cuda_psgd_q_chunks", c_int, [c_int])
        _declare(lib, "gc_cuda_psgd_q_blocks", c_i64, [c_int, c_int])
        _declare(lib, "gc_cuda_psgd_q", c_int, [P, P, c_int, c_i64, P, P, c_i64, c_int, P])
        _declare(lib, "gc_cuda_psgd_out", c_int, [P, P, P, c_int, c_i64, P, P, P, c_int, P, c_float, P])
        _declare(lib, "gc_cuda_topk_state_bytes", c_i64, [c_int])
        _declare(lib, "gc_cuda_topk_chunk", c_int, [])
        _declare(lib, "gc_cuda_topk_select", c_int, [P, P, P, c_int, c_i64, P, P, P, P])
        _declare(lib, "gc_cuda_batched_transpose", c_int, [P, c_int, c_i64, P])
        _declare(lib, "gc_cuda_gemm_tf32_supported", c_int, [P, P, c_int, c_int, c_int, c_i64, c_i64])
        _declare(lib, "gc_cuda_gemm_tf32", c_int, [P, P, P, P, c_int, c_int, c_int, c_i64, c_i64, c_i64, c_int, P, P, P, P])
        _declare(lib, "gc_cuda_bn_fin_scratch_bytes", c_i64, [c_int])
        _declare(lib, "gc_cuda_gemm_tf32_m_tiles", c_int, [c_int])
        _declare(lib, "gc_cuda_gemm_tn_config", None, [c_int, c_int])
        _declare(lib, "gc_cuda_gemm_tn_tf32_supported", c_int, [P, P, P, c_int, c_int, c_int, c_i64, c_i64, c_i64])
        _declare(lib, "gc_cuda_gemm_tn_tf32", c_int, [P, P, P, c_int, c_int, c_int, c_i64, c_i64, c_i64, P, P])
        _declare(lib, "gc_cuda_gemm_tf32_config", None, [c_int, c_int])
        _declare(lib, "gc_cuda_tc_tma_mode", None, [c_int])
        _declare(lib, "gc_cuda_conv_fwd_supported", c_int, [c_int] * 8)
        _declare(lib, "gc_cuda_conv_fwd_splits", c_int, [c_int] * 8)
        _declare(lib, "gc_cuda_conv_wgrad_two_taps", None, [c_int])
        _declare(lib, "gc_cuda_conv_dgrad_supported", c_int, [c_int] * 7)
        _declare(lib, "gc_cuda_conv_dgrad", c_int, [P, P, P, c_int, c_int, c_int, c_int, c_int, c_int, c_int, c_int, P, P])
        _declare(lib, "gc_cuda_gemm_tf32_splits", c_int, [c_int] * 3)
        _declare(lib, "gc_cuda_tc_split_config", None, [c_int])
        _declare(lib, "gc_cuda_conv_fwd", c_int, [P, P, P, P] + [c_int] * 9 + [P, P, P, P])
        _declare(lib, "gc_cuda_conv_dgrad_s2_supported", c_int, [c_int] * 7)
        _declare(lib, "gc_cuda_conv_dgrad_s2", c_int, [P, P, P] + [c_int] * 7 + [P, P])
        _declare(lib, "gc_cuda_conv_wgrad_supported", c_int, [c_int] * 8)
        _declare(lib, "gc_cuda_conv_wgrad", c_int, [P, P, P] + [c_int] * 8 + [P, P])
        _declare(lib, "gc_cuda_im2col_small", c_int, [P, P] + [c_int] * 7 + [P, P, c_int, P])
        _declare(lib, "gc_cuda_bn_finalize_partials", c_int, [P, c_int, c_i64, c_int, P, P, P, c_float, c_float, P])
        _declare(lib, "gc_cuda_varpack_workspace_bytes", c_i64, [c_i64])
        _declare(lib, "gc_cuda_varpack_plan", c_int, [P, c_i64, P, P, P, P])
        _declare(lib, "gc_cuda_varpack_emit", c_int, [P, c_i64, P, P, P])
        _declare(lib, "gc_cuda_bytepack", c_int, [P, c_i64, P, P])
        _declare(lib, "gc_cuda_byteunpack", c_int, [P, c_i64, P, P])
        _declare(lib, "gc_cuda_varunpack_counts", c_int, [P, c_i64, P, P])
        _declare(lib, "gc_cuda_varunpack_emit", c_int, [P, c_i64, P, P, P])
        _declare(lib, "gc_cuda_augment", c_int, [P, P, c_i64, c_u64, c_u32, c_i64, c_i64, c_int, c_int, c_int, P, P, P, P, P])
        PP = ctypes.POINTER(c_void_p)
        _declare(lib, "gc_comm_header_bytes", c_i64, [])
        _declare(lib, "gc_fused_small_grid_plain_launch", None, [c_int])
        _declare(lib, "gc_comm_max_world", c_int, [])
        _declare(lib, "gc_comm_required_bytes", c_i64, [c_i64])
        _declare(lib, "gc_comm_oneshot_bytes", c_i64, [c_i64])
        _declare(lib, "gc_comm_create", c_int, [c_int, c_int, c_i64, PP])
        _declare(lib, "gc_comm_ipc_handle", c_int, [P, P])
        _declare(lib, "gc_comm_open_peers", c_int, [P, P])
        _declare(lib, "gc_comm_set_peer", c_int, [P, c_int, P])
        _declare(lib, "gc_comm_arena_ptr", c_void_p, [P])
        _declare(lib, "gc_comm_arena_bytes", c_i64, [P])
        _declare(lib, "gc_comm_set_step_from_device", None, [P, c_int])
        _declare(lib, "gc_comm_status", c_int, [P, P, P])
        _declare(lib, "gc_comm_status_async", c_int, [P, P, P])
        _declare(lib, "gc_comm_clear_status", c_int, [P, P])
        _declare(lib, "gc_comm_debug_bounds", c_int, [])
        _declare(lib, "gc_comm_destroy", c_int, [P])
        _declare(lib, "gc_fused_qsgd", c_int, [PP, c_int, PP, PP, c_i64, c_int, c_u64, c_u32, c_int, c_int, P])
        _declare(lib, "gc_fused_twoscale", c_int, [PP, c_int, PP, PP, c_i64, c_int, c_int, c_u64, c_u32, c_int,
                                                   c_int, P])
        _declare(lib, "gc_fused_multiscale", c_int, [PP, c_int, PP, PP, c_i64, P, c_int, c_u64, c_u32, c_int, c_int, P])
        _declare(lib, "gc_fused_allreduce", c_int, [PP, c_int, PP, PP, c_i64, c_int, c_int, P])
        _declare(lib, "gc_fused_small_sum", c_int, [PP, c_int, PP, PP, c_i64, c_float, c_int, c_int, P])
        _declare(lib, "gc_fused_randk", c_int, [PP, c_int, PP, PP, c_i64, c_u64, c_u32, c_i64, c_i64, c_int, c_int,
                                                c_int, c_u32, P, c_int, c_int, P])
        _declare(lib, "gc_fused_sparse", c_int, [PP, c_int, PP, PP, PP, c_i64, c_i64, c_float, c_int, c_int, P])
        _cuda = lib
    return _cuda


_launches = 0


def count_launch(n=1):
    """Bookkeeping of how many of this library's kernels were launched (read by the benchmark)."""
    global _launches
    _launches += n


def launches():
    return _launches


def check(err, what):
    if err != 0:
        raise NativeError(f"{what}: CUDA error {err}")
    count_launch()


def stream_ptr():
    return torch.cuda.current_stream().cuda_stream


def ptr(t):
    return t.data_ptr() if t is not None else None
