"""Dispatch from reducers to the fused compress+collective kernels.

Each function returns ``None`` (or ``False``) when the fused path does not apply, in which case the
reducer continues on its collective (``dist``) backend; otherwise it performs the whole reduce and
returns the reference-accounting bit count.
"""
from __future__ import annotations


def _engine(reducer):
    eng = getattr(reducer, "_fused", None)
    if eng is None:
        try:
            from .engine import FusedEngine
        except ImportError:
            return None
        eng = FusedEngine.for_reducer(reducer)
        reducer._fused = eng if eng is not None else False
    return eng or None


def allreduce_mean(reducer, flat, grad_out):
    eng = _engine(reducer)
    return eng.allreduce_mean(reducer, flat, grad_out) if eng else False


def qsgd_maxnorm(reducer, flat, grad_out):
    eng = _engine(reducer)
    return eng.qsgd_maxnorm(reducer, flat, grad_out) if eng else None


def qsgd_twoscale(reducer, flat, grad_out):
    eng = _engine(reducer)
    return eng.qsgd_twoscale(reducer, flat, grad_out) if eng else None


def randk(reducer, flat, grad_out, start, k, npass):
    eng = _engine(reducer)
    return eng.randk(reducer, flat, grad_out, start, k, npass) if eng else None


def powersgd(reducer, flat, grad_out, plan, fresh):
    eng = _engine(reducer)
    return eng.powersgd(reducer, flat, grad_out, plan, fresh) if eng else None


def sparse(reducer, flat, grad_out, idx, vals):
    eng = _engine(reducer)
    return eng.sparse(reducer, flat, grad_out, idx, vals) if eng else False


def qsgd_multiscale(reducer, flat, grad_out):
    eng = _engine(reducer)
    return eng.qsgd_multiscale(reducer, flat, grad_out) if eng else None
