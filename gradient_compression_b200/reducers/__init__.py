"""All reducers under the reference's class names (reference: reducer.py) plus a registry."""
from .base import Reducer, TensorBuffer, n_bits
from .dense import NoneAllReducer, NoneReducer
from .multiscale import QSGDMaxNormMultiScaleReducer, QSGDMaxNormTwoScaleReducer
from .powersgd import RankKReducer
from .qsgd import (NUQSGDMaxNormBiasedMemoryReducer, NUQSGDMaxNormBiasedReducer, NUQSGDMaxNormReducer,
                   NUQSGDModReducer, QSGDBPAllReducer, QSGDBPReducer, QSGDMaxNormBiasedMemoryReducer,
                   QSGDMaxNormBiasedReducer, QSGDMaxNormReducer, QSGDReducer, QSGDWECModReducer, QSGDWECReducer,
                   TernGradModReducer, TernGradReducer)
from .randk import GlobalRandKMaxNormReducer, GlobalRandKMaxNormTwoScaleReducer
from .topk import GlobalTopKReducer, GlobalTopKReducerRatio, TopKReducer, TopKReducerRatio

REDUCERS = {cls.__name__: cls for cls in [
    NoneReducer, NoneAllReducer, QSGDReducer, QSGDWECReducer, QSGDWECModReducer, TernGradReducer,
    TernGradModReducer, QSGDMaxNormReducer, QSGDBPReducer, QSGDBPAllReducer, GlobalRandKMaxNormReducer,
    NUQSGDModReducer, NUQSGDMaxNormReducer, TopKReducer, TopKReducerRatio, GlobalTopKReducer,
    GlobalTopKReducerRatio, QSGDMaxNormBiasedReducer, QSGDMaxNormBiasedMemoryReducer, NUQSGDMaxNormBiasedReducer,
    NUQSGDMaxNormBiasedMemoryReducer, QSGDMaxNormTwoScaleReducer, GlobalRandKMaxNormTwoScaleReducer,
    QSGDMaxNormMultiScaleReducer, RankKReducer]}

# short aliases and the historic name found in the reference's older logs
ALIASES = {
    "allreduce": "NoneAllReducer", "AllReduce-SGD": "NoneAllReducer", "qsgd-mn": "QSGDMaxNormReducer",
    "qsgd-mn-ts": "QSGDMaxNormTwoScaleReducer", "qsgd-mn-ms": "QSGDMaxNormMultiScaleReducer",
    "grandk-mn": "GlobalRandKMaxNormReducer", "grandk-mn-ts": "GlobalRandKMaxNormTwoScaleReducer",
    "topk": "TopKReducer", "topk-ratio": "TopKReducerRatio", "global-topk": "GlobalTopKReducer",
    "powersgd": "RankKReducer", "MaxNormGlobalRandKReducer": "GlobalRandKMaxNormReducer",
}


def make_reducer(name, device, timer=None, config=None, **overrides):
    """Build a reducer by (reference) class name or alias from a config mapping.

    The keys follow the reference's ``config`` dict (trainer.py:44-62): ``quantization_level``,
    ``higher_quantization_level``, ``quantization_levels``, ``K``, ``compression``, ``rank``, ``seed``.
    Unlike the reference's factory (trainer.py:131-138) the two-scale Rand-K reducer receives ``K``."""
    cfg = dict(config or {})
    cfg.update(overrides)
    name = ALIASES.get(name, name)
    if name not in REDUCERS:
        raise NotImplementedError(f"Reducer method not implemented: {name}")
    cls = REDUCERS[name]
    kw = {k: cfg[k] for k in ("backend", "reference_compat") if k in cfg}
    seed = cfg.get("seed", 0)
    q = cfg.get("quantization_level", 8)
    if name in ("NoneReducer", "NoneAllReducer", "TernGradReducer", "TernGradModReducer"):
        return cls(device, timer, seed=seed, **kw)
    if name in ("GlobalRandKMaxNormReducer",):
        return cls(device, timer, seed=seed, K=cfg.get("K", 10000), quantization_level=q, **kw)
    if name in ("TopKReducer", "GlobalTopKReducer"):
        return cls(device, timer, K=cfg.get("K", 100 if name == "TopKReducer" else 10000), **kw)
    if name in ("TopKReducerRatio", "GlobalTopKReducerRatio"):
        return cls(device, timer, compression=cfg.get("compression", 1 / 100), **kw)
    if name == "QSGDMaxNormTwoScaleReducer":
        return cls(device, timer, lower_quantization_level=cfg.get("quantization_level", 6),
                   higher_quantization_level=cfg.get("higher_quantization_level", 10), seed=seed, **kw)
    if name == "GlobalRandKMaxNormTwoScaleReducer":
        return cls(device, timer, seed=seed, K=cfg.get("K", 10000),
                   lower_quantization_level=cfg.get("quantization_level", 6),
                   higher_quantization_level=cfg.get("higher_quantization_level", 10), **kw)
    if name == "QSGDMaxNormMultiScaleReducer":
        return cls(device, timer, quantization_levels=list(cfg.get("quantization_levels", [6, 10])), seed=seed, **kw)
    if name == "RankKReducer":
        return cls(device, timer, rank=cfg.get("rank", 1), seed=seed, **kw)
    return cls(device, timer, quantization_level=q, seed=seed, **kw)


__all__ = list(REDUCERS) + ["Reducer", "TensorBuffer", "n_bits", "REDUCERS", "ALIASES", "make_reducer"]
