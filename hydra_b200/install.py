"""Rebind the reference's module-level names to this package (the same mechanism as the reference's own
``patch_hydra_with_liger``, hydra/kernels/liger_integration.py:150-194).

The reference binds the fused-op functions at import time in several modules
(hydra/layers/common.py:25, hydra/attention/backends/ccgqa/attention.py:13-19) and calls the attention factory
from ``HydraMoRBlock.__init__`` (hydra/model/framework/blocks.py:482-490); ``install()`` replaces every one of
those bindings, ``uninstall()`` restores them.
"""
from __future__ import annotations

import importlib
from typing import Any, Dict, List, Tuple

from . import attention as _attention
from . import kernels as _kernels

_FUSED = ("fused_rope", "fused_qk_norm", "fused_swiglu", "fused_rms_norm")
_KERNEL_MODULES = ("hydra.kernels", "hydra.kernels.fused_ops", "hydra.layers.common",
                   "hydra.attention.backends.ccgqa.attention")
_FACTORY_MODULES = ("hydra.attention", "hydra.attention.factory", "hydra.model.framework.blocks")
_REGISTRY = ("resolve_hybrid_attention_backend", "available_hybrid_attention_backends",
             "is_hybrid_attention_backend_available")
# the attention class itself is bound by name where it is constructed directly: HydraBlock / the MoD block wrapper
# (hydra/model/framework/blocks.py:20,52,383) and the backend's standard constructor (backends/ccgqa/backend.py:5-17)
_CLASS_MODULES = ("hydra.model.framework.blocks", "hydra.attention.backends.ccgqa.backend")
_BUILDER_MODULES = ("hydra.attention.backends.ccgqa", "hydra.attention.backends.ccgqa.backend")

_saved: List[Tuple[Any, str, Any]] = []


def _set(mod, name: str, value) -> None:
    _saved.append((mod, name, getattr(mod, name, None)))
    setattr(mod, name, value)


def install(kernels: bool = True, attention: bool = True) -> Dict[str, List[str]]:
    """Patch an importable ``hydra`` package in place.  Returns what was rebound, per module."""
    done: Dict[str, List[str]] = {}
    if kernels:
        for mname in _KERNEL_MODULES:
            mod = importlib.import_module(mname)
            for fn in _FUSED:
                if hasattr(mod, fn):
                    _set(mod, fn, getattr(_kernels, fn))
                    done.setdefault(mname, []).append(fn)
            if hasattr(mod, "FUSED_KERNELS_AVAILABLE"):
                _set(mod, "FUSED_KERNELS_AVAILABLE", True)
    if attention:
        for mname in _FACTORY_MODULES:
            mod = importlib.import_module(mname)
            if hasattr(mod, "build_hybrid_attention_module"):
                _set(mod, "build_hybrid_attention_module", _attention.build_hybrid_attention_module)
                done.setdefault(mname, []).append("build_hybrid_attention_module")
        mod = importlib.import_module("hydra.attention")
        for fn in _REGISTRY:
            _set(mod, fn, getattr(_attention, fn))
            done.setdefault("hydra.attention", []).append(fn)
        for mname, name, value in [(m_, "CCGQAAttention", _attention.CCGQAAttention) for m_ in _CLASS_MODULES] + \
                                  [(m_, "build_ccqa_attention", _attention.build_ccqa_attention) for m_ in _BUILDER_MODULES]:
            try:
                mod = importlib.import_module(mname)
            except ImportError:
                continue
            if hasattr(mod, name):
                _set(mod, name, value)
                done.setdefault(mname, []).append(name)
    return done


def uninstall() -> None:
    """Undo every rebinding made by install(), most recent first."""
    while _saved:
        mod, name, old = _saved.pop()
        if old is None:
            try:
                delattr(mod, name)
            except AttributeError:
                pass
        else:
            setattr(mod, name, old)


def accelerate(model, **overrides):
    """Reference ``HydraModel`` / ``HydraBaseModel`` instance -> ``HydraB200Model`` / ``HydraB200BaseModel`` holding a
    copy of its weights (the routed model is recognised by its MoR executor)."""
    from .model import HydraB200BaseModel, HydraB200Model
    routed = hasattr(model.layers[0], "mor_executor")
    return (HydraB200Model if routed else HydraB200BaseModel).from_reference(model, **overrides)
