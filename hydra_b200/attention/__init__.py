"""Attention entry points with the reference's names (hydra/attention/__init__.py:10-26)."""
from .registry import (
    HybridAttentionBackend,
    available_hybrid_attention_backends,
    is_hybrid_attention_backend_available,
    resolve_hybrid_attention_backend,
)
from .ccgqa import CCGQAAttention
from .factory import build_hybrid_attention_module


def build_ccqa_attention(**kwargs) -> CCGQAAttention:
    """Standard constructor of the CCQA backend (hydra/attention/backends/ccgqa/backend.py:8-17): ``CCGQAAttention(**kwargs)``."""
    return CCGQAAttention(**kwargs)


__all__ = [
    "build_ccqa_attention",
    "HybridAttentionBackend",
    "available_hybrid_attention_backends",
    "is_hybrid_attention_backend_available",
    "resolve_hybrid_attention_backend",
    "CCGQAAttention",
    "build_hybrid_attention_module",
]
