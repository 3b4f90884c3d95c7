"""Attention entry points with the reference's names (hydra/attention/__init__.py:10-26)."""
from .registry import (
    HybridAttentionBackend,
    available_hybrid_attention_backends,
    is_hybrid_attention_backend_available,
    resolve_hybrid_attention_backend,
)
from .ccgqa import CCGQAAttention
from .factory import build_hybrid_attention_module

__all__ = [
    "HybridAttentionBackend",
    "available_hybrid_attention_backends",
    "is_hybrid_attention_backend_available",
    "resolve_hybrid_attention_backend",
    "CCGQAAttention",
    "build_hybrid_attention_module",
]
