"""Attention backend registry with the reference's entry points (hydra/attention/registry.py:7-49)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

_NAMES = ("ccqa", "ccgqa")


@dataclass(frozen=True, slots=True)
class HybridAttentionBackend:
    """Resolved backend; only CCGQA exists (hydra/attention/registry.py:7-14)."""

    name: str


def is_hybrid_attention_backend_available(name: str) -> bool:
    """True for 'ccqa' / 'ccgqa', any case, surrounding blanks ignored (registry.py:17-20)."""
    return str(name).strip().lower() in _NAMES


def available_hybrid_attention_backends() -> tuple[str, ...]:
    """The one canonical backend name (registry.py:23-25)."""
    return ("ccqa",)


def resolve_hybrid_attention_backend(requested: Optional[str], *, default: str = "ccqa") -> HybridAttentionBackend:
    """None or an alias of CCGQA -> HybridAttentionBackend('ccqa'); anything else raises ValueError, there is
    no silent substitution (registry.py:28-49)."""
    if requested is None or is_hybrid_attention_backend_available(requested):
        return HybridAttentionBackend("ccqa")
    raise ValueError(f"Unknown attention backend '{requested}'. Only 'ccgqa' is supported.")
