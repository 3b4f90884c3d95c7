"""Attention module factory with the reference's signature (hydra/attention/factory.py:28-89)."""
from __future__ import annotations

import os
from typing import Any

import torch.nn as nn

from .registry import is_hybrid_attention_backend_available

_ALLOWED = ("use_rope", "use_qk_norm", "use_convs", "use_qk_mean", "use_value_shift", "conv_kernel_size",
            "use_fused_kernel")


def build_hybrid_attention_module(requested: str, *, dim: int, n_heads: int, n_kv_heads: int, max_seq_len: int,
                                  compression_factor: int, attention_kwargs: dict[str, Any]) -> nn.Module:
    """Instantiate the CCGQA attention module.  Unknown backend names raise ValueError; keys of
    ``attention_kwargs`` outside the CCGQA options (MoD / MoR settings travel in the same dict) are dropped;
    ``HYDRA_CCQA_USE_FUSED_KERNEL`` overrides ``use_fused_kernel`` exactly as in the reference
    (factory.py:56-89)."""
    if not is_hybrid_attention_backend_available(requested):
        raise ValueError(f"Unknown attention backend '{requested}'. Only 'ccgqa' is supported.")
    from .ccgqa import CCGQAAttention

    kwargs = {k: v for k, v in attention_kwargs.items() if k in _ALLOWED}
    env = os.environ.get("HYDRA_CCQA_USE_FUSED_KERNEL", "").strip().lower()
    if env in {"1", "true", "yes", "y"}:
        kwargs["use_fused_kernel"] = True
    elif env in {"0", "false", "no", "n"}:
        kwargs["use_fused_kernel"] = False
    return CCGQAAttention(dim=dim, n_heads=n_heads, n_kv_heads=n_kv_heads, compression_factor=compression_factor,
                          max_seq_len=max_seq_len, **kwargs)
