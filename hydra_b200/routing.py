"""Routing decisions on the device: the index arithmetic of the reference's routers in eval mode.

``mod_select``  MoDRouter.forward's selection (hydra/routing/mixture_of_depths.py:159-216, as used by
                MoDMLPWrapper._forward_hard, blocks.py:243-269): k = max(1, min(L, int(L * clamp(capacity, 1e-4, 1)))),
                the k highest scores of every sequence, returned as ascending positions (``topk`` then ``sort``).
``mor_depths``  MoRRouter.forward's depth assignment (hydra/routing/mixture_of_recursions.py:251-291): raw logits ->
                3 tanh(l / 2) -> sigmoid -> continuous depth -> round half to even -> clamp to [min_depth, R - 1].

Both go through the C ABI (``hb200_mod_topk_select``, ``hb200_mor_depths``); tensors must live on a CUDA device."""
from __future__ import annotations

import torch
from torch import Tensor

from . import _lib, kernels


def mod_k(seq_len: int, capacity: float) -> int:
    """Tokens kept per sequence (mixture_of_depths.py:179-181), evaluated in double like the reference's Python floats."""
    cap = float(min(max(capacity, 1e-4), 1.0))
    return max(1, min(int(seq_len), int(seq_len * cap)))


def mod_select(scores: Tensor, capacity: float) -> Tensor:
    """scores fp32 [B, L] on a CUDA device -> int64 [B, k] ascending positions of each row's k highest scores (among
    equal scores the lower positions are taken; NaN ranks above +inf as in ATen)."""
    if not scores.is_cuda:
        raise RuntimeError("mod_select needs a CUDA tensor (there is no CPU fallback)")
    if scores.dim() != 2:
        raise ValueError("mod_select: scores must be [batch, seq_len]")
    B, L = scores.shape
    k = mod_k(L, capacity)
    sc = scores.to(torch.float32).contiguous()
    idx = torch.empty((B, k), dtype=torch.int32, device=scores.device)
    with kernels._on(scores.device):
        _lib.check(_lib.lib().hb200_mod_topk_select(sc.data_ptr(), B, L, k, idx.data_ptr(), None, 0, None, None,
                                                    kernels._stream(scores.device)), "mod_topk_select")
    return idx.to(torch.int64)


def mor_depths(logits: Tensor, n_recursions: int, min_depth: int = 0) -> Tensor:
    """Raw depth-router logits fp32 [...] on a CUDA device -> int64 depths of the same shape."""
    if not logits.is_cuda:
        raise RuntimeError("mor_depths needs a CUDA tensor (there is no CPU fallback)")
    lg = logits.to(torch.float32).contiguous()
    out = torch.empty(lg.shape, dtype=torch.int32, device=logits.device)
    with kernels._on(logits.device):
        _lib.check(_lib.lib().hb200_mor_depths(lg.data_ptr(), out.data_ptr(), lg.numel(), int(n_recursions),
                                               int(min_depth), kernels._stream(logits.device)), "mor_depths")
    return out.to(torch.int64)
