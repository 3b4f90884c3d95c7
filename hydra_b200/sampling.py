"""Next-token sampling on the device (``hb200_sample_rows``): the sampler of the reference's generation helper
(diagnostics/eval_checkpoint.py:133-155: temperature, top-k, top-p, one draw) for bf16 logit rows.  The reference draws
with ``torch.multinomial``; here the draw is the inverse CDF at one uniform number per row, so a result is reproducible
from (logits, uniform)."""
from __future__ import annotations

from typing import Optional

import torch
from torch import Tensor

from . import _lib, kernels


def cross_entropy_rows(logits: Tensor, targets: Tensor, vocab: Optional[int] = None, ignore_index: int = -100) -> Tensor:
    """Per-row negative log-likelihood (``hb200_cross_entropy_rows``): logits bf16 [N, ld] on a CUDA device (row
    stride ``logits.stride(0)``, the first ``vocab`` columns count), targets int64 [N] -> fp32 [N], 0 where the target
    is ``ignore_index``.  Summed or averaged it is ``F.cross_entropy`` of the reference's evaluation helper
    (diagnostics/eval_checkpoint.py:168-193), computed in fp32 from the bf16 logits."""
    if not logits.is_cuda or targets.device != logits.device:
        raise RuntimeError("cross_entropy_rows needs CUDA tensors on one device (there is no CPU fallback)")
    if logits.dtype != torch.bfloat16 or logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("cross_entropy_rows: logits must be bf16 [N, V] with unit column stride")
    N = logits.shape[0]
    V = int(vocab) if vocab is not None else logits.shape[1]
    targets = targets.to(torch.int64).contiguous().view(-1)
    if targets.numel() != N or not 1 <= V <= logits.shape[1]:
        raise ValueError("cross_entropy_rows: one target per row, vocab within the row length")
    bad = (targets != ignore_index) & ((targets < 0) | (targets >= V))
    if bool(bad.any()):
        raise ValueError("cross_entropy_rows: a target lies outside [0, vocab)")
    out = torch.empty(N, dtype=torch.float32, device=logits.device)
    with kernels._on(logits.device):
        _lib.check(_lib.lib().hb200_cross_entropy_rows(
            logits.data_ptr(), targets.data_ptr(), N, V, logits.stride(0) if N > 1 else max(logits.stride(0), V),
            int(ignore_index), out.data_ptr(), kernels._stream(logits.device)), "cross_entropy_rows")
    return out


def sample_rows(logits: Tensor, temperature: float = 0.8, top_k: int = 50, top_p: float = 0.9,
                uniforms: Optional[Tensor] = None, generator: Optional[torch.Generator] = None,
                vocab: Optional[int] = None, out: Optional[Tensor] = None) -> Tensor:
    """logits bf16 [B, ld] on a CUDA device (row stride ``logits.stride(0)``; the first ``vocab`` columns count,
    default all) -> int64 [B] token ids.  ``uniforms`` fp32 [B] in [0, 1) are drawn from ``generator`` (a CUDA
    generator, or the device's default) when not given.  Defaults are the reference's (0.8 / 50 / 0.9);
    ``temperature <= 0`` or ``top_k == 1`` is the argmax."""
    if not logits.is_cuda:
        raise RuntimeError("sample_rows needs CUDA tensors (there is no CPU fallback)")
    if logits.dtype != torch.bfloat16 or logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("sample_rows: logits must be bf16 [B, V] with unit column stride")
    dev = logits.device
    B = logits.shape[0]
    V = int(vocab) if vocab is not None else logits.shape[1]
    if not 1 <= V <= logits.shape[1]:
        raise ValueError(f"sample_rows: vocab {V} outside the row length {logits.shape[1]}")
    greedy = not (temperature > 0.0) or top_k == 1
    if uniforms is None and not greedy:
        uniforms = torch.rand(B, dtype=torch.float32, device=dev, generator=generator)
    if uniforms is not None:
        if uniforms.device != dev or uniforms.dtype != torch.float32 or uniforms.numel() != B:
            raise ValueError("sample_rows: uniforms must be fp32 [B] on the logits' device")
        uniforms = uniforms.contiguous()
    if out is None:
        out = torch.empty(B, dtype=torch.int64, device=dev)
    elif out.device != dev or out.dtype != torch.int64 or out.numel() != B or not out.is_contiguous():
        raise ValueError("sample_rows: out must be a contiguous int64 [B] tensor on the logits' device")
    with kernels._on(dev):
        _lib.check(_lib.lib().hb200_sample_rows(
            logits.data_ptr(), B, V, logits.stride(0) if B > 1 else max(logits.stride(0), V), float(temperature),
            int(top_k), float(top_p), uniforms.data_ptr() if uniforms is not None else None, out.data_ptr(),
            kernels._stream(dev)), "sample_rows")
    return out
