"""Fused ops with the reference's signatures (``hydra.kernels``: hydra/kernels/__init__.py:13-38), running as
hand-written sm_100a CUDA kernels behind PyTorch-registered custom ops (``torch.ops.hydra_b200.*``).

    fused_rope(x, cos, sin)                         hydra/kernels/fused_ops.py:240-306
    fused_qk_norm(q, k, scale, temperature=1.0)     hydra/kernels/fused_ops.py:474-493
    fused_swiglu(gate, up)                          hydra/kernels/fused_ops.py:808-883
    fused_rms_norm(x, weight, eps=1e-6)             hydra/kernels/fused_ops.py:1114-1132
    set_use_triton_kernels / get_kernel_status      hydra/kernels/fused_ops.py:123-166

Same argument meaning and result shapes/dtypes as the reference.  Differences, by design: tensors must live on
a CUDA device (a CPU tensor raises instead of silently taking a PyTorch path), the ops are forward-only
(inference), and arithmetic is fp32 inside the kernels whatever the storage dtype.
"""
from __future__ import annotations

from contextlib import nullcontext
from typing import Tuple

import torch

from . import _lib

Tensor = torch.Tensor

# Flags the reference exports.  No Triton is involved here; the names are kept so callers that read them
# keep working, and they report whether the CUDA path is active.
TRITON_AVAILABLE = False
USE_TRITON_KERNELS = False
USE_FUSED_ROPE = True
USE_FUSED_QK_NORM = True
USE_FUSED_SWIGLU = True
USE_FUSED_RMS_NORM = True
# fused_qk_norm formula: "normalize" = x / max(||x||, 1e-12) (the reference's PyTorch path and what the
# attention module computes); "rsqrt" = x * rsqrt(sum x^2 + 1e-8) (the reference's device kernel).
QK_NORM_MODE = "rsqrt"

_DTYPES = {torch.float32: _lib.HB200_F32, torch.bfloat16: _lib.HB200_BF16, torch.float16: _lib.HB200_F16}


def _dtype_code(t: Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"hydra_b200 kernels support float32, bfloat16 and float16, got {t.dtype}") from None


def _require_cuda(*ts: Tensor) -> torch.device:
    dev = ts[0].device
    for t in ts:
        if not t.is_cuda:
            raise RuntimeError("hydra_b200 kernels run on CUDA tensors only (there is no CPU fallback); "
                               f"got a tensor on {t.device}")
        if t.device != dev:
            raise RuntimeError(f"hydra_b200: tensors on different devices ({dev} and {t.device})")
    return dev


def _on(dev: torch.device):
    """Context that makes `dev` the current CUDA device (kernels launch on the current device)."""
    return nullcontext() if torch.cuda.current_device() == dev.index else torch.cuda.device(dev)


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


# ----------------------------------------------------------------------------- custom ops
@torch.library.custom_op("hydra_b200::fused_rms_norm", mutates_args=())
def _rms_norm_op(x: Tensor, weight: Tensor, eps: float) -> Tensor:
    dev = _require_cuda(x, weight)
    dim = x.shape[-1]
    if weight.numel() != dim:
        raise ValueError(f"fused_rms_norm: weight has {weight.numel()} elements, last dim is {dim}")
    xc = x.contiguous()
    w = weight.contiguous()
    if w.dtype != torch.float32 and w.dtype != x.dtype:
        w = w.float()
    y = torch.empty_like(xc)
    rows = xc.numel() // dim if dim else 0
    if rows == 0:
        return y
    with _on(dev):
        _lib.check(_lib.lib().hb200_rms_norm(xc.data_ptr(), w.data_ptr(), y.data_ptr(), rows, dim, float(eps),
                                             _dtype_code(xc), _dtype_code(w), _stream(dev)), "fused_rms_norm")
    return y


@_rms_norm_op.register_fake
def _(x, weight, eps):
    return torch.empty_like(x, memory_format=torch.contiguous_format)


@torch.library.custom_op("hydra_b200::fused_rope", mutates_args=())
def _rope_op(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    dev = _require_cuda(x, cos, sin)
    if x.dim() != 4:
        raise ValueError(f"fused_rope: x must be [B, H, S, head_dim], got {tuple(x.shape)}")
    B, H, S, hd = x.shape
    if hd % 2:
        raise ValueError("fused_rope: head_dim must be even")
    if cos.dim() == 4:
        cos, sin = cos[0, 0], sin[0, 0]
    if cos.shape[0] < S or cos.shape[1] != hd // 2 or sin.shape != cos.shape:
        raise ValueError(f"fused_rope: tables {tuple(cos.shape)} do not cover S={S}, head_dim/2={hd // 2}")
    cos = cos.float().contiguous() if (cos.dtype != torch.float32 or cos.stride(1) != 1) else cos
    sin = sin.float().contiguous() if (sin.dtype != torch.float32 or sin.stride(1) != 1) else sin
    if x.stride(3) != 1 and x.numel() > 0:
        x = x.contiguous()
    y = torch.empty((B, H, S, hd), dtype=x.dtype, device=x.device)
    if y.numel() == 0:
        return y
    with _on(dev):
        _lib.check(_lib.lib().hb200_rope(x.data_ptr(), cos.data_ptr(), sin.data_ptr(), y.data_ptr(), B, H, S, hd,
                                         x.stride(0), x.stride(1), x.stride(2), cos.stride(0), _dtype_code(x),
                                         _stream(dev)), "fused_rope")
    return y


@_rope_op.register_fake
def _(x, cos, sin):
    return torch.empty(x.shape, dtype=x.dtype, device=x.device)


@torch.library.custom_op("hydra_b200::fused_qk_norm", mutates_args=())
def _qk_norm_op(q: Tensor, k: Tensor, scale: float, temperature: float, mode: int) -> Tuple[Tensor, Tensor]:
    dev = _require_cuda(q, k)
    if q.dtype != k.dtype or q.shape[-1] != k.shape[-1]:
        raise ValueError("fused_qk_norm: q and k must share dtype and head_dim")
    hd = q.shape[-1]
    qc, kc = q.contiguous(), k.contiguous()
    qo, ko = torch.empty_like(qc), torch.empty_like(kc)
    if qc.numel() + kc.numel() == 0:
        return qo, ko
    if qc.numel() == 0 or kc.numel() == 0:   # an empty tensor has a null data pointer: give the kernel a valid one
        dummy = torch.zeros(hd, dtype=q.dtype, device=q.device)
        qc = qc if qc.numel() else dummy
        kc = kc if kc.numel() else dummy
    with _on(dev):
        _lib.check(_lib.lib().hb200_qk_norm(qc.data_ptr(), kc.data_ptr(), qo.data_ptr(), ko.data_ptr(),
                                            qo.numel() // hd, ko.numel() // hd, hd, float(scale), float(temperature),
                                            int(mode), _dtype_code(qc), _stream(dev)), "fused_qk_norm")
    return qo, ko


@_qk_norm_op.register_fake
def _(q, k, scale, temperature, mode):
    return (torch.empty_like(q, memory_format=torch.contiguous_format),
            torch.empty_like(k, memory_format=torch.contiguous_format))


@torch.library.custom_op("hydra_b200::fused_swiglu", mutates_args=())
def _swiglu_op(gate: Tensor, up: Tensor) -> Tensor:
    dev = _require_cuda(gate, up)
    if gate.shape != up.shape or gate.dtype != up.dtype:
        raise ValueError("fused_swiglu: gate and up must have the same shape and dtype")
    cols = gate.shape[-1]
    out = torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)
    if gate.numel() == 0:
        return out

    def rows_view(t: Tensor):
        """(tensor, leading dimension) if t is a [rows, cols] view with one row stride, else a copy."""
        if t.stride(-1) == 1:
            t2 = t.reshape(-1, cols) if t.dim() != 2 else t
            if t2.data_ptr() == t.data_ptr() and (t2.shape[0] == 1 or t2.stride(0) >= cols):
                return t2, (t2.stride(0) if t2.shape[0] > 1 else cols)
        c = t.contiguous().view(-1, cols)
        return c, cols

    g2, ldg = rows_view(gate)
    u2, ldu = rows_view(up)
    with _on(dev):
        _lib.check(_lib.lib().hb200_swiglu(g2.data_ptr(), u2.data_ptr(), out.data_ptr(), g2.shape[0], cols, ldg, ldu,
                                           _dtype_code(gate), _stream(dev)), "fused_swiglu")
    return out


@_swiglu_op.register_fake
def _(gate, up):
    return torch.empty(gate.shape, dtype=gate.dtype, device=gate.device)


# ----------------------------------------------------------------------------- reference-signature wrappers
def fused_rope(x: Tensor, cos: Tensor, sin: Tensor) -> Tensor:
    """Rotary embedding, interleaved pairs.  x [B, n_heads, S, head_dim] (may be a strided view);
    cos/sin [1, 1, max_seq, head_dim//2] or [S, head_dim//2].  Returns a contiguous tensor of x's dtype."""
    return _rope_op(x, cos, sin)


def fused_qk_norm(q: Tensor, k: Tensor, scale: float, temperature: float = 1.0) -> Tuple[Tensor, Tensor]:
    """L2-normalise q [B,Hq,S,hd] and k [B,Hkv,S,hd] over the last dim and scale (k also by temperature)."""
    return _qk_norm_op(q, k, float(scale), float(temperature), 0 if QK_NORM_MODE == "normalize" else 1)


def fused_swiglu(gate: Tensor, up: Tensor) -> Tensor:
    """silu(gate) * up; inputs may be the two chunk views of one gate_up projection."""
    return _swiglu_op(gate, up)


def fused_rms_norm(x: Tensor, weight: Tensor, eps: float = 1e-6) -> Tensor:
    """x * rsqrt(mean(x^2, -1) + eps) * weight."""
    return _rms_norm_op(x, weight, float(eps))


def set_use_triton_kernels(enabled: bool) -> None:
    """Kept for API compatibility (hydra/kernels/fused_ops.py:123-148).  There is exactly one implementation
    here and it has no Triton or PyTorch alternative, so the switch only records the request."""
    global USE_TRITON_KERNELS
    USE_TRITON_KERNELS = bool(enabled) and TRITON_AVAILABLE


def get_kernel_status() -> dict:
    """Same keys as the reference (hydra/kernels/fused_ops.py:151-166) plus a ``backend`` entry."""
    return {
        "triton_available": TRITON_AVAILABLE,
        "triton_version": "N/A",
        "use_triton_kernels": USE_TRITON_KERNELS,
        "fused_rope": USE_FUSED_ROPE,
        "fused_qk_norm": USE_FUSED_QK_NORM,
        "fused_qk_norm_backward": False,
        "fused_swiglu": USE_FUSED_SWIGLU,
        "fused_swiglu_backward": False,
        "fused_rms_norm": USE_FUSED_RMS_NORM,
        "fused_rms_norm_backward": False,
        "liger_ce_available": False,
        "use_liger_ce": False,
        "backend": "hydra_b200 sm_100a CUDA (C ABI v%d)" % _lib.lib().hb200_version(),
    }


__all__ = [
    "fused_rope", "fused_qk_norm", "fused_swiglu", "fused_rms_norm", "set_use_triton_kernels",
    "get_kernel_status", "TRITON_AVAILABLE", "USE_TRITON_KERNELS", "USE_FUSED_ROPE", "USE_FUSED_QK_NORM",
    "USE_FUSED_SWIGLU", "USE_FUSED_RMS_NORM",
]
