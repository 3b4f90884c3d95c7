"""Helpers shared by the GPU parity tests."""
from __future__ import annotations

import torch


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    a, b = a.double().cpu(), b.double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def max_abs(a: torch.Tensor, b: torch.Tensor) -> float:
    return float((a.double().cpu() - b.double().cpu()).abs().max())


def bf16_round(t: torch.Tensor) -> torch.Tensor:
    return t.to(torch.bfloat16).to(torch.float32)


def assert_close_bf16(got: torch.Tensor, ref: torch.Tensor, *, ulps: float = 2.0, what: str = "",
                      floor_frac: float = 2.0 ** -4) -> None:
    """|got - ref| <= ulps * 2^-8 * max(|ref|, floor_frac * max|ref|) elementwise (bf16 has an 8-bit mantissa;
    the floor keeps near-zero outputs of a sum of O(max) terms from demanding absolute exactness)."""
    got, ref = got.double().cpu(), ref.double().cpu()
    scale = ref.abs().max().clamp_min(1e-30)
    tol = ulps * 2.0 ** -8 * torch.maximum(ref.abs(), scale * floor_frac)
    bad = (got - ref).abs() > tol
    if bad.any():
        i = int(((got - ref).abs() / tol).argmax())
        raise AssertionError(f"{what}: {int(bad.sum())}/{bad.numel()} elements beyond {ulps} bf16 ulps; worst at flat index "
                             f"{i}: got {got.flatten()[i]:.6g} ref {ref.flatten()[i]:.6g}; rel_l2 {rel_l2(got, ref):.3e}")
